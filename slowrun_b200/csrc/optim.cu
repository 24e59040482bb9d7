// Optimizer kernels: the element-wise / row-wise parts of the Muon step around the Newton-Schulz GEMMs, and AdamW.
// Math follows the reference's muon_step_fused / adamw_step_fused (train.py:594-639); the reference runs them as
// Inductor-generated Triton. All kernels work on a stack [n, r, c] of same-shape matrices (one launch per group).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// Momentum + Nesterov + (row_norm != 0) MuonEq-R row normalisation, one warp per row.
//   G *= gscale (1/world for SUM-reduced gradients);  M <- M + (1-mu)(G - M);  g = G + mu(M - G);  g /= max(||g_row||, 1e-7);  X = bf16(g);  sumsq[b] += sum X^2
// The limited, two-hour and unlimited tracks normalise rows (train.py:611-613); the tiny track does not
// (tiny/train.py:770-778).
__global__ void muon_pre_kernel(const float* __restrict__ G, float* __restrict__ Mom, __nv_bfloat16* __restrict__ X,
                                float* __restrict__ sumsq, long rows_total, int r, int c, float mu, float gscale,
                                int row_norm) {
  const long row = (long)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int lane = threadIdx.x & 31;
  const float* g = G + row * c;
  float* m = Mom + row * c;
  float ss = 0.f;
  for (int j = lane * 4; j < c; j += 128) {
    float4 gv = *reinterpret_cast<const float4*>(g + j);
    gv.x *= gscale; gv.y *= gscale; gv.z *= gscale; gv.w *= gscale;
    float4 mv = *reinterpret_cast<const float4*>(m + j);
    mv.x += (1.f - mu) * (gv.x - mv.x); mv.y += (1.f - mu) * (gv.y - mv.y);
    mv.z += (1.f - mu) * (gv.z - mv.z); mv.w += (1.f - mu) * (gv.w - mv.w);
    *reinterpret_cast<float4*>(m + j) = mv;
    const float a = gv.x + mu * (mv.x - gv.x), b = gv.y + mu * (mv.y - gv.y);
    const float cc = gv.z + mu * (mv.z - gv.z), d = gv.w + mu * (mv.w - gv.w);
    ss += a * a + b * b + cc * cc + d * d;
  }
  ss = warp_sum(ss);
  const float inv = row_norm ? 1.f / fmaxf(sqrtf(ss), 1e-7f) : 1.f;
  __nv_bfloat16* x = X + row * c;
  float xs = 0.f;
  for (int j = lane * 4; j < c; j += 128) {
    float4 gv = *reinterpret_cast<const float4*>(g + j);
    gv.x *= gscale; gv.y *= gscale; gv.z *= gscale; gv.w *= gscale;
    const float4 mv = *reinterpret_cast<const float4*>(m + j);
    const __nv_bfloat162 lo = __floats2bfloat162_rn((gv.x + mu * (mv.x - gv.x)) * inv, (gv.y + mu * (mv.y - gv.y)) * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn((gv.z + mu * (mv.z - gv.z)) * inv, (gv.w + mu * (mv.w - gv.w)) * inv);
    *reinterpret_cast<__nv_bfloat162*>(x + j) = lo;
    *reinterpret_cast<__nv_bfloat162*>(x + j + 2) = hi;
    const float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    xs += l.x * l.x + l.y * l.y + h.x * h.x + h.y * h.y;
  }
  xs = warp_sum(xs);
  if (lane == 0) atomicAdd(sumsq + row / r, xs);
}

// X[b] *= 1 / (1.02*sqrt(sumsq[b]) + 1e-6)
__global__ void muon_fnorm_scale_kernel(__nv_bfloat16* __restrict__ X, const float* __restrict__ sumsq, long per_mat,
                                        long total) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < total; i += (long)gridDim.x * blockDim.x * 2) {
    const float s = 1.f / (1.02f * sqrtf(sumsq[i / per_mat]) + 1e-6f);
    const float2 v = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(X + i));
    *reinterpret_cast<__nv_bfloat162*>(X + i) = __floats2bfloat162_rn(v.x * s, v.y * s);
  }
}

// vmean[b, i] = mean over the reduced dim of X^2.  row mode (r >= c): i indexes rows; col mode: i indexes columns.
__global__ void muon_rowstat_kernel(const __nv_bfloat16* __restrict__ X, float* __restrict__ vmean, long rows_total,
                                    int c) {
  const long row = (long)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* x = X + row * c;
  float ss = 0.f;
  for (int j = lane * 2; j < c; j += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + j));
    ss += v.x * v.x + v.y * v.y;
  }
  ss = warp_sum(ss);
  if (lane == 0) vmean[row] = ss / c;
}
__global__ void muon_colstat_kernel(const __nv_bfloat16* __restrict__ X, float* __restrict__ vmean, int n, int r,
                                    int c) {
  // grid: (ceil(c/ (2*blockDim)), n, row_slices); partial sums over a slice of rows, atomically added
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (col >= c) return;
  const int b = blockIdx.y;
  const int slices = gridDim.z;
  const int r0 = (int)((long)r * blockIdx.z / slices), r1 = (int)((long)r * (blockIdx.z + 1) / slices);
  const __nv_bfloat16* x = X + (long)b * r * c + col;
  float s0 = 0.f, s1 = 0.f;
  for (int i = r0; i < r1; ++i) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (long)i * c));
    s0 += v.x * v.x;
    s1 += v.y * v.y;
  }
  atomicAdd(vmean + (long)b * c + col, s0 / r);
  atomicAdd(vmean + (long)b * c + col + 1, s1 / r);
}

// One CTA per matrix: second-moment update and the per-row/column scale of the NorMuon variance reduction.
//   S <- S + (1-b2)(v - S); step = rsqrt(max(S,1e-10)); fs = step * ||X||_F / max(sqrt(sum v*n_red*step^2), 1e-10)
__global__ void muon_finalize_kernel(const float* __restrict__ vmean, float* __restrict__ S, float* __restrict__ fs,
                                     int len, int n_red, float beta2) {
  __shared__ float red[2][kWarps];
  const int b = blockIdx.x;
  const float* v = vmean + (long)b * len;
  float* s = S + (long)b * len;
  float* o = fs + (long)b * len;
  float a0 = 0.f, a1 = 0.f;
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    const float vm = v[i];
    float sv = s[i];
    sv += (1.f - beta2) * (vm - sv);
    s[i] = sv;
    const float step = rsqrtf(fmaxf(sv, 1e-10f));
    o[i] = step;
    a0 += vm * n_red;
    a1 += vm * n_red * step * step;
  }
  a0 = warp_sum(a0);
  a1 = warp_sum(a1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red[0][warp] = a0;
    red[1][warp] = a1;
  }
  __syncthreads();
  float t0 = 0.f, t1 = 0.f;
  for (int i = 0; i < kWarps; ++i) {
    t0 += red[0][i];
    t1 += red[1][i];
  }
  const float ratio = sqrtf(t0) / fmaxf(sqrtf(t1), 1e-10f);
  for (int i = threadIdx.x; i < len; i += blockDim.x) o[i] *= ratio;
}

// U = bf16(X * bf16(fs[row or col]))  -- the orthogonalised, variance-reduced update that is gathered
__global__ void muon_scale_update_kernel(const __nv_bfloat16* __restrict__ X, const float* __restrict__ fs,
                                         __nv_bfloat16* __restrict__ U, int r, int c, int row_mode, long total) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < total; i += (long)gridDim.x * blockDim.x * 2) {
    const long row = i / c;           // global row over the stack
    const int col = (int)(i - row * c);
    const long b = row / r;
    float f0, f1;
    if (row_mode) {
      f0 = f1 = bf16_round(fs[row]);
    } else {
      f0 = bf16_round(fs[b * c + col]);
      f1 = bf16_round(fs[b * c + col + 1]);
    }
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(X + i));
    *reinterpret_cast<__nv_bfloat162*>(U + i) = __floats2bfloat162_rn(v.x * f0, v.y * f1);
  }
}

// Cautious weight decay + apply:  P -= bf16(lr*u) + lrwd * P * [u*P >= 0];  shadow = bf16(P)
__global__ void muon_apply_kernel(float* __restrict__ P, const __nv_bfloat16* __restrict__ U,
                                  __nv_bfloat16* __restrict__ shadow, float lr_b, float lrwd_b, long total,
                                  const int* __restrict__ status) {
  // multi-GPU callers pass the status word: after a peer wait that gave up, the step must leave the parameters alone
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += (long)gridDim.x * blockDim.x * 4) {
    float4 p = *reinterpret_cast<float4*>(P + i);
    const float2 u0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(U + i));
    const float2 u1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(U + i + 2));
    p.x -= bf16_round(lr_b * u0.x) + ((u0.x * p.x >= 0.f) ? lrwd_b * p.x : 0.f);
    p.y -= bf16_round(lr_b * u0.y) + ((u0.y * p.y >= 0.f) ? lrwd_b * p.y : 0.f);
    p.z -= bf16_round(lr_b * u1.x) + ((u1.x * p.z >= 0.f) ? lrwd_b * p.z : 0.f);
    p.w -= bf16_round(lr_b * u1.y) + ((u1.y * p.w >= 0.f) ? lrwd_b * p.w : 0.f);
    *reinterpret_cast<float4*>(P + i) = p;
    if (shadow != nullptr) {
      *reinterpret_cast<__nv_bfloat162*>(shadow + i) = __floats2bfloat162_rn(p.x, p.y);
      *reinterpret_cast<__nv_bfloat162*>(shadow + i + 2) = __floats2bfloat162_rn(p.z, p.w);
    }
  }
}

// AdamW (decoupled decay first, bias-corrected step). P/m/v fp32 or bf16 (P_BF16: every in-place op rounds to bf16,
// which is what the reference's bf16 embedding state does); gradient fp32; optional bf16 shadow of an fp32 param.
template <bool P_BF16>
__global__ void adamw_kernel(void* __restrict__ Pv, const float* __restrict__ G, void* __restrict__ Mv,
                             void* __restrict__ Vv, __nv_bfloat16* __restrict__ shadow, long n, float lr, float wd,
                             float b1, float b2, float eps, float bias1, float bias2, float gscale) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float p, m, v;
    float g = G[i] * gscale;
    if (P_BF16) {
      p = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(Pv)[i]);
      m = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(Mv)[i]);
      v = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(Vv)[i]);
      g = bf16_round(g);
      p = bf16_round(p * (1.f - lr * wd));
      m = bf16_round(m + (1.f - b1) * (g - m));
      v = bf16_round(v + (1.f - b2) * (g * g - v));
      p = bf16_round(p - (lr / bias1) * (m / (sqrtf(v / bias2) + eps)));
      reinterpret_cast<__nv_bfloat16*>(Pv)[i] = __float2bfloat16(p);
      reinterpret_cast<__nv_bfloat16*>(Mv)[i] = __float2bfloat16(m);
      reinterpret_cast<__nv_bfloat16*>(Vv)[i] = __float2bfloat16(v);
    } else {
      p = reinterpret_cast<float*>(Pv)[i];
      m = reinterpret_cast<float*>(Mv)[i];
      v = reinterpret_cast<float*>(Vv)[i];
      p *= (1.f - lr * wd);
      m += (1.f - b1) * (g - m);
      v += (1.f - b2) * (g * g - v);
      p -= (lr / bias1) * (m / (sqrtf(v / bias2) + eps));
      reinterpret_cast<float*>(Pv)[i] = p;
      reinterpret_cast<float*>(Mv)[i] = m;
      reinterpret_cast<float*>(Vv)[i] = v;
      if (shadow != nullptr) shadow[i] = __float2bfloat16(p);
    }
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long n) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long)gridDim.x * blockDim.x * 4) {
    if (i + 3 < n) {
      const float4 v = *reinterpret_cast<const float4*>(src + i);
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(v.x, v.y);
      *reinterpret_cast<__nv_bfloat162*>(dst + i + 2) = __floats2bfloat162_rn(v.z, v.w);
    } else {
      for (long j = i; j < n; ++j) dst[j] = __float2bfloat16(src[j]);
    }
  }
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}
inline int grid_for(long n, int per_block) {
  long b = (n + per_block - 1) / per_block;
  const long cap = (long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }

}  // namespace

extern "C" int sr_muon_pre(const float* G, float* Mom, void* X, float* sumsq, int n, int r, int c, float mu,
                           float gscale, int row_norm, cudaStream_t s) {
  if (n <= 0) return 0;
  if (c % 4) return -2;
  const long rows = (long)n * r;
  cudaMemsetAsync(sumsq, 0, sizeof(float) * n, s);
  muon_pre_kernel<<<(unsigned)((rows + kWarps - 1) / kWarps), kThreads, 0, s>>>(G, Mom, reinterpret_cast<__nv_bfloat16*>(X), sumsq, rows, r, c, mu, gscale, row_norm);
  const long total = rows * c;
  muon_fnorm_scale_kernel<<<grid_for(total / 2, kThreads), kThreads, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(X), sumsq, (long)r * c, total);
  return rc();
}

// vmean/fs: fp32 scratch [n, len], len = r (row mode, r >= c) or c. S: second-moment state [n, len].
extern "C" int sr_muon_post(const void* X, float* vmean, float* S, float* fs, void* U, int n, int r, int c,
                            float beta2, cudaStream_t s) {
  if (n <= 0) return 0;
  if (c % 4) return -2;
  const int row_mode = r >= c;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(X);
  if (row_mode) {
    const long rows = (long)n * r;
    muon_rowstat_kernel<<<(unsigned)((rows + kWarps - 1) / kWarps), kThreads, 0, s>>>(x, vmean, rows, c);
  } else {
    cudaMemsetAsync(vmean, 0, sizeof(float) * (long)n * c, s);
    int slices = r / 128;
    if (slices < 1) slices = 1;
    if (slices > 32) slices = 32;
    dim3 grid((c / 2 + 127) / 128, n, slices);
    muon_colstat_kernel<<<grid, 128, 0, s>>>(x, vmean, n, r, c);
  }
  const int len = row_mode ? r : c;
  const int n_red = row_mode ? c : r;
  muon_finalize_kernel<<<n, kThreads, 0, s>>>(vmean, S, fs, len, n_red, beta2);
  const long total = (long)n * r * c;
  muon_scale_update_kernel<<<grid_for(total / 2, kThreads), kThreads, 0, s>>>(x, fs, reinterpret_cast<__nv_bfloat16*>(U), r, c, row_mode, total);
  return rc();
}

extern "C" int sr_muon_apply(float* P, const void* U, void* shadow, long total, float lr_b, float lrwd_b,
                             cudaStream_t s) {
  if (total <= 0) return 0;
  if (total % 4) return -2;
  muon_apply_kernel<<<grid_for(total / 4, kThreads), kThreads, 0, s>>>(P, reinterpret_cast<const __nv_bfloat16*>(U), reinterpret_cast<__nv_bfloat16*>(shadow), lr_b, lrwd_b, total, nullptr);
  return rc();
}

// Same, for a step whose update arrived from other ranks: does nothing when the status word is set.
extern "C" int sr_muon_apply_status(float* P, const void* U, void* shadow, long total, float lr_b, float lrwd_b,
                                    const int* status, cudaStream_t s) {
  if (total <= 0) return 0;
  if (total % 4) return -2;
  muon_apply_kernel<<<grid_for(total / 4, kThreads), kThreads, 0, s>>>(P, reinterpret_cast<const __nv_bfloat16*>(U), reinterpret_cast<__nv_bfloat16*>(shadow), lr_b, lrwd_b, total, status);
  return rc();
}

extern "C" int sr_adamw(void* P, const float* G, void* M, void* V, void* shadow, long n, int p_bf16, float lr, float wd,
                        float b1, float b2, float eps, float bias1, float bias2, float gscale, cudaStream_t s) {
  if (n <= 0) return 0;
  if (p_bf16)
    adamw_kernel<true><<<grid_for(n, kThreads), kThreads, 0, s>>>(P, G, M, V, nullptr, n, lr, wd, b1, b2, eps, bias1, bias2, gscale);
  else
    adamw_kernel<false><<<grid_for(n, kThreads), kThreads, 0, s>>>(P, G, M, V, reinterpret_cast<__nv_bfloat16*>(shadow), n, lr, wd, b1, b2, eps, bias1, bias2, gscale);
  return rc();
}

extern "C" int sr_cast_f32_to_bf16(const float* src, void* dst, long n, cudaStream_t s) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for((n + 3) / 4, kThreads), kThreads, 0, s>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return rc();
}

// ------------------------------------------------------------------------------------------------------------------
// Allocation-free variant of sr_muon_post (declared in no_alloc.h; no counterpart in the reference).
//
// sr_muon_post needs two fp32 work arrays of n*len elements (per-row or per-column mean squares and the resulting
// scale factors) that its caller has to allocate on the device. Some callers cannot do that: a step that runs inside a
// host framework whose caching allocator must not be re-entered (an allocator hook, a gradient-ready callback fired
// from another library's thread), or a process whose device memory is fully handed out up front and that has no
// cudaMalloc budget left. For them the work arrays live in the file-scope device array below, which every GPU that
// loads this library keeps resident until the process exits (2 * kNoAllocMaxElems * 4 bytes = 2 MiB).
//
// Rules of use:
//  * n * max(r, c) (row mode: n * r; column mode: n * c) must not exceed sr_muon_post_noalloc_max_elems(); larger
//    problems are refused with SR_NOALLOC_TOO_LARGE and nothing is launched.
//  * The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with that device
//    current) and remembers it; make that first call outside of any stream capture.
//  * All calls share the one array and it keeps whatever the last call left in it. What has to start at zero (the
//    column sums) is cleared on the caller's stream before use. Two calls whose kernels overlap on the GPU (different
//    streams, no ordering between them) race on the array: order them.
//  * The stream must belong to the device that is current at the call, and two threads must not race on the first
//    call for the same device (later calls only read the cached address).
//  * No cudaMalloc, cudaFree or allocating library routine is called on any path of this function.
constexpr long kNoAllocMaxElems = 1L << 18;
static __device__ __align__(256) float g_noalloc_scratch[2 * kNoAllocMaxElems];

constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

enum { SR_NOALLOC_TOO_LARGE = -8, SR_NOALLOC_NO_SYMBOL = -9, SR_NOALLOC_BAD_DEVICE = -10 };

extern "C" long sr_muon_post_noalloc_max_elems() { return kNoAllocMaxElems; }

extern "C" int sr_muon_post_noalloc(const void* X, float* S, void* U, int n, int r, int c, float beta2,
                                    cudaStream_t s) {
  if (n <= 0) return 0;
  if (c % 4) return -2;
  const int row_mode = r >= c;
  const int len = row_mode ? r : c;
  if ((long)n * len > kNoAllocMaxElems) return SR_NOALLOC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return SR_NOALLOC_BAD_DEVICE;
  if (g_noalloc_ptr[dev] == nullptr) {
    // In host code the array's name is only a stand-in; the kernels need its device address on THIS device.
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return SR_NOALLOC_NO_SYMBOL;
    g_noalloc_ptr[dev] = p;
  }
  float* vmean = g_noalloc_ptr[dev];
  float* fs = vmean + kNoAllocMaxElems;
  // Same launch sequence as the ordinary entry point, on the library's own work arrays (it clears what must start at
  // zero on the caller's stream and allocates nothing).
  return sr_muon_post(X, vmean, S, fs, U, n, r, c, beta2, s);
}
