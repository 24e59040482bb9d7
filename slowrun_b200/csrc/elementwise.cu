// Bandwidth-bound fused elementwise / row-wise kernels of the transformer block (bf16 activations, fp32 math).
// The reference leaves all of these to torch.compile (Inductor-generated Triton, train.py:1060); here each is
// one hand-written kernel with 16-byte vector accesses, one warp per row for the row reductions.
//
//   rmsnorm fwd/bwd            weight-less RMSNorm (train.py:235-236)
//   lambda_mix fwd/bwd         x = resid_l*(x + skip_w*skip) + x0_l*x0 (train.py:519-522)
//   rope_qknorm fwd/bwd        RoPE then per-head RMSNorm on q and k (train.py:242-245, 304-306)
//   gated_add fwd/bwd          v += gate[b,t,h] * ve (value residual, train.py:299-303)
//   head_scale fwd/bwd         y *= gate[b,t,h] (attention gate, train.py:308-309)
//   swiglu fwd/bwd             silu(g) * f on a fused [M, 2h] GEMM output (train.py:322-323)
//   dropout_add fwd/bwd        out = x_in + keep*(x_mid + dropout(y) - x_in) (train.py:333-344); the mask is a hash of
//                              (per-call salt, device-resident step counter, element index), so a captured CUDA graph
//                              draws a fresh mask on every replay
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(t.v[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? smem[threadIdx.x] : 0.f;
  if (warp == 0) r = warp_sum(r);
  __syncthreads();
  return r;  // valid in warp 0
}

// counter-based uniform in [0,1): one hash per element index, reproducible in backward
__device__ __forceinline__ uint32_t mix32(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return static_cast<uint32_t>((z ^ (z >> 31)) >> 32);
}
__device__ __forceinline__ bool keep_elem(uint64_t seed, uint64_t idx, float p) {
  const uint32_t h = mix32(seed * 0x100000001B3ull + idx);
  return (h >> 8) * (1.0f / 16777216.0f) >= p;
}

// ------------------------------------------------------------------ rmsnorm
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows,
                                   int D, long ldx, float eps) {
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + row * ldx;
  float ss = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
  __nv_bfloat16* yr = y + row * (long)D;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= r;
    store8(yr + c, f);
  }
}

// dx (+)= r*dy - x * r^3 * mean(dy*x)
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, long rows,
                                   int D, long ldx, float eps) {
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + row * ldx;
  const __nv_bfloat16* gr = dy + row * (long)D;
  float ss = 0.f, dot = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], g[8];
    load8(xr + c, f);
    load8(gr + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss += f[i] * f[i];
      dot += f[i] * g[i];
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss / D + eps);
  const float k = r * r * r * dot / D;
  __nv_bfloat16* dr = dx + row * (long)D;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], g[8], o[8];
    load8(xr + c, f);
    load8(gr + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = r * g[i] - k * f[i];
    if (dres != nullptr) {
      float a[8];
      load8(dres + row * (long)D + c, a);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += a[i];
    }
    store8(dr + c, o);
  }
}

// ------------------------------------------------------------------ lambda mix
// out = lr*(x + ws*skip) + l0*x0 ; scalars come from device memory (no host sync)
__global__ void lambda_mix_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                                      const __nv_bfloat16* __restrict__ skip, __nv_bfloat16* __restrict__ out,
                                      const float* __restrict__ lr_p, const float* __restrict__ l0_p,
                                      const float* __restrict__ ws_p, long n8) {
  const float lr = *lr_p, l0 = *l0_p, ws = skip ? *ws_p : 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    load8(x + i * 8, a);
    load8(x0 + i * 8, b);
    if (skip) {
      float s[8];
      load8(skip + i * 8, s);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += ws * s[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = lr * a[j] + l0 * b[j];
    store8(out + i * 8, o);
  }
}

// dx = lr*g ; dskip = lr*ws*g ; dx0 = l0*g ; dscal[0..2] += (sum g*(x+ws*skip), sum g*x0, sum g*lr*skip)
__global__ void lambda_mix_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ skip,
                                      __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dx0,
                                      __nv_bfloat16* __restrict__ dskip, const float* __restrict__ lr_p,
                                      const float* __restrict__ l0_p, const float* __restrict__ ws_p,
                                      float* __restrict__ dscal, long n8) {
  __shared__ float red[32];
  const float lr = *lr_p, l0 = *l0_p, ws = skip ? *ws_p : 0.f;
  float s_lr = 0.f, s_l0 = 0.f, s_ws = 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float gg[8], a[8], b[8], o[8];
    load8(g + i * 8, gg);
    load8(x + i * 8, a);
    load8(x0 + i * 8, b);
    if (skip) {
      float s[8];
      load8(skip + i * 8, s);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] += ws * s[j];
        s_ws += gg[j] * lr * s[j];
        o[j] = lr * ws * gg[j];
      }
      store8(dskip + i * 8, o);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s_lr += gg[j] * a[j];
      s_l0 += gg[j] * b[j];
      o[j] = lr * gg[j];
    }
    store8(dx + i * 8, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = l0 * gg[j];
    store8(dx0 + i * 8, o);
  }
  s_lr = block_sum(s_lr, red);
  s_l0 = block_sum(s_l0, red);
  s_ws = block_sum(s_ws, red);
  if (threadIdx.x == 0) {
    atomicAdd(dscal + 0, s_lr);
    atomicAdd(dscal + 1, s_l0);
    if (skip) atomicAdd(dscal + 2, s_ws);
  }
}


// ------------------------------------------------------------------ lambda mix fused with the block's first RMSNorm
// x = lr*(xp + ws*skip) + l0*x0 ; a = rmsnorm(x) (of the bf16-rounded x). One warp per row.
__global__ void mix_norm_fwd_kernel(const __nv_bfloat16* __restrict__ xp, const __nv_bfloat16* __restrict__ x0,
                                    const __nv_bfloat16* __restrict__ skip, __nv_bfloat16* __restrict__ x,
                                    __nv_bfloat16* __restrict__ a_out, const float* __restrict__ lr_p,
                                    const float* __restrict__ l0_p, const float* __restrict__ ws_p, long rows, int D,
                                    float eps) {
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float lr = *lr_p, l0 = *l0_p, ws = skip ? *ws_p : 0.f;
  const long base = row * (long)D;
  float ss = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float a[8], b[8];
    load8(xp + base + c, a);
    load8(x0 + base + c, b);
    if (skip) {
      float s[8];
      load8(skip + base + c, s);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += ws * s[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[j] = __bfloat162float(__float2bfloat16(lr * a[j] + l0 * b[j]));
      ss += a[j] * a[j];
    }
    store8(x + base + c, a);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    load8(x + base + c, f);   // this lane's own stores
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= r;
    store8(a_out + base + c, f);
  }
}

// Backward of the pair above: g = rmsnorm_bwd(x, da) + g_res (rounded to bf16, never stored), then
// dxp = lr*g ; dskip = lr*ws*g ; dx0 = l0*g ; dscal[0..2] += (sum g*(xp + ws*skip), sum g*x0, sum g*lr*skip).
__global__ void norm_bwd_mix_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ da,
                                    const __nv_bfloat16* __restrict__ g_res, const __nv_bfloat16* __restrict__ g_res2,
                                    const __nv_bfloat16* __restrict__ xp,
                                    const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ skip,
                                    __nv_bfloat16* __restrict__ dxp, __nv_bfloat16* __restrict__ dx0,
                                    __nv_bfloat16* __restrict__ dskip, const float* __restrict__ lr_p,
                                    const float* __restrict__ l0_p, const float* __restrict__ ws_p,
                                    float* __restrict__ d_lr, float* __restrict__ d_l0, float* __restrict__ d_ws,
                                    long rows, int D, float eps) {
  __shared__ float red[32];
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const float lr = *lr_p, l0 = *l0_p, ws = skip ? *ws_p : 0.f;
  float s_lr = 0.f, s_l0 = 0.f, s_ws = 0.f;
  if (row < rows) {
    const long base = row * (long)D;
    float ss = 0.f, dot = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float f[8], g[8];
      load8(x + base + c, f);
      load8(da + base + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss += f[i] * f[i];
        dot += f[i] * g[i];
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float r = rsqrtf(ss / D + eps);
    const float k = r * r * r * dot / D;
    for (int c = lane * 8; c < D; c += 256) {
      float f[8], g[8], e[8], a[8], b[8], o[8];
      load8(x + base + c, f);
      load8(da + base + c, g);
      load8(g_res + base + c, e);
      if (g_res2 != nullptr) {   // second residual gradient (the stochastic-depth bypass), added in bf16 like a separate add would
        float e2[8];
        load8(g_res2 + base + c, e2);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = __bfloat162float(__float2bfloat16(e[i] + e2[i]));
      }
      load8(xp + base + c, a);
      load8(x0 + base + c, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = __bfloat162float(__float2bfloat16(r * g[i] - k * f[i] + e[i]));
      if (skip) {
        float sk[8];
        load8(skip + base + c, sk);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[j] += ws * sk[j];
          s_ws += g[j] * lr * sk[j];
          o[j] = lr * ws * g[j];
        }
        store8(dskip + base + c, o);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s_lr += g[j] * a[j];
        s_l0 += g[j] * b[j];
        o[j] = lr * g[j];
      }
      store8(dxp + base + c, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = l0 * g[j];
      store8(dx0 + base + c, o);
    }
  }
  s_lr = block_sum(s_lr, red);
  s_l0 = block_sum(s_l0, red);
  s_ws = block_sum(s_ws, red);
  if (threadIdx.x == 0) {
    atomicAdd(d_lr, s_lr);
    atomicAdd(d_l0, s_l0);
    if (skip) atomicAdd(d_ws, s_ws);
  }
}

// ------------------------------------------------------------------ RoPE + QK-norm, head_dim = 128
// One warp per (token, head). Lane l owns elements {2l, 2l+1} of the first half and {64+2l, 64+2l+1} of the second.
// in : [tokens, ld_in] with head h at column offset h*128 ; out: [tokens, H, 128] contiguous
__global__ void rope_qknorm_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                       const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb,
                                       long tokens, int H, int T, long ld_in, float eps) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const int t = (int)(tok % T);
  const __nv_bfloat16* p = in + tok * ld_in + h * 128;
  const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 2 * lane));
  const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 64 + 2 * lane));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(cosb + (long)t * 64 + 2 * lane));
  const float2 s = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sinb + (long)t * 64 + 2 * lane));
  float2 o1, o2;
  o1.x = x1.x * c.x + x2.x * s.x;
  o1.y = x1.y * c.y + x2.y * s.y;
  o2.x = -x1.x * s.x + x2.x * c.x;
  o2.y = -x1.y * s.y + x2.y * c.y;
  float ss = o1.x * o1.x + o1.y * o1.y + o2.x * o2.x + o2.y * o2.y;
  ss = warp_sum(ss);
  const float r = rsqrtf(ss * (1.f / 128.f) + eps);
  __nv_bfloat16* q = out + wid * 128;
  *reinterpret_cast<__nv_bfloat162*>(q + 2 * lane) = __floats2bfloat162_rn(o1.x * r, o1.y * r);
  *reinterpret_cast<__nv_bfloat162*>(q + 64 + 2 * lane) = __floats2bfloat162_rn(o2.x * r, o2.y * r);
}

// g: [tokens, H, 128] gradient of the normed output; din: written at [tokens, ld_in] + h*128
__global__ void rope_qknorm_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ g,
                                       __nv_bfloat16* __restrict__ din, const __nv_bfloat16* __restrict__ cosb,
                                       const __nv_bfloat16* __restrict__ sinb, long tokens, int H, int T, long ld_in,
                                       long ld_din, float eps) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const int t = (int)(tok % T);
  const __nv_bfloat16* p = in + tok * ld_in + h * 128;
  const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 2 * lane));
  const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 64 + 2 * lane));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(cosb + (long)t * 64 + 2 * lane));
  const float2 s = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sinb + (long)t * 64 + 2 * lane));
  float2 o1, o2;
  o1.x = x1.x * c.x + x2.x * s.x;
  o1.y = x1.y * c.y + x2.y * s.y;
  o2.x = -x1.x * s.x + x2.x * c.x;
  o2.y = -x1.y * s.y + x2.y * c.y;
  const __nv_bfloat16* gp = g + wid * 128;
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + 2 * lane));
  const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + 64 + 2 * lane));
  float ss = o1.x * o1.x + o1.y * o1.y + o2.x * o2.x + o2.y * o2.y;
  float dot = o1.x * g1.x + o1.y * g1.y + o2.x * g2.x + o2.y * g2.y;
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss * (1.f / 128.f) + eps);
  const float k = r * r * r * dot * (1.f / 128.f);
  float2 d1, d2;  // gradient w.r.t. rotated values
  d1.x = r * g1.x - k * o1.x;
  d1.y = r * g1.y - k * o1.y;
  d2.x = r * g2.x - k * o2.x;
  d2.y = r * g2.y - k * o2.y;
  // inverse rotation: dx1 = d1*c - d2*s ; dx2 = d1*s + d2*c
  __nv_bfloat16* q = din + tok * ld_din + h * 128;
  *reinterpret_cast<__nv_bfloat162*>(q + 2 * lane) = __floats2bfloat162_rn(d1.x * c.x - d2.x * s.x, d1.y * c.y - d2.y * s.y);
  *reinterpret_cast<__nv_bfloat162*>(q + 64 + 2 * lane) =
      __floats2bfloat162_rn(d1.x * s.x + d2.x * c.x, d1.y * s.y + d2.y * c.y);
}

// ------------------------------------------------------------------ per-head gate ops, head_dim = 128
// mode 0: out = a + gate*b   (value residual; a at [tokens, ld_a] + h*128, b,out contiguous / ld given)
// mode 1: out = a * gate     (attention gate)
__global__ void head_gate_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                     const float* __restrict__ gate, __nv_bfloat16* __restrict__ out, long tokens, int H,
                                     long ld_a, long ld_b, long ld_out, int mode) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const float gt = gate[wid];
  const __nv_bfloat16* ap = a + tok * ld_a + h * 128 + lane * 4;
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ap));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ap + 2));
  float o[4];
  if (mode == 0) {
    const __nv_bfloat16* bp = b + tok * ld_b + h * 128 + lane * 4;
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bp));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bp + 2));
    o[0] = a0.x + gt * b0.x; o[1] = a0.y + gt * b0.y; o[2] = a1.x + gt * b1.x; o[3] = a1.y + gt * b1.y;
  } else {
    o[0] = a0.x * gt; o[1] = a0.y * gt; o[2] = a1.x * gt; o[3] = a1.y * gt;
  }
  __nv_bfloat16* op = out + tok * ld_out + h * 128 + lane * 4;
  *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(o[0], o[1]);
  *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(o[2], o[3]);
}

// mode 0: db = gate*g ; dgate = sum_d g*b           (da = g, handled by the caller)
// mode 1: da = gate*g ; dgate = sum_d g*a
__global__ void head_gate_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ other,
                                     const float* __restrict__ gate, __nv_bfloat16* __restrict__ dother,
                                     float* __restrict__ dgate, long tokens, int H, long ld_g, long ld_other,
                                     long ld_dother, float* __restrict__ delta, int T) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const float gt = gate[wid];
  const __nv_bfloat16* gp = g + tok * ld_g + h * 128 + lane * 4;
  const __nv_bfloat16* bp = other + tok * ld_other + h * 128 + lane * 4;
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + 2));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bp));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bp + 2));
  float dot = g0.x * b0.x + g0.y * b0.y + g1.x * b1.x + g1.y * b1.y;
  dot = warp_sum(dot);
  if (lane == 0) {
    dgate[wid] = dot;
    // rowsum(d_other * other) = gate * dot: the `delta` term of the attention backward, laid out (B, H, T)
    if (delta != nullptr) delta[((tok / T) * H + h) * T + (tok % T)] = gt * dot;
  }
  __nv_bfloat16* op = dother + tok * ld_dother + h * 128 + lane * 4;
  *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(gt * g0.x, gt * g0.y);
  *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(gt * g1.x, gt * g1.y);
}

// ------------------------------------------------------------------ SwiGLU on a fused [M, 2h] buffer
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gf, __nv_bfloat16* __restrict__ out, long M, int h) {
  const long per_row = h / 8;
  const long n8 = M * per_row;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long row = i / per_row;
    const long c = (i - row * per_row) * 8;
    float g[8], f[8], o[8];
    load8(gf + row * 2 * h + c, g);
    load8(gf + row * 2 * h + h + c, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * f[j];
    store8(out + row * h + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gf, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgf, long M, int h) {
  const long per_row = h / 8;
  const long n8 = M * per_row;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long row = i / per_row;
    const long c = (i - row * per_row) * 8;
    float g[8], f[8], d[8], dg[8], df[8];
    load8(gf + row * 2 * h + c, g);
    load8(gf + row * 2 * h + h + c, f);
    load8(dout + row * h + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      df[j] = d[j] * silu;
      dg[j] = d[j] * f[j] * (sg + silu * (1.f - sg));
    }
    store8(dgf + row * 2 * h + c, dg);
    store8(dgf + row * 2 * h + h + c, df);
  }
}

// ------------------------------------------------------------------ residual + dropout (+ stochastic depth)
// out = x_in + keep*(x_mid + drop(y) - x_in); with x_in == nullptr: out = x_mid + drop(y)
__global__ void dropout_add_fwd_kernel(const __nv_bfloat16* __restrict__ x_mid, const __nv_bfloat16* __restrict__ y,
                                       const __nv_bfloat16* __restrict__ x_in, const float* __restrict__ keep_p,
                                       __nv_bfloat16* __restrict__ out, long n8, float p, uint64_t salt,
                                       const unsigned long long* __restrict__ seed_ptr) {
  const uint64_t seed = salt + (seed_ptr ? (*seed_ptr) * 0x9E3779B97F4A7C15ull : 0ull);
  const float keep = (x_in != nullptr) ? *keep_p : 1.f;
  const float scale = 1.f / (1.f - p);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    load8(x_mid + i * 8, a);
    load8(y + i * 8, b);
    if (p > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = keep_elem(seed, (uint64_t)i * 8 + j, p) ? b[j] * scale : 0.f;
    }
    if (x_in != nullptr) {
      float xi[8];
      load8(x_in + i * 8, xi);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = xi[j] + keep * (a[j] + b[j] - xi[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = a[j] + b[j];
    }
    store8(out + i * 8, o);
  }
}
// dy = keep * mask/(1-p) * g ; (optional) dmid = keep*g ; (optional) din = (1-keep)*g
__global__ void dropout_add_bwd_kernel(const __nv_bfloat16* __restrict__ g, const float* __restrict__ keep_p,
                                       __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dmid,
                                       __nv_bfloat16* __restrict__ din, long n8, float p, uint64_t salt,
                                       const unsigned long long* __restrict__ seed_ptr) {
  const uint64_t seed = salt + (seed_ptr ? (*seed_ptr) * 0x9E3779B97F4A7C15ull : 0ull);
  const float keep = (keep_p != nullptr) ? *keep_p : 1.f;
  const float scale = 1.f / (1.f - p);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float gg[8], o[8];
    load8(g + i * 8, gg);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool k = (p > 0.f) ? keep_elem(seed, (uint64_t)i * 8 + j, p) : true;
      o[j] = k ? keep * scale * gg[j] : 0.f;
    }
    store8(dy + i * 8, o);
    if (dmid != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = keep * gg[j];
      store8(dmid + i * 8, o);
    }
    if (din != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (1.f - keep) * gg[j];
      store8(din + i * 8, o);
    }
  }
}


// ------------------------------------------------------------------ residual + dropout fused with the following RMSNorm
// x_mid = x + drop(y);  n = rmsnorm(x_mid).  One warp per row; the norm is taken of the bf16-rounded x_mid, exactly as
// the two separate kernels would. Element (row, c) uses the same mask index as dropout_add_fwd_kernel (row * D + c).
__global__ void add_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                    __nv_bfloat16* __restrict__ x_mid, __nv_bfloat16* __restrict__ n, long rows, int D,
                                    float eps, float p, uint64_t salt, const unsigned long long* __restrict__ seed_ptr) {
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint64_t seed = salt + (seed_ptr ? (*seed_ptr) * 0x9E3779B97F4A7C15ull : 0ull);
  const float scale = 1.f / (1.f - p);
  const long base = row * (long)D;
  float ss = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float a[8], b[8];
    load8(x + base + c, a);
    load8(y + base + c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (p > 0.f) b[j] = keep_elem(seed, (uint64_t)(base + c + j), p) ? b[j] * scale : 0.f;
      a[j] = __bfloat162float(__float2bfloat16(a[j] + b[j]));
      ss += a[j] * a[j];
    }
    store8(x_mid + base + c, a);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    load8(x_mid + base + c, f);   // this lane's own stores
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= r;
    store8(n + base + c, f);
  }
}

// Backward of the pair above seen from the MLP side: dx_mid = rmsnorm_bwd(x_mid, dn) + g_res, and the gradient of the
// dropped branch dy = mask/(1-p) * dx_mid (of the bf16-rounded dx_mid), in one pass over the row.
__global__ void norm_bwd_drop_kernel(const __nv_bfloat16* __restrict__ x_mid, const __nv_bfloat16* __restrict__ dn,
                                     const __nv_bfloat16* __restrict__ g_res, __nv_bfloat16* __restrict__ dx_mid,
                                     __nv_bfloat16* __restrict__ dy, long rows, int D, float eps, float p, uint64_t salt,
                                     const unsigned long long* __restrict__ seed_ptr) {
  const long row = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint64_t seed = salt + (seed_ptr ? (*seed_ptr) * 0x9E3779B97F4A7C15ull : 0ull);
  const float scale = 1.f / (1.f - p);
  const long base = row * (long)D;
  float ss = 0.f, dot = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], g[8];
    load8(x_mid + base + c, f);
    load8(dn + base + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss += f[i] * f[i];
      dot += f[i] * g[i];
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss / D + eps);
  const float k = r * r * r * dot / D;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], g[8], a[8], o[8], d[8];
    load8(x_mid + base + c, f);
    load8(dn + base + c, g);
    load8(g_res + base + c, a);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o[i] = __bfloat162float(__float2bfloat16(r * g[i] - k * f[i] + a[i]));
      const bool keep = (p > 0.f) ? keep_elem(seed, (uint64_t)(base + c + i), p) : true;
      d[i] = keep ? scale * o[i] : 0.f;
    }
    store8(dx_mid + base + c, o);
    store8(dy + base + c, d);
  }
}

// grad_fp32 += g (bf16)   -- accumulation of a bf16 weight gradient into the fp32 gradient arena
__global__ void acc_bf16_into_f32_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ g, long n8) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float f[8];
    load8(g + i * 8, f);
    float4* a = reinterpret_cast<float4*>(acc + i * 8);
    float4 a0 = a[0], a1 = a[1];
    a0.x += f[0]; a0.y += f[1]; a0.z += f[2]; a0.w += f[3];
    a1.x += f[4]; a1.y += f[5]; a1.z += f[6]; a1.w += f[7];
    a[0] = a0;
    a[1] = a1;
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

#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int sr_rmsnorm_fwd(const void* x, void* y, long rows, int D, long ldx, float eps, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (D % 8 || ldx % 8) return -2;
  rmsnorm_fwd_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(x), BFM(y), rows, D, ldx, eps);
  return rc();
}
extern "C" int sr_rmsnorm_bwd(const void* x, const void* dy, const void* dres, void* dx, long rows, int D, long ldx,
                              float eps, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (D % 8 || ldx % 8) return -2;
  rmsnorm_bwd_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(x), BF(dy), BF(dres), BFM(dx), rows, D, ldx, eps);
  return rc();
}
extern "C" int sr_lambda_mix_fwd(const void* x, const void* x0, const void* skip, void* out, const float* lr,
                                 const float* l0, const float* ws, long n, cudaStream_t s) {
  if (n % 8) return -2;
  lambda_mix_fwd_kernel<<<grid_for(n / 8, kThreads), kThreads, 0, s>>>(BF(x), BF(x0), BF(skip), BFM(out), lr, l0, ws, n / 8);
  return rc();
}
extern "C" int sr_lambda_mix_bwd(const void* g, const void* x, const void* x0, const void* skip, void* dx, void* dx0,
                                 void* dskip, const float* lr, const float* l0, const float* ws, float* dscal, long n,
                                 cudaStream_t s) {
  if (n % 8) return -2;
  lambda_mix_bwd_kernel<<<grid_for(n / 8, kThreads), kThreads, 0, s>>>(BF(g), BF(x), BF(x0), BF(skip), BFM(dx), BFM(dx0), BFM(dskip), lr, l0, ws, dscal, n / 8);
  return rc();
}
extern "C" int sr_rope_qknorm_fwd(const void* in, void* out, const void* cosb, const void* sinb, long tokens, int H,
                                  int T, long ld_in, float eps, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  rope_qknorm_fwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(in), BFM(out), BF(cosb), BF(sinb), tokens, H, T, ld_in, eps);
  return rc();
}
extern "C" int sr_rope_qknorm_bwd(const void* in, const void* g, void* din, const void* cosb, const void* sinb,
                                  long tokens, int H, int T, long ld_in, long ld_din, float eps, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  rope_qknorm_bwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(in), BF(g), BFM(din), BF(cosb), BF(sinb), tokens, H, T, ld_in, ld_din, eps);
  return rc();
}
extern "C" int sr_head_gate_fwd(const void* a, const void* b, const float* gate, void* out, long tokens, int H,
                                long ld_a, long ld_b, long ld_out, int mode, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  head_gate_fwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(a), BF(b), gate, BFM(out), tokens, H, ld_a, ld_b, ld_out, mode);
  return rc();
}
extern "C" int sr_head_gate_bwd(const void* g, const void* other, const float* gate, void* dother, float* dgate,
                                long tokens, int H, long ld_g, long ld_other, long ld_dother, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  head_gate_bwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(g), BF(other), gate, BFM(dother), dgate, tokens, H, ld_g, ld_other, ld_dother, nullptr, 1);
  return rc();
}
// Scale-mode backward that also emits delta[b, h, t] = sum_d dother * other (tokens = B * T rows, row = b * T + t).
extern "C" int sr_head_gate_bwd_delta(const void* g, const void* other, const float* gate, void* dother, float* dgate,
                                      float* delta, long tokens, int H, int T, long ld_g, long ld_other, long ld_dother,
                                      cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  head_gate_bwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(BF(g), BF(other), gate, BFM(dother), dgate, tokens, H, ld_g, ld_other, ld_dother, delta, T);
  return rc();
}
extern "C" int sr_swiglu_fwd(const void* gf, void* out, long M, int h, cudaStream_t s) {
  if (h % 8) return -2;
  swiglu_fwd_kernel<<<grid_for(M * (h / 8), kThreads), kThreads, 0, s>>>(BF(gf), BFM(out), M, h);
  return rc();
}
extern "C" int sr_swiglu_bwd(const void* gf, const void* dout, void* dgf, long M, int h, cudaStream_t s) {
  if (h % 8) return -2;
  swiglu_bwd_kernel<<<grid_for(M * (h / 8), kThreads), kThreads, 0, s>>>(BF(gf), BF(dout), BFM(dgf), M, h);
  return rc();
}
extern "C" int sr_dropout_add_fwd(const void* x_mid, const void* y, const void* x_in, const float* keep, void* out,
                                  long n, float p, unsigned long long seed, const unsigned long long* seed_ptr,
                                  cudaStream_t s) {
  if (n % 8) return -2;
  dropout_add_fwd_kernel<<<grid_for(n / 8, kThreads), kThreads, 0, s>>>(BF(x_mid), BF(y), BF(x_in), keep, BFM(out), n / 8, p, seed, seed_ptr);
  return rc();
}
extern "C" int sr_dropout_add_bwd(const void* g, const float* keep, void* dy, void* dmid, void* din, long n, float p,
                                  unsigned long long seed, const unsigned long long* seed_ptr, cudaStream_t s) {
  if (n % 8) return -2;
  dropout_add_bwd_kernel<<<grid_for(n / 8, kThreads), kThreads, 0, s>>>(BF(g), keep, BFM(dy), BFM(dmid), BFM(din), n / 8, p, seed, seed_ptr);
  return rc();
}
extern "C" int sr_acc_bf16_into_f32(float* acc, const void* g, long n, cudaStream_t s) {
  if (n % 8) return -2;
  acc_bf16_into_f32_kernel<<<grid_for(n / 8, kThreads), kThreads, 0, s>>>(acc, BF(g), n / 8);
  return rc();
}

// x_mid = x + dropout(y); n = rmsnorm(x_mid). Contiguous [rows, D] bf16, D % 8 == 0. Same mask as sr_dropout_add_fwd.
extern "C" int sr_add_norm_fwd(const void* x, const void* y, void* x_mid, void* n, long rows, int D, float eps, float p,
                               unsigned long long seed, const unsigned long long* seed_ptr, cudaStream_t s) {
  if (D % 8) return -2;
  if (rows <= 0) return 0;
  add_norm_fwd_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(x), BF(y), BFM(x_mid), BFM(n), rows, D, eps, p, seed, seed_ptr);
  return rc();
}
// dx_mid = rmsnorm_bwd(x_mid, dn) + g_res; dy = dropout_bwd(dx_mid) with the mask of sr_add_norm_fwd / sr_dropout_add_fwd.
extern "C" int sr_norm_bwd_drop(const void* x_mid, const void* dn, const void* g_res, void* dx_mid, void* dy, long rows,
                                int D, float eps, float p, unsigned long long seed, const unsigned long long* seed_ptr,
                                cudaStream_t s) {
  if (D % 8) return -2;
  if (rows <= 0) return 0;
  norm_bwd_drop_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(x_mid), BF(dn), BF(g_res), BFM(dx_mid), BFM(dy), rows, D, eps, p, seed, seed_ptr);
  return rc();
}

// x = lr*(xp + ws*skip) + l0*x0 and a = rmsnorm(x) in one pass; scalars are device pointers; skip may be null.
extern "C" int sr_mix_norm_fwd(const void* xp, const void* x0, const void* skip, void* x, void* a, const float* lr,
                               const float* l0, const float* ws, long rows, int D, float eps, cudaStream_t s) {
  if (D % 8) return -2;
  if (rows <= 0) return 0;
  mix_norm_fwd_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(xp), BF(x0), BF(skip), BFM(x), BFM(a), lr, l0, ws, rows, D, eps);
  return rc();
}
// Backward through the first norm and the lambda mix: see norm_bwd_mix_kernel. d_lr / d_l0 / d_ws: the fp32 gradient
// entries of the three scalars, accumulated into (d_ws is not touched without a skip input). g_res2: optional second
// residual gradient, added to g_res first.
extern "C" int sr_norm_bwd_mix(const void* x, const void* da, const void* g_res, const void* g_res2, const void* xp,
                               const void* x0,
                               const void* skip, void* dxp, void* dx0, void* dskip, const float* lr, const float* l0,
                               const float* ws, float* d_lr, float* d_l0, float* d_ws, long rows, int D, float eps,
                               cudaStream_t s) {
  if (D % 8) return -2;
  if (rows <= 0) return 0;
  norm_bwd_mix_kernel<<<(unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(x), BF(da), BF(g_res), BF(g_res2), BF(xp), BF(x0), BF(skip), BFM(dxp), BFM(dx0), BFM(dskip), lr, l0, ws, d_lr, d_l0, d_ws, rows, D, eps);
  return rc();
}
