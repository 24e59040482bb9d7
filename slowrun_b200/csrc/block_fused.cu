// Kernels that exist only because the transformer block is executed as ONE autograd node with a hand-written
// backward (slowrun_b200/ops/block.py): every gradient buffer is written exactly once, so no slice/concat/zero-fill
// glue is left to the autograd engine.
//
//   qkv_prep fwd/bwd   split the fused [M, 3d] projection, add the gated value residual to v, apply RoPE and the
//                      per-head RMSNorm to q and k; backward writes one dense dqkv buffer (train.py:296-306).
//                      With `key_offset` the upper half of every key vector is the one computed for the previous token
//                      of the same sequence (token 0 keeps its own): the tiny track's partial key offset on
//                      long-window layers (tiny/train.py:447-449), done as a shifted store / shifted gradient load.
//   attn_post fwd/bwd  what follows the attention kernel per (token, head): exclusive self-attention
//                      y -= tanh(alpha_h) (y . v^) v^ with v^ the normalised value vector of the same token
//                      (tiny/train.py:451-458), then the per-head sigmoid gate (train.py:308-309). The backward also
//                      emits the attention backward's `delta` = rowsum(dO * O), the XSA contribution to dV and the
//                      gradient of alpha.
//   iha_mix fwd/bwd    Interleaved-head mixing of projection weights W'[h] = sum_m mix[h,m] W[m] on bf16 shadows and
//                      its gradients (dW += mix^T dW', dmix = dW' W^T). The reference leaves the [H, d*D] x [d*D, H]
//                      product to a library GEMM (train.py:277-280); with H <= 20 that is a long skinny reduction,
//                      done here as a streaming kernel plus a shared-memory tree.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// ---------------------------------------------------------------------------------------------- qkv prep
// One warp per (token, head); lane l owns elements {2l, 2l+1} and {64+2l, 64+2l+1} of each 128-wide head vector.
__global__ void qkv_prep_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ ve,
                                    const float* __restrict__ gate, const __nv_bfloat16* __restrict__ cosb,
                                    const __nv_bfloat16* __restrict__ sinb, __nv_bfloat16* __restrict__ q_out,
                                    __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ v_out, long tokens, int H,
                                    int T, float eps, int key_offset) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const int t = (int)(tok % T);
  const long d = (long)H * 128;
  const float2 c = ld2(cosb + (long)t * 64 + 2 * lane);
  const float2 s = ld2(sinb + (long)t * 64 + 2 * lane);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* p = qkv + tok * 3 * d + which * d + h * 128;
    const float2 x1 = ld2(p + 2 * lane), x2 = ld2(p + 64 + 2 * lane);
    float2 o1, o2;
    o1.x = x1.x * c.x + x2.x * s.x;
    o1.y = x1.y * c.y + x2.y * s.y;
    o2.x = -x1.x * s.x + x2.x * c.x;
    o2.y = -x1.y * s.y + x2.y * c.y;
    float ss = o1.x * o1.x + o1.y * o1.y + o2.x * o2.x + o2.y * o2.y;
    ss = warp_sum(ss);
    const float r = rsqrtf(ss * (1.f / 128.f) + eps);
    __nv_bfloat16* o = (which == 0 ? q_out : k_out) + wid * 128;
    st2(o + 2 * lane, o1.x * r, o1.y * r);
    if (which == 1 && key_offset) {
      // upper half goes to the next token of the sequence (same head: H rows further); token 0 also keeps its own
      if (t + 1 < T) st2(o + (long)H * 128 + 64 + 2 * lane, o2.x * r, o2.y * r);
      if (t == 0) st2(o + 64 + 2 * lane, o2.x * r, o2.y * r);
    } else {
      st2(o + 64 + 2 * lane, o2.x * r, o2.y * r);
    }
  }
  {
    const __nv_bfloat16* p = qkv + tok * 3 * d + 2 * d + h * 128 + lane * 4;
    float2 a0 = ld2(p), a1 = ld2(p + 2);
    if (ve != nullptr) {
      const float g = gate[wid];
      const __nv_bfloat16* e = ve + tok * d + h * 128 + lane * 4;
      const float2 e0 = ld2(e), e1 = ld2(e + 2);
      a0.x += g * e0.x; a0.y += g * e0.y; a1.x += g * e1.x; a1.y += g * e1.y;
    }
    __nv_bfloat16* o = v_out + wid * 128 + lane * 4;
    st2(o, a0.x, a0.y);
    st2(o + 2, a1.x, a1.y);
  }
}

__global__ void qkv_prep_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ ve,
                                    const float* __restrict__ gate, const __nv_bfloat16* __restrict__ cosb,
                                    const __nv_bfloat16* __restrict__ sinb, const __nv_bfloat16* __restrict__ dq,
                                    const __nv_bfloat16* __restrict__ dk, const __nv_bfloat16* __restrict__ dv,
                                    __nv_bfloat16* __restrict__ dqkv, __nv_bfloat16* __restrict__ dve,
                                    float* __restrict__ dgate, long tokens, int H, int T, float eps,
                                    const float* __restrict__ dq_f32, int key_offset,
                                    const __nv_bfloat16* __restrict__ dv_extra) {
  const long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long tok = wid / H;
  const int h = (int)(wid - tok * H);
  const int t = (int)(tok % T);
  const long d = (long)H * 128;
  const float2 c = ld2(cosb + (long)t * 64 + 2 * lane);
  const float2 s = ld2(sinb + (long)t * 64 + 2 * lane);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* p = qkv + tok * 3 * d + which * d + h * 128;
    const float2 x1 = ld2(p + 2 * lane), x2 = ld2(p + 64 + 2 * lane);
    float2 o1, o2;
    o1.x = x1.x * c.x + x2.x * s.x;
    o1.y = x1.y * c.y + x2.y * s.y;
    o2.x = -x1.x * s.x + x2.x * c.x;
    o2.y = -x1.y * s.y + x2.y * c.y;
    float2 g1, g2;
    if (which == 0 && dq_f32 != nullptr) {   // dQ straight from the attention kernel's fp32 accumulator
      const float* gp = dq_f32 + wid * 128;
      g1 = *reinterpret_cast<const float2*>(gp + 2 * lane);
      g2 = *reinterpret_cast<const float2*>(gp + 64 + 2 * lane);
    } else {
      const __nv_bfloat16* gp = (which == 0 ? dq : dk) + wid * 128;
      g1 = ld2(gp + 2 * lane);
      if (which == 1 && key_offset) {
        // the upper half computed here was consumed by the next token (and by token 0 itself)
        g2 = make_float2(0.f, 0.f);
        if (t + 1 < T) g2 = ld2(gp + (long)H * 128 + 64 + 2 * lane);
        if (t == 0) {
          const float2 own = ld2(gp + 64 + 2 * lane);
          g2.x += own.x;
          g2.y += own.y;
        }
      } else {
        g2 = ld2(gp + 64 + 2 * lane);
      }
    }
    float ss = o1.x * o1.x + o1.y * o1.y + o2.x * o2.x + o2.y * o2.y;
    float dot = o1.x * g1.x + o1.y * g1.y + o2.x * g2.x + o2.y * g2.y;
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float r = rsqrtf(ss * (1.f / 128.f) + eps);
    const float k = r * r * r * dot * (1.f / 128.f);
    float2 d1, d2;
    d1.x = r * g1.x - k * o1.x;
    d1.y = r * g1.y - k * o1.y;
    d2.x = r * g2.x - k * o2.x;
    d2.y = r * g2.y - k * o2.y;
    __nv_bfloat16* o = dqkv + tok * 3 * d + which * d + h * 128;
    st2(o + 2 * lane, d1.x * c.x - d2.x * s.x, d1.y * c.y - d2.y * s.y);
    st2(o + 64 + 2 * lane, d1.x * s.x + d2.x * c.x, d1.y * s.y + d2.y * c.y);
  }
  {
    const __nv_bfloat16* gp = dv + wid * 128 + lane * 4;
    float2 g0 = ld2(gp), g1 = ld2(gp + 2);
    if (dv_extra != nullptr) {    // second consumer of v (exclusive self-attention)
      const float2 x0 = ld2(dv_extra + wid * 128 + lane * 4), x1 = ld2(dv_extra + wid * 128 + lane * 4 + 2);
      g0.x += x0.x; g0.y += x0.y; g1.x += x1.x; g1.y += x1.y;
    }
    __nv_bfloat16* o = dqkv + tok * 3 * d + 2 * d + h * 128 + lane * 4;
    st2(o, g0.x, g0.y);
    st2(o + 2, g1.x, g1.y);
    if (ve != nullptr) {
      const float g = gate[wid];
      const __nv_bfloat16* e = ve + tok * d + h * 128 + lane * 4;
      const float2 e0 = ld2(e), e1 = ld2(e + 2);
      float dot = g0.x * e0.x + g0.y * e0.y + g1.x * e1.x + g1.y * e1.y;
      dot = warp_sum(dot);
      if (lane == 0) dgate[wid] = dot;
      __nv_bfloat16* de = dve + tok * d + h * 128 + lane * 4;
      st2(de, g * g0.x, g * g0.y);
      st2(de + 2, g * g1.x, g * g1.y);
    }
  }
}

// ---------------------------------------------------------------------------------------------- after attention
// One warp per (token, head) row of 128; lane l owns elements 4l .. 4l+3. alpha: fp32 [H] (raw, tanh applied here) or
// null = no exclusive self-attention.
struct Row4 {
  float v[4];
};
__device__ __forceinline__ Row4 ld4(const __nv_bfloat16* p) {
  const float2 a = ld2(p), b = ld2(p + 2);
  return Row4{{a.x, a.y, b.x, b.y}};
}
__device__ __forceinline__ float dot4(const Row4& a, const Row4& b) {
  return a.v[0] * b.v[0] + a.v[1] * b.v[1] + a.v[2] * b.v[2] + a.v[3] * b.v[3];
}

__global__ void attn_post_fwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ v,
                                     const float* __restrict__ gate, const float* __restrict__ alpha,
                                     __nv_bfloat16* __restrict__ out, long rows, int H, float xsa_eps) {
  const int lane = threadIdx.x & 31;
  for (long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); wid < rows; wid += (long)gridDim.x * kWarpsPerBlock) {
    Row4 yy = ld4(y + wid * 128 + lane * 4);
    if (alpha != nullptr) {
      const Row4 vv = ld4(v + wid * 128 + lane * 4);
      const float n = fmaxf(sqrtf(warp_sum(dot4(vv, vv))), xsa_eps);
      const float c = warp_sum(dot4(yy, vv)) / n;
      const float k = tanhf(alpha[wid % H]) * c / n;
#pragma unroll
      for (int i = 0; i < 4; ++i) yy.v[i] -= k * vv.v[i];
    }
    const float s = gate[wid];
    __nv_bfloat16* o = out + wid * 128 + lane * 4;
    st2(o, yy.v[0] * s, yy.v[1] * s);
    st2(o + 2, yy.v[2] * s, yy.v[3] * s);
  }
}

// g: gradient of the gated output. Writes dy (gradient of the attention output), dgate (w.r.t. the gate value),
// delta[b, h, t] = sum_d dy * y, and with alpha: dv_x (this op's gradient of v) and dalpha[H] += (atomics, one per
// block and head).
__global__ void attn_post_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ y,
                                     const __nv_bfloat16* __restrict__ v, const float* __restrict__ gate,
                                     const float* __restrict__ alpha, __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dgate, float* __restrict__ delta,
                                     __nv_bfloat16* __restrict__ dv_x, float* __restrict__ dalpha, long rows, int H, int T,
                                     float xsa_eps) {
  __shared__ float dal[64];
  const int lane = threadIdx.x & 31;
  if (alpha != nullptr) {
    if (threadIdx.x < 64) dal[threadIdx.x] = 0.f;
    __syncthreads();
  }
  for (long wid = (long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); wid < rows; wid += (long)gridDim.x * kWarpsPerBlock) {
    const long tok = wid / H;
    const int h = (int)(wid - tok * H);
    const Row4 gg = ld4(g + wid * 128 + lane * 4);
    const Row4 yy = ld4(y + wid * 128 + lane * 4);
    const float s = gate[wid];
    Row4 d;      // gradient of the attention output
    float dg;    // sum_d g * (output before the gate)
    if (alpha != nullptr) {
      const Row4 vv = ld4(v + wid * 128 + lane * 4);
      const float nrm = sqrtf(warp_sum(dot4(vv, vv)));
      const float n = fmaxf(nrm, xsa_eps);
      const float inv = 1.f / n;
      const float c = warp_sum(dot4(yy, vv)) * inv;          // y . u,  u = v / n
      const float a = tanhf(alpha[h]);
      const float gy = warp_sum(dot4(gg, yy)), gu = warp_sum(dot4(gg, vv)) * inv;
      dg = gy - a * c * gu;                                   // g . (y - a c u)
      const float p = s * gu;                                 // (s g) . u
      Row4 du;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float u = vv.v[i] * inv, dyp = s * gg.v[i];
        d.v[i] = dyp - a * p * u;
        du.v[i] = -a * (p * yy.v[i] + c * dyp);
      }
      // v -> u = v / max(|v|, eps): the projection term only where the norm is not clamped
      const float duu = nrm > xsa_eps ? warp_sum(dot4(du, vv)) * inv : 0.f;
      __nv_bfloat16* o = dv_x + wid * 128 + lane * 4;
      st2(o, (du.v[0] - duu * vv.v[0] * inv) * inv, (du.v[1] - duu * vv.v[1] * inv) * inv);
      st2(o + 2, (du.v[2] - duu * vv.v[2] * inv) * inv, (du.v[3] - duu * vv.v[3] * inv) * inv);
      if (lane == 0) atomicAdd(&dal[h], -c * p * (1.f - a * a));
    } else {
      dg = warp_sum(dot4(gg, yy));
#pragma unroll
      for (int i = 0; i < 4; ++i) d.v[i] = s * gg.v[i];
    }
    const float dl = warp_sum(dot4(d, yy));
    if (lane == 0) {
      dgate[wid] = dg;
      delta[((tok / T) * H + h) * T + (tok % T)] = dl;
    }
    __nv_bfloat16* o = dy + wid * 128 + lane * 4;
    st2(o, d.v[0], d.v[1]);
    st2(o + 2, d.v[2], d.v[3]);
  }
  if (alpha != nullptr) {
    __syncthreads();
    if (threadIdx.x < H && dal[threadIdx.x] != 0.f) atomicAdd(dalpha + threadIdx.x, dal[threadIdx.x]);
  }
}

// ---------------------------------------------------------------------------------------------- IHA weight mixing
// W, out: [P, H, J] bf16 (J = head_dim * d_in); mix: [P, H, H] fp32, used rounded to bf16 as the reference's autocast
// matmul does. One thread per pair of columns.
template <int H>
__global__ void iha_mix_fwd_kernel(const float* __restrict__ mix, const __nv_bfloat16* __restrict__ W,
                                   __nv_bfloat16* __restrict__ out, long J) {
  __shared__ float sm[H * H];
  const int p = blockIdx.y;
  for (int i = threadIdx.x; i < H * H; i += blockDim.x)
    sm[i] = __bfloat162float(__float2bfloat16(mix[(long)p * H * H + i]));
  __syncthreads();
  const long j = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (j >= J) return;
  const __nv_bfloat16* w = W + (long)p * H * J + j;
  float2 x[H];
#pragma unroll
  for (int m = 0; m < H; ++m) x[m] = ld2(w + (long)m * J);
  __nv_bfloat16* o = out + (long)p * H * J + j;
#pragma unroll
  for (int h = 0; h < H; ++h) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int m = 0; m < H; ++m) {
      a += sm[h * H + m] * x[m].x;
      b += sm[h * H + m] * x[m].y;
    }
    st2(o + (long)h * J, a, b);
  }
}

// gradW[p, m, j] += sum_h mix[p, h, m] * dWp[p, h, j]      (fp32 accumulate into the gradient arena)
template <int H>
__global__ void iha_mix_bwd_w_kernel(const float* __restrict__ mix, const __nv_bfloat16* __restrict__ dWp,
                                     float* __restrict__ gradW, long J) {
  __shared__ float sm[H * H];
  const int p = blockIdx.y;
  for (int i = threadIdx.x; i < H * H; i += blockDim.x)
    sm[i] = __bfloat162float(__float2bfloat16(mix[(long)p * H * H + i]));
  __syncthreads();
  const long j = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (j >= J) return;
  const __nv_bfloat16* g = dWp + (long)p * H * J + j;
  float2 x[H];
#pragma unroll
  for (int h = 0; h < H; ++h) x[h] = ld2(g + (long)h * J);
  float* o = gradW + (long)p * H * J + j;
#pragma unroll
  for (int m = 0; m < H; ++m) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int h = 0; h < H; ++h) {
      a += sm[h * H + m] * x[h].x;
      b += sm[h * H + m] * x[h].y;
    }
    // fire-and-forget vector reduction: a load-add-store here would serialise H DRAM round trips per thread
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(o + (long)m * J), "f"(a), "f"(b) : "memory");
  }
}

// dmix[p, h, m] += sum_j dWp[p, h, j] * W[p, m, j].  Each CTA stages `kCols` columns of both operands in shared memory
// (rows padded by one word against bank conflicts). The H x H result is cut into 4 x 4 register blocks; a thread owns
// one block for one slice of the staged columns, so every shared-memory word it loads feeds four multiply-adds.
// Slices are combined with shared-memory atomics, CTAs with one global atomicAdd per entry.
constexpr int kCols = 512;
constexpr int kChunksPerCta = 3;
template <int H>
__global__ void __launch_bounds__(kThreads)
iha_mix_bwd_mix_kernel(const __nv_bfloat16* __restrict__ dWp, const __nv_bfloat16* __restrict__ W,
                       float* __restrict__ dmix, long J) {
  constexpr int kStride = kCols + 2;
  constexpr int HB = (H + 3) / 4;                 // 4-row blocks per side
  constexpr int HP = HB * 4;                      // padded head count (extra rows are zero)
  constexpr int kBlocks = HB * HB;
  constexpr int kSlices = kThreads / kBlocks > 0 ? kThreads / kBlocks : 1;
  constexpr int kSliceCols = (kCols / 2 + kSlices - 1) / kSlices;   // bf16 pairs per slice
  __shared__ __nv_bfloat16 sg[HP * kStride];
  __shared__ __nv_bfloat16 sw[HP * kStride];
  __shared__ float sacc[HP * HP];
  const int p = blockIdx.y;
  for (int i = threadIdx.x; i < HP * HP; i += kThreads) sacc[i] = 0.f;
  const int blk = threadIdx.x % kBlocks, slice = threadIdx.x / kBlocks;
  const int bh = (blk / HB) * 4, bm = (blk % HB) * 4;
  const bool active = slice < kSlices;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  for (int ch = 0; ch < kChunksPerCta; ++ch) {
    const long j0 = ((long)blockIdx.x * kChunksPerCta + ch) * kCols;
    if (j0 >= J) break;
    const int ncols = (int)min((long)kCols, J - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < HP * (kCols / 2); i += kThreads) {
      const int row = i / (kCols / 2), c2 = (i - row * (kCols / 2)) * 2;
      __nv_bfloat162 a = __floats2bfloat162_rn(0.f, 0.f), b = a;
      if (row < H && c2 < ncols) {
        a = *reinterpret_cast<const __nv_bfloat162*>(dWp + ((long)p * H + row) * J + j0 + c2);
        b = *reinterpret_cast<const __nv_bfloat162*>(W + ((long)p * H + row) * J + j0 + c2);
      }
      *reinterpret_cast<__nv_bfloat162*>(sg + row * kStride + c2) = a;
      *reinterpret_cast<__nv_bfloat162*>(sw + row * kStride + c2) = b;
    }
    __syncthreads();
    if (active) {
      const int c_lo = slice * kSliceCols, c_hi = min(kCols / 2, c_lo + kSliceCols);
      for (int c = c_lo; c < c_hi; ++c) {
        float2 g[4], w[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          g[a] = ld2(sg + (bh + a) * kStride + 2 * c);
          w[a] = ld2(sw + (bm + a) * kStride + 2 * c);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] += g[a].x * w[b].x + g[a].y * w[b].y;
      }
    }
  }
  if (active) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) atomicAdd(&sacc[(bh + a) * HP + bm + b], acc[a][b]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H * H; i += kThreads) {
    const int h = i / H, m = i - h * H;
    atomicAdd(dmix + (long)p * H * H + i, sacc[h * HP + m]);
  }
}


// ---------------------------------------------------------------------------------------------- per-head gates
// gate[r, h] = scale * sigmoid(bf16(sum_c a[r, c] * bf16(W[h, c]))) over the first nc channels of the normed input
// (the reference's attn_gate / ve_gate linears under bf16 autocast, train.py:296-312). One thread per (row, head).
__global__ void gate_fwd_kernel(const __nv_bfloat16* __restrict__ a, long lda, const float* __restrict__ W,
                                float* __restrict__ gate, long M, int H, int nc, float scale) {
  extern __shared__ float gsm[];   // [H * nc] weights rounded to bf16
  for (int i = threadIdx.x; i < H * nc; i += blockDim.x) gsm[i] = __bfloat162float(__float2bfloat16(W[i]));
  __syncthreads();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * H) return;
  const long r = idx / H;
  const int h = (int)(idx - r * H);
  const __nv_bfloat16* ar = a + r * lda;
  float z = 0.f;
  for (int c = 0; c < nc; ++c) z += __bfloat162float(ar[c]) * gsm[h * nc + c];
  z = __bfloat162float(__float2bfloat16(z));
  gate[idx] = scale / (1.f + __expf(-z));
}

// dz = dgate * gate * (1 - gate / scale);  dW[h, c] += sum_r dz[r, h] * a[r, c];  da[r, c] += bf16(sum_h dz[r, h] * bf16(W[h, c])).
// A CTA stages kGateRows rows; thread (h, c) owns one weight-gradient entry, then the threads sweep the (row, c) pairs.
constexpr int kGateRows = 64;
__global__ void gate_bwd_kernel(const float* __restrict__ dgate, const float* __restrict__ gate,
                                const __nv_bfloat16* __restrict__ a, long lda, const float* __restrict__ W,
                                float* __restrict__ dW, __nv_bfloat16* __restrict__ da, long ldda, long M, int H, int nc,
                                float scale) {
  extern __shared__ float gsm[];
  float* sw = gsm;                       // [H * nc]
  float* sdz = sw + H * nc;              // [kGateRows * H]
  float* sa = sdz + kGateRows * H;       // [kGateRows * nc]
  const long r0 = (long)blockIdx.x * kGateRows;
  const int rows = (int)min((long)kGateRows, M - r0);
  for (int i = threadIdx.x; i < H * nc; i += blockDim.x) sw[i] = __bfloat162float(__float2bfloat16(W[i]));
  for (int i = threadIdx.x; i < rows * H; i += blockDim.x) {
    const float g = gate[r0 * H + i];
    sdz[i] = dgate[r0 * H + i] * g * (1.f - g / scale);
  }
  for (int i = threadIdx.x; i < rows * nc; i += blockDim.x) {
    const int r = i / nc, c = i - r * nc;
    sa[i] = __bfloat162float(a[(r0 + r) * lda + c]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < H * nc; e += blockDim.x) {
    const int h = e / nc, c = e - h * nc;
    float acc = 0.f;
    for (int r = 0; r < rows; ++r) acc += sdz[r * H + h] * sa[r * nc + c];
    atomicAdd(dW + e, acc);
  }
  for (int i = threadIdx.x; i < rows * nc; i += blockDim.x) {
    const int r = i / nc, c = i - r * nc;
    float acc = 0.f;
    for (int h = 0; h < H; ++h) acc += sdz[r * H + h] * sw[h * nc + c];
    __nv_bfloat16* d = da + (r0 + r) * ldda + c;
    *d = __float2bfloat16(__bfloat162float(*d) + __bfloat162float(__float2bfloat16(acc)));
  }
}

inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }

template <int H>
int iha_launch(int which, const float* mix, const void* W, const void* dWp, void* out, float* gradW, float* dmix, int P,
               long J, cudaStream_t s) {
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(W);
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(dWp);
  const dim3 grid((unsigned)((J / 2 + kThreads - 1) / kThreads), P);
  if (which == 0) {
    iha_mix_fwd_kernel<H><<<grid, kThreads, 0, s>>>(mix, w, reinterpret_cast<__nv_bfloat16*>(out), J);
  } else {
    iha_mix_bwd_w_kernel<H><<<grid, kThreads, 0, s>>>(mix, g, gradW, J);
    if (dmix != nullptr) {   // callers with a split-K GEMM at hand form dmix = dW' W^T there and pass null
      const long chunks = (J + kCols - 1) / kCols;
      const dim3 grid2((unsigned)((chunks + kChunksPerCta - 1) / kChunksPerCta), P);
      iha_mix_bwd_mix_kernel<H><<<grid2, kThreads, 0, s>>>(g, w, dmix, J);
    }
  }
  return rc();
}

int iha_dispatch(int which, int H, const float* mix, const void* W, const void* dWp, void* out, float* gradW,
                 float* dmix, int P, long J, cudaStream_t s) {
  if (J % 2) return -2;
  switch (H) {
    case 2: return iha_launch<2>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    case 4: return iha_launch<4>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    case 8: return iha_launch<8>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    case 14: return iha_launch<14>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    case 16: return iha_launch<16>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    case 20: return iha_launch<20>(which, mix, W, dWp, out, gradW, dmix, P, J, s);
    default: return -7;  // unsupported head count: the caller falls back to library matmuls
  }
}

}  // namespace

#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

// qkv: [tokens, 3*H*128]; ve: [tokens, H*128] or null; gate: fp32 [tokens, H] (only read when ve != null)
extern "C" int sr_qkv_prep_fwd(const void* qkv, const void* ve, const float* gate, const void* cosb, const void* sinb,
                               void* q, void* k, void* v, long tokens, int H, int T, float eps, int key_offset,
                               cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  qkv_prep_fwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(qkv), BF(ve), gate, BF(cosb), BF(sinb), BFM(q), BFM(k), BFM(v), tokens, H, T, eps, key_offset);
  return rc();
}
extern "C" int sr_qkv_prep_bwd(const void* qkv, const void* ve, const float* gate, const void* cosb, const void* sinb,
                               const void* dq, const void* dk, const void* dv, void* dqkv, void* dve, float* dgate,
                               long tokens, int H, int T, float eps, int key_offset, const void* dv_extra,
                               cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  qkv_prep_bwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(qkv), BF(ve), gate, BF(cosb), BF(sinb), BF(dq), BF(dk), BF(dv), BFM(dqkv), BFM(dve), dgate, tokens, H, T, eps,
      nullptr, key_offset, BF(dv_extra));
  return rc();
}
// Same with dQ given as the fp32 accumulator of the attention backward, (tokens, H, 128) contiguous.
extern "C" int sr_qkv_prep_bwd_f32dq(const void* qkv, const void* ve, const float* gate, const void* cosb,
                                     const void* sinb, const float* dq_f32, const void* dk, const void* dv, void* dqkv,
                                     void* dve, float* dgate, long tokens, int H, int T, float eps, int key_offset,
                                     const void* dv_extra, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  qkv_prep_bwd_kernel<<<(unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock), kThreads, 0, s>>>(
      BF(qkv), BF(ve), gate, BF(cosb), BF(sinb), nullptr, BF(dk), BF(dv), BFM(dqkv), BFM(dve), dgate, tokens, H, T, eps,
      dq_f32, key_offset, BF(dv_extra));
  return rc();
}

// y, v, out: [tokens, H, 128] bf16 contiguous; gate: fp32 [tokens, H]; alpha: fp32 [H] or null (v is then unused).
extern "C" int sr_attn_post_fwd(const void* y, const void* v, const float* gate, const float* alpha, void* out, long tokens,
                                int H, float xsa_eps, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  if (H > 64) return -2;
  long blocks = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long cap = (long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  attn_post_fwd_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(BF(y), BF(v), gate, alpha, BFM(out), n, H, xsa_eps);
  return rc();
}
// g: gradient of `out`. dy, dv_x: [tokens, H, 128] bf16; dgate: fp32 [tokens, H]; delta: fp32 [B, H, T] with tokens = B * T;
// dalpha: fp32 [H], ADDED to (the caller passes the parameter's gradient buffer). dv_x / dalpha only with alpha.
extern "C" int sr_attn_post_bwd(const void* g, const void* y, const void* v, const float* gate, const float* alpha, void* dy,
                                float* dgate, float* delta, void* dv_x, float* dalpha, long tokens, int H, int T,
                                float xsa_eps, cudaStream_t s) {
  const long n = tokens * H;
  if (n <= 0) return 0;
  if (H > 64 || (alpha != nullptr && (dv_x == nullptr || dalpha == nullptr))) return -2;
  long blocks = (n + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  attn_post_bwd_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(BF(g), BF(y), BF(v), gate, alpha, BFM(dy), dgate, delta,
                                                             BFM(dv_x), dalpha, n, H, T, xsa_eps);
  return rc();
}
// out[p] = bf16(mix[p]) @ W[p] for P stacked projections, W viewed as [P, H, J]
extern "C" int sr_iha_mix_fwd(const float* mix, const void* W, void* out, int P, int H, long J, cudaStream_t s) {
  return iha_dispatch(0, H, mix, W, nullptr, out, nullptr, nullptr, P, J, s);
}
// gradW[p] += bf16(mix[p])^T @ dWp[p] (fp32) and dmix[p] += dWp[p] @ W[p]^T (fp32, atomically accumulated)
extern "C" int sr_iha_mix_bwd(const float* mix, const void* W, const void* dWp, float* gradW, float* dmix, int P, int H,
                              long J, cudaStream_t s) {
  return iha_dispatch(1, H, mix, W, dWp, nullptr, gradW, dmix, P, J, s);
}

// gate[M, H] (fp32) = scale * sigmoid(a[:, :nc] @ bf16(W)^T); a: bf16 rows with leading dimension lda; W: fp32 [H, nc]
extern "C" int sr_gate_fwd(const void* a, long lda, const float* W, float* gate, long M, int H, int nc, float scale,
                           cudaStream_t s) {
  if (M <= 0) return 0;
  const long n = M * H;
  gate_fwd_kernel<<<(unsigned)((n + kThreads - 1) / kThreads), kThreads, H * nc * sizeof(float), s>>>(BF(a), lda, W, gate,
                                                                                                     M, H, nc, scale);
  return rc();
}
// Backward of sr_gate_fwd: dW (fp32 [H, nc]) is accumulated into, da[:, :nc] (bf16, leading dimension ldda) is added to.
extern "C" int sr_gate_bwd(const float* dgate, const float* gate, const void* a, long lda, const float* W, float* dW,
                           void* da, long ldda, long M, int H, int nc, float scale, cudaStream_t s) {
  if (M <= 0) return 0;
  const size_t smem = (size_t)(H * nc + kGateRows * H + kGateRows * nc) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  gate_bwd_kernel<<<(unsigned)((M + kGateRows - 1) / kGateRows), kThreads, smem, s>>>(dgate, gate, BF(a), lda, W, dW,
                                                                                     BFM(da), ldda, M, H, nc, scale);
  return rc();
}
