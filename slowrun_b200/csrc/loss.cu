// Soft-capped cross-entropy over bf16 logits, forward and backward in one kernel: one CTA per token row,
// pass 1 = online max/sum of z = cap*tanh(x/cap), pass 2 (row is L2 resident) writes
// dlogits = scale * (S_w * softmax(z) - sum_k w_k onehot(y_k)) * (1 - tanh^2) in place as bf16.
// Supports the shifted-target multi-token loss of the tiny track (weights w_k for targets at flattened
// index row+k, tiny/cuda_kernels.py:226-240) and ignore_index = -1. The reference computes the limited-track
// loss with fp32 logits through Inductor (train.py:559-564) and the tiny one with its NVRTC kernel.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxPredict = 4;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// z = cap * tanh(x / cap) with the hardware tanh (one special-function op; its 2^-11 relative error is an eighth of
// the bf16 quantisation of the logits themselves). The kernel is bound by the special-function pipe, so the softcap
// costs one op instead of the two of an exp + reciprocal formulation.
__device__ __forceinline__ float softcap(float x, float cap, float inv_cap, float& t) {
  if (cap <= 0.f) {
    t = 0.f;
    return x;
  }
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x * inv_cap));
  return cap * t;
}

__global__ void __launch_bounds__(kThreads)
softcap_ce_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ targets, float* __restrict__ loss,
                  const float* __restrict__ weights, int n_predict, const float* __restrict__ scale_ptr, long M,
                  int Vpad, int V, long ld, float cap, int write_grad) {
  __shared__ float red_m[kThreads / 32], red_s[kThreads / 32];
  __shared__ float sh_lse;
  const long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

  long tgt[kMaxPredict];
  float w[kMaxPredict];
  float sw = 0.f;
  for (int k = 0; k < kMaxPredict; ++k) {
    tgt[k] = -1;
    w[k] = 0.f;
    if (k < n_predict && row + k < M) {
      const long y = targets[row + k];
      const float wk = weights ? weights[k] : 1.f;
      if (y >= 0 && y < V && wk != 0.f) {
        tgt[k] = y;
        w[k] = wk;
        sw += wk;
      }
    }
  }
  if (sw == 0.f && n_predict == 1) {
    // ignored row: zero loss, zero gradient
    if (threadIdx.x == 0) loss[row] = 0.f;
    if (write_grad) {
      bf16x8 z;
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int c = threadIdx.x * 8; c < Vpad; c += kThreads * 8) *reinterpret_cast<bf16x8*>(lr + c) = z;
    }
    return;
  }

  // pass 1: online max / sum over the valid vocabulary
  float m = cap > 0.f ? cap : -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < Vpad; c += kThreads * 8) {
    const bf16x8 v = *reinterpret_cast<const bf16x8*>(lr + c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(v.v[i]);
      float t;
      if (c + 2 * i < V) {
        const float z = softcap(f.x, cap, inv_cap, t);
        if (cap > 0.f) {          // |z| <= cap: the bound serves as the maximum, exp(z - cap) >= exp(-2 cap)
          s += __expf(z - cap);
        } else if (z > m) {
          s = s * __expf(m - z) + 1.f;
          m = z;
        } else {
          s += __expf(z - m);
        }
      }
      if (c + 2 * i + 1 < V) {
        const float z = softcap(f.y, cap, inv_cap, t);
        if (cap > 0.f) {
          s += __expf(z - cap);
        } else if (z > m) {
          s = s * __expf(m - z) + 1.f;
          m = z;
        } else {
          s += __expf(z - m);
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    m = mm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red_m[warp] = m;
    red_s[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = red_m[0], ss = red_s[0];
    for (int i = 1; i < kThreads / 32; ++i) {
      const float m2 = red_m[i], s2 = red_s[i];
      const float mx = fmaxf(mm, m2);
      ss = (mm == -INFINITY ? 0.f : ss * __expf(mm - mx)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mx));
      mm = mx;
    }
    const float lse = mm + logf(ss);
    sh_lse = lse;
    float l = 0.f;
    for (int k = 0; k < kMaxPredict; ++k) {
      if (tgt[k] >= 0) {
        float t;
        const float z = softcap(__bfloat162float(lr[tgt[k]]), cap, inv_cap, t);
        l += w[k] * (lse - z);
      }
    }
    loss[row] = l;
  }
  if (!write_grad) return;
  __syncthreads();
  const float lse = sh_lse;
  const float scale = scale_ptr ? *scale_ptr : 1.f;

  // pass 2: gradient in place
  for (int c = threadIdx.x * 8; c < Vpad; c += kThreads * 8) {
    bf16x8 v = *reinterpret_cast<const bf16x8*>(lr + c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(v.v[i]);
      float g[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = c + 2 * i + e;
        float t;
        const float z = softcap(e ? f.y : f.x, cap, inv_cap, t);
        float gv = 0.f;
        if (col < V) {
          gv = sw * __expf(z - lse);
#pragma unroll
          for (int k = 0; k < kMaxPredict; ++k)
            if (tgt[k] == col) gv -= w[k];
          gv *= scale * (1.f - t * t);
        }
        g[e] = gv;
      }
      v.v[i] = __floats2bfloat162_rn(g[0], g[1]);
    }
    *reinterpret_cast<bf16x8*>(lr + c) = v;
  }
}

}  // namespace

// logits: [M, ld] bf16 (ld >= Vpad, Vpad % 8 == 0), overwritten with the gradient when write_grad != 0.
// targets: int64 [M]; loss: fp32 [M]; weights: optional device fp32[n_predict]; scale_ptr: optional device scalar
// multiplied into the gradient (e.g. 1 / number of valid tokens).
extern "C" int sr_softcap_ce(void* logits, const long* targets, float* loss, const float* weights, int n_predict,
                             const float* scale_ptr, long M, int Vpad, int V, long ld, float cap, int write_grad,
                             cudaStream_t s) {
  if (M <= 0) return 0;
  if (Vpad % 8 || ld % 8 || n_predict < 1 || n_predict > kMaxPredict || V > Vpad) return -2;
  softcap_ce_kernel<<<(unsigned)M, kThreads, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(logits), targets, loss, weights,
                                                     n_predict, scale_ptr, M, Vpad, V, ld, cap, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
