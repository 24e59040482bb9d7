// Gated delta rule (linear attention with a decayed, error-correcting fast-weight state), forward recurrence.
//
// Per head the state S is a [Dk x Dv] matrix and every token does
//     S <- diag(exp(g_t)) S                 decay (one log-decay per head, or one per key channel)
//     r  = v_t - S^T k_t                    what the state does not yet predict for this key
//     S <- S + beta_t k_t r^T               delta-rule write
//     o_t = S^T q_t
// With a scalar log-decay this is the Gated DeltaNet layer, with a per-key-channel log-decay it is Kimi Delta
// Attention (the research/hybrid_attn fork of the reference calls flash-linear-attention's Triton kernels for both,
// research/hybrid_attn/train.py:459-468, 612-628).
//
// Work split: one warp owns kChan value channels of one (batch, head); its lanes split the key dimension
// (lane l holds key channels l, l + 32, ...), so the two contractions over keys per token (S^T k and S^T q) are warp
// reductions and nothing crosses warps. The state lives in registers in fp32 for the whole sequence; inputs of the
// next token are fetched while the current one is processed. Optionally the state is saved every `ckpt_every` tokens
// (before the token is applied), which is what a chunk-wise backward restarts from.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kChan = 2;           // value channels per warp
constexpr int kWarpsPerBlock = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int KPL, bool VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gated_delta_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                       const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                       __nv_bfloat16* __restrict__ o, float* __restrict__ ckpt, int T, int H, int Dv, int ckpt_every) {
  constexpr int Dk = KPL * 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int bh = blockIdx.x;
  const int b = bh / H, h = bh - b * H;
  const int c0 = (blockIdx.y * kWarpsPerBlock + warp) * kChan;     // first value channel of this warp
  if (c0 >= Dv) return;
  const long tok0 = (long)b * T;
  float s[kChan][KPL];
#pragma unroll
  for (int c = 0; c < kChan; ++c)
#pragma unroll
    for (int i = 0; i < KPL; ++i) s[c][i] = 0.f;

  // registers holding the inputs of the token being processed and of the next one
  float kk[KPL], qq[KPL], dd[KPL], vv[kChan], bb;
  auto load = [&](int t, float (&K)[KPL], float (&Q)[KPL], float (&D)[KPL], float (&V)[kChan], float& B) {
    const long row = (tok0 + t) * H + h;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      K[i] = __bfloat162float(k[row * Dk + lane + 32 * i]);
      Q[i] = __bfloat162float(q[row * Dk + lane + 32 * i]);
      D[i] = VEC ? __expf(g[row * Dk + lane + 32 * i]) : 0.f;
    }
    if (!VEC) {
      const float d = __expf(g[row]);
#pragma unroll
      for (int i = 0; i < KPL; ++i) D[i] = d;
    }
#pragma unroll
    for (int c = 0; c < kChan; ++c) V[c] = (c0 + c < Dv) ? __bfloat162float(v[row * Dv + c0 + c]) : 0.f;
    B = beta[row];
  };
  load(0, kk, qq, dd, vv, bb);
  const int n_ck = ckpt_every > 0 ? (T + ckpt_every - 1) / ckpt_every : 0;
  for (int t = 0; t < T; ++t) {
    float nk[KPL], nq[KPL], nd[KPL], nv[kChan], nb = 0.f;
    if (t + 1 < T) load(t + 1, nk, nq, nd, nv, nb);
    if (ckpt != nullptr && t % ckpt_every == 0) {
      // [B, H, n_ck, Dv, Dk]
      float* dst = ckpt + ((((long)bh * n_ck + t / ckpt_every) * Dv + c0) * Dk);
#pragma unroll
      for (int c = 0; c < kChan; ++c)
        if (c0 + c < Dv)
#pragma unroll
          for (int i = 0; i < KPL; ++i) dst[(long)c * Dk + lane + 32 * i] = s[c][i];
    }
    float u[kChan];
#pragma unroll
    for (int c = 0; c < kChan; ++c) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        s[c][i] *= dd[i];
        a += s[c][i] * kk[i];
      }
      u[c] = a;
    }
#pragma unroll
    for (int c = 0; c < kChan; ++c) u[c] = warp_sum(u[c]);
    float out[kChan];
#pragma unroll
    for (int c = 0; c < kChan; ++c) {
      const float r = bb * (vv[c] - u[c]);
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        s[c][i] += kk[i] * r;
        a += s[c][i] * qq[i];
      }
      out[c] = a;
    }
#pragma unroll
    for (int c = 0; c < kChan; ++c) out[c] = warp_sum(out[c]);
    if (lane == 0) {
      const long row = (tok0 + t) * H + h;
#pragma unroll
      for (int c = 0; c < kChan; ++c)
        if (c0 + c < Dv) o[row * Dv + c0 + c] = __float2bfloat16(out[c]);
    }
    if (t + 1 < T) {
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        kk[i] = nk[i];
        qq[i] = nq[i];
        dd[i] = nd[i];
      }
#pragma unroll
      for (int c = 0; c < kChan; ++c) vv[c] = nv[c];
      bb = nb;
    }
  }
}

}  // namespace

// q, k: bf16 [B, T, H, Dk] (already normalised / scaled by the caller), v, o: bf16 [B, T, H, Dv],
// g: fp32 log-decay [B, T, H] (vec_decay = 0) or [B, T, H, Dk] (vec_decay = 1), beta: fp32 [B, T, H].
// ckpt: optional fp32 [B, H, ceil(T / ckpt_every), Dv, Dk], receives the state before tokens 0, ckpt_every, ...
// Dk must be 64 or 128. Returns 0, -2 for unsupported sizes, -5 for a launch failure.
extern "C" int sr_gated_delta_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o,
                                  float* ckpt, int B, int T, int H, int Dk, int Dv, int vec_decay, int ckpt_every,
                                  cudaStream_t s) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  if ((Dk != 64 && Dk != 128) || Dv <= 0) return -2;
  if (ckpt != nullptr && ckpt_every <= 0) return -2;
  dim3 grid(B * H, (Dv + kWarpsPerBlock * kChan - 1) / (kWarpsPerBlock * kChan));
  const int threads = kWarpsPerBlock * 32;
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto K = reinterpret_cast<const __nv_bfloat16*>(k);
  auto V = reinterpret_cast<const __nv_bfloat16*>(v);
  auto O = reinterpret_cast<__nv_bfloat16*>(o);
  if (Dk == 64) {
    if (vec_decay) gated_delta_fwd_kernel<2, true><<<grid, threads, 0, s>>>(Q, K, V, g, beta, O, ckpt, T, H, Dv, ckpt_every);
    else           gated_delta_fwd_kernel<2, false><<<grid, threads, 0, s>>>(Q, K, V, g, beta, O, ckpt, T, H, Dv, ckpt_every);
  } else {
    if (vec_decay) gated_delta_fwd_kernel<4, true><<<grid, threads, 0, s>>>(Q, K, V, g, beta, O, ckpt, T, H, Dv, ckpt_every);
    else           gated_delta_fwd_kernel<4, false><<<grid, threads, 0, s>>>(Q, K, V, g, beta, O, ckpt, T, H, Dv, ckpt_every);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
