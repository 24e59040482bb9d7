// lm-head GEMM fused with the tanh-soft-capped cross-entropy (forward and the producer half of the backward).
//
// The logits never reach memory. The CTA-pair tcgen05 GEMM (gemm_pair_kernel.cuh) computes 256 x 256 tiles of
// x W^T in TMEM; its epilogue warps turn each accumulator row chunk, in registers, into
//     t = tanh(l / cap),  z = cap * t,  e = exp(z - cap)            (|z| <= cap, so cap serves as the row maximum)
// and keep three things: the tile's partial row sum of e, the soft-capped logit at the row's target columns, and
//     E[r, v] = e * (1 - t^2)      (bf16)
// the gradient of the loss with respect to the raw logit up to a per-row factor. A second, row-wise kernel sums the
// partials in a fixed order, forms lse = cap + log(sum), the loss, the per-row factor
//     rscale[r] = scale * S_w / sum[r]        (S_w = sum of the row's target weights, scale = 1 / #tokens)
// and rewrites the (at most four) target entries of the row to E' = (1 - t^2) (e - sum * w / S_w), so that
//     dL/dlogits = diag(rscale) E'   exactly as softmax-minus-onehot requires.
// The backward is then two plain GEMMs on E': dx = diag(rscale) (E' W) with the row factor applied in the GEMM
// epilogue, and dW += E'^T (diag(rscale) x) with the pre-scaled activations written by the same row-wise kernel.
// Against a GEMM + separate loss kernel this removes one full read and one full write of the [tokens, vocab]
// tensor per head, and the special-function work (2 per logit) runs under the tensor pipe of the next tile.
//
// Operands may be bf16 or fp8 (e4m3, per-tensor scales folded into alpha; kind::f8f6f4 at twice the bf16 rate).
// The multi-token form scores row i against targets[i + k], k < n_predict, over the flattened batch.
//
// Reference counterparts: bf16 head + fp32 softcap + F.cross_entropy through Inductor (train.py:558-568); the tiny
// track's fp8 _scaled_mm + one-CTA-per-row loss kernel + fp8 backward GEMMs (tiny/cuda_kernels.py:125-414).
#include "gemm_pair_kernel.cuh"

namespace {

constexpr int kMaxPredict = 4;

__device__ __forceinline__ float tanh_approx(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}

struct EpiCE {
  struct Row {
    float sum;
    int tgt[kMaxPredict];
  };
  static __device__ __forceinline__ void begin(Row& st, const GemmParams& p, int r, bool row_ok) {
    st.sum = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPredict; ++k) {
      st.tgt[k] = -1;
      if (row_ok && k < p.ce.n_predict && (long)r + k < p.M) {
        const long y = p.ce.targets[r + k];
        if (y >= 0 && y < p.ce.V) st.tgt[k] = (int)y;
      }
    }
  }
  template <int BN>
  static __device__ __forceinline__ void chunk(Row& st, const GemmParams& p, float (&f)[32], int r, int c0, bool,
                                               uint8_t* cbase, const uint8_t*) {
    const float cap = p.ce.cap, inv_cap = p.ce.inv_cap;
    const int V = p.ce.V;
    // target logits: rare (a chunk holds a given row's target with probability 32 / vocab), so off the main path
#pragma unroll
    for (int k = 0; k < kMaxPredict; ++k) {
      const unsigned d = (unsigned)(st.tgt[k] - c0);
      if (st.tgt[k] >= 0 && d < 32u) {
        float l = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) l = (d == (unsigned)j) ? f[j] : l;
        p.ce.ztgt[(size_t)r * kMaxPredict + k] = cap * tanh_approx(l * inv_cap);
      }
    }
    __nv_bfloat16* dst = p.C ? reinterpret_cast<__nv_bfloat16*>(cbase) + (size_t)r * p.ldc + c0 : nullptr;
    float s = 0.f;
    if (c0 + 32 <= V) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float t = tanh_approx(f[j] * inv_cap);
        const float e = __expf(cap * t - cap);
        s += e;
        f[j] = e * (1.f - t * t);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float t = tanh_approx(f[j] * inv_cap);
        const float e = (c0 + j < V) ? __expf(cap * t - cap) : 0.f;
        s += e;
        f[j] = e * (1.f - t * t);
      }
    }
    st.sum += s;
    if (dst != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[j + 2 * e], f[j + 2 * e + 1]);
        *reinterpret_cast<uint4*>(dst + j) = o;
      }
    }
  }
  static __device__ __forceinline__ void end(Row& st, const GemmParams& p, int r, bool row_ok, int nj) {
    if (row_ok) p.ce.partials[(size_t)nj * p.M + r] = st.sum;
  }
};

// scale = 1 / max(#targets >= 0, 1), or 1 / M when `mean_over_rows`
__global__ void ce_scale_kernel(const long* __restrict__ targets, long M, int mean_over_rows, float* __restrict__ scale) {
  __shared__ int red[32];
  if (mean_over_rows) {
    if (threadIdx.x == 0) *scale = 1.f / (float)M;
    return;
  }
  int n = 0;
  for (long i = threadIdx.x; i < M; i += blockDim.x) n += targets[i] >= 0 ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = n;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    *scale = 1.f / (float)(t > 0 ? t : 1);
  }
}

// One warp per row. See the file header for what it forms.
__global__ void __launch_bounds__(256)
ce_finish_kernel(const float* __restrict__ partials, int tiles_n, const float* __restrict__ ztgt,
                 const long* __restrict__ targets, const float* __restrict__ weights, int n_predict, int V, float cap,
                 const float* __restrict__ scale_ptr, long M, float* __restrict__ loss_rows, float* __restrict__ rscale,
                 __nv_bfloat16* __restrict__ E, long ldE, const __nv_bfloat16* __restrict__ X, long ldx, int D,
                 __nv_bfloat16* __restrict__ Xs) {
  const int lane = threadIdx.x & 31;
  const long r = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= M) return;
  float s = 0.f;
  for (int j = lane; j < tiles_n; j += 32) s += partials[(size_t)j * M + r];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  float rs = 0.f;
  if (lane == 0) {
    const float lse = cap + logf(s);
    int tg[kMaxPredict];
    float w[kMaxPredict];
    float sw = 0.f, loss = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPredict; ++k) {
      tg[k] = -1;
      w[k] = 0.f;
      if (k < n_predict && r + k < M) {
        const long y = targets[r + k];
        const float wk = weights ? weights[k] : 1.f;
        if (y >= 0 && y < V && wk != 0.f) {
          tg[k] = (int)y;
          w[k] = wk;
          sw += wk;
          loss += wk * (lse - ztgt[(size_t)r * kMaxPredict + k]);
        }
      }
    }
    loss_rows[r] = loss;
    const float scale = scale_ptr ? *scale_ptr : 1.f;
    rs = sw != 0.f ? scale * sw / s : 0.f;
    if (rscale) rscale[r] = rs;
    if (E != nullptr && sw != 0.f) {
#pragma unroll
      for (int k = 0; k < kMaxPredict; ++k) {
        if (tg[k] < 0) continue;
        float wsum = 0.f;
#pragma unroll
        for (int k2 = 0; k2 < kMaxPredict; ++k2) wsum += (tg[k2] == tg[k]) ? w[k2] : 0.f;
        const float z = ztgt[(size_t)r * kMaxPredict + k];
        const float t = z / cap;
        const float e = __expf(z - cap);
        E[(size_t)r * ldE + tg[k]] = __float2bfloat16((1.f - t * t) * (e - s * (wsum / sw)));
      }
    }
  }
  if (Xs == nullptr) return;
  rs = __shfl_sync(0xffffffffu, rs, 0);
  const __nv_bfloat16* x = X + (size_t)r * ldx;
  __nv_bfloat16* xs = Xs + (size_t)r * D;
  for (int j = lane * 8; j < D; j += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + j);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      oh[e] = __floats2bfloat162_rn(v.x * rs, v.y * rs);
    }
    *reinterpret_cast<uint4*>(xs + j) = o;
  }
}

// loss = scale * sum(loss_rows), summed in a fixed order by one block
__global__ void ce_sum_kernel(const float* __restrict__ loss_rows, long M, const float* __restrict__ scale_ptr,
                              float* __restrict__ out) {
  __shared__ float red[32];
  float a = 0.f;
  for (long i = threadIdx.x; i < M; i += blockDim.x) a += loss_rows[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    *out = t * (scale_ptr ? *scale_ptr : 1.f);
  }
}

// ---------------------------------------------------------------- fp8 quantisation (per-tensor scale)
__device__ __forceinline__ uint16_t cvt_fp8x2(float lo, float hi, int e5m2) {
  uint16_t r;
  if (e5m2) asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  else      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// out[i] = fp8(x[i] * inv_scale); rows of `cols` elements, source row stride ldx, destination row stride ldo
__global__ void quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, long rows, int cols,
                                 long ldx, long ldo, float inv_scale, int e5m2) {
  const int cpr = cols / 8;   // 8-element groups per row
  const long total = rows * cpr;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cpr;
    const int c = (int)(i - r * cpr) * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint16_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      o[e] = cvt_fp8x2(v.x * inv_scale, v.y * inv_scale, e5m2);
    }
    *reinterpret_cast<uint2*>(out + r * ldo + c) = make_uint2((uint32_t)o[0] | ((uint32_t)o[1] << 16),
                                                              (uint32_t)o[2] | ((uint32_t)o[3] << 16));
  }
}

// out[c, r] = fp8(x[r, c] * inv_scale): quantise and transpose through a 64 x 64 shared-memory tile
__global__ void quant_fp8_t_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, int rows, int cols,
                                   long ldx, long ldo, float inv_scale, int e5m2) {
  __shared__ uint8_t tile[64][65];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) {
    const int rr = i / 32, cc = (i % 32) * 2;
    float a = 0.f, b = 0.f;
    if (r0 + rr < rows) {
      if (c0 + cc < cols) a = __bfloat162float(x[(size_t)(r0 + rr) * ldx + c0 + cc]);
      if (c0 + cc + 1 < cols) b = __bfloat162float(x[(size_t)(r0 + rr) * ldx + c0 + cc + 1]);
    }
    const uint16_t q = cvt_fp8x2(a * inv_scale, b * inv_scale, e5m2);
    tile[rr][cc] = (uint8_t)(q & 0xff);
    tile[rr][cc + 1] = (uint8_t)(q >> 8);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
    const int cc = i / 64, rr = i % 64;
    if (c0 + cc < cols && r0 + rr < rows) out[(size_t)(c0 + cc) * ldo + r0 + rr] = tile[rr][cc];
  }
}

// out[r, c] = fp8(x[r, c] * f_r) and out_t[c, r] = the same value, f_r = row_scale[r] * mult / *div_ptr: the logit
// gradient of the fused head in both operand layouts its two fp8 backward products need (K-major for each).
// One CTA converts a 64-row x 128-column tile: 16-byte loads, 8-byte stores of the row-major copy, and the transposed
// copy through shared memory (bytes stored column-major with a per-column rotation that keeps the 16 lanes of a row on
// 16 different banks) written back as 16-byte pieces of 16 consecutive rows. cols % 8 == 0.
constexpr int kQR = 64, kQC = 128;
__global__ void __launch_bounds__(256)
quant_fp8_dual_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ row_scale,
                      const float* __restrict__ div_ptr, float mult, uint8_t* __restrict__ out,
                      uint8_t* __restrict__ out_t, int rows, int cols, long ldx, long ldo, long ldt, int e5m2) {
  __shared__ __align__(16) uint8_t T[kQC * kQR];       // [column][row], row index rotated by 4 * ((column >> 3) & 15)
  const int r0 = blockIdx.y * kQR, c0 = blockIdx.x * kQC;
  const float m = mult / (div_ptr ? *div_ptr : 1.f);
#pragma unroll
  for (int it = 0; it < (kQR * kQC / 8) / 256; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int rr = idx >> 4, cg = idx & 15;
    const int r = r0 + rr, c = c0 + cg * 8;
    uint32_t lo = 0, hi = 0;
    if (r < rows && c < cols) {
      const float f = (row_scale ? row_scale[r] : 1.f) * m;
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)r * ldx + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      uint16_t q[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 v = __bfloat1622float2(h[e]);
        q[e] = cvt_fp8x2(v.x * f, v.y * f, e5m2);
      }
      lo = (uint32_t)q[0] | ((uint32_t)q[1] << 16);
      hi = (uint32_t)q[2] | ((uint32_t)q[3] << 16);
      *reinterpret_cast<uint2*>(out + (size_t)r * ldo + c) = make_uint2(lo, hi);
    }
    const int rot = 4 * (cg & 15);
#pragma unroll
    for (int jb = 0; jb < 8; ++jb) {
      const uint32_t w = jb < 4 ? lo : hi;
      T[(cg * 8 + jb) * kQR + ((rr + rot) & (kQR - 1))] = (uint8_t)(w >> (8 * (jb & 3)));
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < (kQR * kQC / 16) / 256; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int cc = idx >> 2, seg = idx & 3;
    const int c = c0 + cc, r = r0 + seg * 16;
    if (c >= cols || r >= rows) continue;
    const int rot = 4 * ((cc >> 3) & 15);
    uint32_t w[4];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4)
      w[q4] = *reinterpret_cast<const uint32_t*>(&T[cc * kQR + ((seg * 16 + q4 * 4 + rot) & (kQR - 1))]);
    uint8_t* dst = out_t + (size_t)c * ldt + r;
    if (r + 16 <= rows) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int b = 0; b < 16 && r + b < rows; ++b) dst[b] = (uint8_t)(w[b >> 2] >> (8 * (b & 3)));
    }
  }
}

inline int last_rc() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }

}  // namespace

// Forward of the fused head. X [M, K] and W [N, K] are both K-major: bf16 (fp8 = 0) or fp8 e4m3 (fp8 = 1, lda/ldb in
// bytes); with b_mn = 1 (bf16 only) W is stored [K, N]. `alpha` multiplies the accumulator (the product of the
// per-tensor scales for fp8 operands).
//   E         bf16 [M, ldE >= N] or null (loss only): receives E' (see the file header); columns V..N-1 are zero
//   targets   int64 [M], -1 = ignored;  weights: optional device fp32 [n_predict];  n_predict <= 4
//   V         columns that enter the softmax (<= N);  cap > 0
//   scale_ptr device fp32 scalar written here: 1 / #valid targets, or 1 / M when mean_over_rows
//   partials  fp32 scratch [ceil(N / 256), M];  ztgt: fp32 scratch [M, 4]
//   loss_rows fp32 [M];  loss: optional device fp32 scalar = scale * sum(loss_rows)
//   rscale    fp32 [M] or null;  Xs: bf16 [M, K] or null, receives rscale[r] * Xsrc[r, :] where Xsrc (bf16 [M, ldxs]) is
//             the activation matrix in bf16 (= X when fp8 = 0)
extern "C" int sr_lmhead_ce_fwd(const void* X, const void* W, void* E, long long ldE, int M, int N, int K, long long lda,
                                long long ldb, int b_mn, int fp8, float alpha, const long* targets, const float* weights,
                                int n_predict, int V, float cap, int mean_over_rows, float* scale_ptr, float* partials,
                                float* ztgt, float* loss_rows, float* loss, float* rscale, const void* Xsrc,
                                long long ldxs, void* Xs, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (cap <= 0.f || n_predict < 1 || n_predict > kMaxPredict || V > N || N % 32 != 0 || K % 8 != 0) return -2;
  if (fp8 && b_mn) return -2;
  if (E != nullptr && (ldE % 8 != 0 || ldE < N)) return -2;
  constexpr int BN = 256;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.a_mn = 0; p.b_mn = b_mn;
  p.C = E; p.ldc = ldE; p.strideC = 0; p.c_fp32 = 0;
  p.alpha = alpha; p.beta = 0.f; p.status = status;
  p.ce.targets = targets; p.ce.partials = partials; p.ce.ztgt = ztgt;
  p.ce.n_predict = n_predict; p.ce.V = V; p.ce.cap = cap; p.ce.inv_cap = 1.f / cap;
  ce_scale_kernel<<<1, 1024, 0, stream>>>(targets, M, mean_over_rows, scale_ptr);
  CUtensorMap ma, mb;
  int rc;
  if (fp8) {
    rc = encode_u8_map(&ma, X, K, M, 1, lda, 0, 128, BM);
    if (rc) return rc;
    rc = encode_u8_map(&mb, W, K, N, 1, ldb, 0, 128, BN / 2);
    if (rc) return rc - 10;
    rc = launch_pair<BN, 1, EpiCE>(ma, mb, p, max_ctas, 0, stream);
  } else {
    rc = encode_bf16_map(&ma, X, K, M, 1, lda, 0, BK, BM);
    if (rc) return rc;
    if (!b_mn) rc = encode_bf16_map(&mb, W, K, N, 1, ldb, 0, BK, BN / 2);
    else       rc = encode_bf16_map(&mb, W, N, K, 1, ldb, 0, 64, BK);
    if (rc) return rc - 10;
    rc = launch_pair<BN, 2, EpiCE>(ma, mb, p, max_ctas, 0, stream);
  }
  if (rc) return rc;
  const int tiles_n = (N + BN - 1) / BN;
  ce_finish_kernel<<<(unsigned)((M + 7) / 8), 256, 0, stream>>>(
      partials, tiles_n, ztgt, targets, weights, n_predict, V, cap, scale_ptr, M, loss_rows, rscale,
      reinterpret_cast<__nv_bfloat16*>(E), ldE, reinterpret_cast<const __nv_bfloat16*>(Xsrc), ldxs, K,
      reinterpret_cast<__nv_bfloat16*>(Xs));
  if (loss != nullptr) ce_sum_kernel<<<1, 1024, 0, stream>>>(loss_rows, M, scale_ptr, loss);
  return last_rc();
}

// out = fp8(x / scale) for a bf16 matrix [rows, cols] (cols % 8 == 0); transpose = 1 writes out[cols, rows].
// e5m2 = 0: e4m3 (saturating at 448), 1: e5m2.
extern "C" int sr_quant_fp8(const void* x, void* out, long rows, int cols, long ldx, long ldo, float scale,
                            int transpose, int e5m2, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (scale <= 0.f) return -2;
  const float inv = 1.f / scale;
  if (!transpose) {
    if (cols % 8 || ldx % 8 || ldo % 8) return -2;
    const long total = rows * (cols / 8);
    long blocks = (total + 255) / 256;
    const long cap = (long)num_sms() * 8;
    if (blocks > cap) blocks = cap;
    quant_fp8_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                           reinterpret_cast<uint8_t*>(out), rows, cols, ldx, ldo, inv, e5m2);
  } else {
    dim3 grid((cols + 63) / 64, (unsigned)((rows + 63) / 64));
    quant_fp8_t_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(out),
                                                 (int)rows, cols, ldx, ldo, inv, e5m2);
  }
  return last_rc();
}

// out [rows, ldo] and out_t [cols, ldt] (both fp8) = x[r, c] * row_scale[r] * mult / (*div_ptr), row_scale and div_ptr
// optional. cols, ldx and ldo must be multiples of 8, ldt a multiple of 16, all base pointers 16-byte aligned.
extern "C" int sr_quant_fp8_dual(const void* x, const float* row_scale, const float* div_ptr, float mult, void* out,
                                 void* out_t, long rows, int cols, long ldx, long ldo, long ldt, int e5m2,
                                 cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 || ldx % 8 || ldo % 8 || ldt % 16) return -2;
  dim3 grid((cols + kQC - 1) / kQC, (unsigned)((rows + kQR - 1) / kQR));
  quant_fp8_dual_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), row_scale, div_ptr, mult,
                                                  reinterpret_cast<uint8_t*>(out), reinterpret_cast<uint8_t*>(out_t),
                                                  (int)rows, cols, ldx, ldo, ldt, e5m2);
  return last_rc();
}
