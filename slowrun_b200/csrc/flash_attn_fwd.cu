// Flash attention forward for sm_100a: causal with a left sliding window, head_dim 128, bf16, (B, T, H, D) layout.
//
// One CTA per (batch*head, 128-query tile). Warp roles (192 threads):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles (128 keys) through a 2-stage ring
//   warp 1      MMA issuer + TMEM owner:  S_j = Q K_j^T   (SS, both operands K-major, accumulator in TMEM)
//                                          O  += P_j V_j   (SS, P from shared memory, V_j as an MN-major operand)
//   warps 2..5  softmax: thread i owns query row i (TMEM lane i), so row max / row sum need no shuffles. They read
//               S_j from TMEM, apply scale + mask, keep running (m, l), rescale O in TMEM when the max moved,
//               write P_j (bf16) into shared memory in the 128B-swizzled K-major layout, and at the end write
//               O / l and the log-sum-exp.
// S is double buffered in TMEM so S_{j+1} is computed while the softmax of tile j runs.
// Keys visible to query i: max(0, i - window) <= k <= i  (window < 0 means unlimited), the convention of
// flash_attn's window_size=(window, 0) that the reference uses (train.py:211-213, 432-438).
#include "sm100_common.cuh"

namespace {

using namespace sr;

constexpr int BQ = 128, D = 128;
constexpr int kThreads = 192;
constexpr uint32_t kQBytes = BQ * D * 2;           // 32 KB
constexpr uint32_t kQHalf = BQ * 128;              // one 64-column half of a 128-row tile: 128 rows x 128 B

// BKV = keys per tile. 128: one CTA per SM; 64: two CTAs per SM (their softmax and MMA phases overlap).
template <int BKV>
struct FwdCfg {
  static constexpr uint32_t kKVBytes = BKV * D * 2;       // K or V tile
  static constexpr uint32_t kKVHalf = BKV * 128;          // 64 d-columns of a K/V tile
  static constexpr uint32_t kPBytes = BQ * BKV * 2;
  static constexpr uint32_t kTmemCols = (BKV == 128) ? 512 : 256;   // 2 S buffers + O
  static constexpr int kSmemBytes = kQBytes + 4 * kKVBytes + kPBytes + 256;
};

struct FwdParams {
  __nv_bfloat16* out;   // [B, T, H, D]
  float* lse;           // [B, H, T]
  int B, T, H;
  int window;           // < 0: unlimited
  float scale_log2;     // softmax scale * log2(e)
  int* status;
};

template <int BKV>
__device__ __forceinline__ void kv_range(int q0, int T, int window, int& j_lo, int& j_hi) {
  const int q_last = min(q0 + BQ - 1, T - 1);
  j_hi = q_last / BKV;
  j_lo = (window < 0) ? 0 : max(0, q0 - window) / BKV;
}

template <int BKV>
__global__ void __launch_bounds__(kThreads, (BKV == 64) ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
  using C_ = FwdCfg<BKV>;
  constexpr uint32_t kKVBytes = C_::kKVBytes, kKVHalf = C_::kKVHalf;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kQBytes;                       // 2 stages
  uint8_t* sV = sK + 2 * kKVBytes;                    // 2 stages
  uint8_t* sP = sV + 2 * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C_::kPBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* v_full = bars + 3;        // 2
  uint64_t* kv_empty = bars + 5;      // 2
  uint64_t* s_full = bars + 7;        // 2
  uint64_t* p_full = bars + 9;        // 1 (count 128)
  uint64_t* pv_done = bars + 10;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + BQ - 1) / BQ;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);   // heavy (late) tiles first
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh - b * p.H;
  const int q0 = qt * BQ;
  int j_lo, j_hi;
  kv_range<BKV>(q0, p.T, p.window, j_lo, j_hi);
  const int n_kv = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    if ((smem_u32(smem) & 1023u) != 0u) report_error(p.status, SR_ERR_BAD_ARG, 1000, 0);   // swizzle needs 1 KB alignment
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C_::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;          // two buffers of BKV columns
  const uint32_t tmem_O = tmem_base + 2 * BKV;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, kQBytes);
      tma_load_4d(sQ, &map_q, q_full, 0, h, q0, b);
      tma_load_4d(sQ + kQHalf, &map_q, q_full, 64, h, q0, b);
      for (int it = 0; it < n_kv; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1u;
        if (!mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, p.status, 1100)) break;
        const int k0 = (j_lo + it) * BKV;
        mbar_arrive_expect_tx(&k_full[st], kKVBytes);
        tma_load_4d(sK + st * kKVBytes, &map_k, &k_full[st], 0, h, k0, b);
        tma_load_4d(sK + st * kKVBytes + kKVHalf, &map_k, &k_full[st], 64, h, k0, b);
        mbar_arrive_expect_tx(&v_full[st], kKVBytes);
        tma_load_4d(sV + st * kKVBytes, &map_v, &v_full[st], 0, h, k0, b);
        tma_load_4d(sV + st * kKVBytes + kKVHalf, &map_v, &v_full[st], 64, h, k0, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(1, 1, 0, 0, BQ, BKV);   // Q (K-major) x K_j (K-major)
      const uint32_t idesc_o = make_idesc(1, 1, 0, 1, BQ, D);     // P (K-major) x V_j (MN-major)
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 1200);
      auto issue_s = [&](int it) {
        const int st = it & 1;
        const uint32_t aK = smem_u32(sK + st * kKVBytes);
        const uint32_t d = tmem_S + static_cast<uint32_t>((it & 1) * BKV);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qoff = (k >> 2) * kQHalf + (k & 3) * 32;
          const uint32_t koff = (k >> 2) * kKVHalf + (k & 3) * 32;
          umma_f16_ss(d, make_smem_desc_sw128(aQ + qoff, 16, 1024), make_smem_desc_sw128(aK + koff, 16, 1024), idesc_s,
                      k != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[it & 1]);
      };
      if (ok) {
        ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, 1201);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
      }
      for (int it = 0; it < n_kv && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1u;
        if (it + 1 < n_kv) {
          ok = mbar_wait(&k_full[(it + 1) & 1], ((it + 1) >> 1) & 1u, abort_flag, p.status, 1202);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        ok = mbar_wait(p_full, it & 1u, abort_flag, p.status, 1203);
        if (!ok) break;
        ok = mbar_wait(&v_full[st], ph, abort_flag, p.status, 1204);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + st * kKVBytes);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P: K-major over keys (64-key halves of 128 rows); B = V_j: [key rows x d], d contiguous -> MN-major,
          // its two 64-column groups kKVHalf apart
          const uint64_t adesc = make_smem_desc_sw128(aP + (k >> 2) * kQHalf + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(aV + k * (16 * 128), kKVHalf, 1024);
          umma_f16_ss(tmem_O, adesc, bdesc, idesc_o, (it | k) != 0 ? 1u : 0u);
        }
        tc_commit(pv_done);
        tc_commit(&kv_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;               // row inside the tile == TMEM lane
    const int qg = q0 + r;                     // global query index
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_kv; ++it) {
      ok = mbar_wait(&s_full[it & 1], (it >> 1) & 1u, abort_flag, p.status, 1300);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tS = tmem_S + lane_addr + static_cast<uint32_t>((it & 1) * BKV);
      const int k0 = (j_lo + it) * BKV;
      const int k_hi = min(qg, p.T - 1);                              // last visible key
      const int k_lo = (p.window < 0) ? 0 : max(0, qg - p.window);    // first visible key
      const bool need_mask = (k0 + BKV - 1 > k_hi) || (k0 < k_lo);
      // The S row is read from TMEM once and stays in registers for both the maximum and the exponentials.
      uint32_t sv[BKV];
#pragma unroll
      for (int ch = 0; ch < BKV / 32; ++ch)
        tmem_ld_32x32(tS + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(sv + ch * 32));
      tc_wait_ld();
      // four independent running maxima (and sums below): one dependent chain of 64 would expose its latency, with only
      // two softmax warps per scheduler there is nothing else to issue meanwhile
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < BKV; ++j) {
          const int kg = k0 + j;
          if (!(kg <= k_hi && kg >= k_lo)) sv[j] = __float_as_uint(-INFINITY);
          mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sv[j]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < BKV; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sv[j]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Lazy reference maximum: the reference point of the exponentials only moves when the row maximum has grown by
      // more than 2^kLazyLog2 since it was set. In between, probabilities are at most 2^kLazyLog2 (exact in bf16's
      // range), alpha is exactly 1 and O needs no rescaling; l and the log-sum-exp use the same reference, so the
      // result is unchanged.
      constexpr float kLazyLog2 = 8.f;
      const float m_cand = fmaxf(m, mx * p.scale_log2);
      const float m_new = (m == -INFINITY || m_cand - m > kLazyLog2) ? m_cand : m;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
      // probabilities, packed to bf16 (masked entries are -inf -> 0)
      uint32_t pk[BKV / 2];
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < BKV; j += 2) {
        const float e0 = exp2f(fmaf(__uint_as_float(sv[j]), p.scale_log2, -m_use));
        const float e1 = exp2f(fmaf(__uint_as_float(sv[j + 1]), p.scale_log2, -m_use));
        const __nv_bfloat162 pb = __floats2bfloat162_rn(e0, e1);
        const float2 back = __bfloat1622float2(pb);      // the sum uses the rounded values the PV product will see
        rs4[(j >> 1) & 3] += back.x + back.y;
        pk[j / 2] = *reinterpret_cast<const uint32_t*>(&pb);
      }
      const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      l = l * alpha + rs;
      m = m_new;
      // O and the P buffer are free once the previous P V product has completed
      if (it > 0) {
        ok = mbar_wait(pv_done, (it - 1) & 1u, abort_flag, p.status, 1301);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (!__all_sync(0xffffffffu, alpha == 1.f)) {
          const uint32_t tO = tmem_O + lane_addr;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t v[32];
            tmem_ld_32x32(tO + ch * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st_32x32(tO + ch * 32, v);
          }
          tc_wait_st();
        }
      }
      // P row -> shared memory (K-major, 128B swizzle): 16 chunks of 8 keys
#pragma unroll
      for (int c = 0; c < BKV / 8; ++c) {
        const uint32_t off = sw128_offset(r, c * 8, kQHalf);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok) {
      ok = mbar_wait(pv_done, (n_kv - 1) & 1u, abort_flag, p.status, 1302);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      const uint32_t tO = tmem_O + lane_addr;
      const bool row_ok = qg < p.T;
      __nv_bfloat16* orow = p.out + (((size_t)b * p.T + (row_ok ? qg : 0)) * p.H + h) * D;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32(tO + ch * 32, v);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 t;
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              hh[e] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * e]) * inv, __uint_as_float(v[j + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(orow + ch * 32 + j) = t;
          }
        }
      }
      if (row_ok) p.lse[((size_t)b * p.H + h) * p.T + qg] = (l > 0.f) ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C_::kTmemCols);
  }
}

}  // namespace

namespace sr_attn {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

extern "C" void* sr_driver_encode_tiled(void);   // process-wide handle, gemm_tcgen05.cu

EncodeTiledFn encode_fn() {
  // a driver-API call: the device's context must be current on this thread (see gemm_common.cuh)
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  return reinterpret_cast<EncodeTiledFn>(sr_driver_encode_tiled());
}

// (B, T, H, 128) bf16 tensor with row stride `ld_t` elements between tokens (the head h slice starts at h*128);
// box = 64 columns x `rows` tokens of one head, 128B swizzle, zero fill past T.
int encode_bthd(CUtensorMap* map, const void* ptr, int B, int T, int H, long ld_t, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld_t % 8) != 0) return -2;
  cuuint64_t dims[4] = {128, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {128 * 2, (cuuint64_t)ld_t * 2, (cuuint64_t)ld_t * 2 * (cuuint64_t)T};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Contiguous (B, T, H, 128) fp32 tensor; box = 32 columns (128 B) x `rows` tokens of one head, 128B swizzle. Used for the
// bulk reduce-add of dQ tiles from shared memory.
int encode_bthd_f32(CUtensorMap* map, const void* ptr, int B, int T, int H, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return -2;
  cuuint64_t dims[4] = {128, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {128 * 4, (cuuint64_t)H * 128 * 4, (cuuint64_t)H * 128 * 4 * (cuuint64_t)T};
  cuuint32_t box[4] = {32, 1, (cuuint32_t)rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace sr_attn

// q, k, v: (B, T, H, 128) bf16 with token stride ld_* elements (contiguous tensors: H*128); out contiguous;
// lse: fp32 (B, H, T), natural log of sum exp(scale * s). window < 0 = full causal.
template <int BKV>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<BKV>::kSmemBytes) !=
        cudaSuccess)
      return -4;
    configured = true;
  }
  dim3 grid((p.T + BQ - 1) / BQ, p.B * p.H);
  flash_fwd_kernel<BKV><<<grid, kThreads, FwdCfg<BKV>::kSmemBytes, stream>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// q, k, v: (B, T, H, 128) bf16 with token stride ld_* elements (contiguous tensors: H*128); out contiguous;
// lse: fp32 (B, H, T), natural log of sum exp(scale * s). window < 0 = full causal. bkv: 64 or 128 keys per tile.
extern "C" int sr_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int T, int H,
                                 long ld_q, long ld_k, long ld_v, int window, float scale, int bkv, int* status,
                                 cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  if (bkv != 64 && bkv != 128) return -2;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = sr_attn::encode_bthd(&mq, q, B, T, H, ld_q, BQ))) return rc;
  if ((rc = sr_attn::encode_bthd(&mk, k, B, T, H, ld_k, bkv))) return rc - 10;
  if ((rc = sr_attn::encode_bthd(&mv, v, B, T, H, ld_v, bkv))) return rc - 20;
  FwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B; p.T = T; p.H = H;
  p.window = (window < 0 || window >= T) ? -1 : window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  return bkv == 64 ? launch_fwd<64>(mq, mk, mv, p, stream) : launch_fwd<128>(mq, mk, mv, p, stream);
}
