// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) -> tcgen05.mma with the
// fp32 accumulator in TMEM (double buffered) -> tcgen05.ld epilogue.
//
//   out[b] = alpha * op(A[b]) * op(B[b]) + beta * Cin[b]
//
// A is an (M x K) operand, B an (N x K) operand ("TN" form). Either operand may be stored K-major
// (row-major [rows, K]) or MN-major (row-major [K, rows]); the difference is only in the TMA box and the
// shared-memory descriptor, the instruction reads both. This covers every GEMM of the training step without a
// transpose pass: y = x W^T (K/K), dx = dy W (K/MN), dW += dy^T x (MN/MN, fp32 accumulate into the gradient
// buffer through Cin == out), and the Newton-Schulz products X X^T, bA + cA^2, aX + BX.
//
// `sym` mode: the result is known to be symmetric (gram matrices); only tiles that touch the upper triangle
// are computed and every element is also stored mirrored.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2..5 = epilogue.
// The reference does these products with cuBLAS through torch (train.py:286-323 F.linear, train.py:614-621 bmm).
#include <cstdlib>
#include "gemm_common.cuh"

namespace {

template <int BN>
struct Cfg {
  // BN = 160 exists for N = 2560-like widths, where 128x256 tiles leave a third of the last wave idle.
  static constexpr int kBNLoad = ((BN + 63) / 64) * 64;   // columns staged per k-block (MN-major boxes are 64 wide)
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 160 ? 5 : 6);
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = kBNLoad * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = (BN == 128) ? 256 : 512;   // two accumulators, power of two
  static constexpr int kAccStride = (BN == 128) ? 128 : 256;  // column offset of the second accumulator
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
  using C_ = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C_::kStages * C_::kStageBytes);
  uint64_t* full_bar = bars;                      // [kStages]
  uint64_t* empty_bar = bars + C_::kStages;       // [kStages]
  uint64_t* tfull_bar = bars + 2 * C_::kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C_::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C_::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, num_kb, blockIdx.x, gridDim.x, BN);
      int tile, kb0, kb1;
      bool partial;
      while (ok && wi.next(tile, kb0, kb1, partial)) {
        int b, mi, nj;
        tile_coords<BN>(p, tile, b, mi, nj);
        const int m0 = mi * BM, n0 = nj * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 100);
          if (!ok) break;
          uint8_t* sa = smem + stage * C_::kStageBytes;
          uint8_t* sb = sa + C_::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], C_::kABytes + (p.b_mn ? C_::kBBytes : BN * BK * 2));
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_3d(sa, &map_a, &full_bar[stage], k0, m0, b);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g) tma_load_3d(sa + g * (BK * 128), &map_a, &full_bar[stage], m0 + g * 64, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d(sb, &map_b, &full_bar[stage], k0, n0, b);
          } else {
#pragma unroll
            for (int g = 0; g < C_::kBNLoad / 64; ++g) tma_load_3d(sb + g * (BK * 128), &map_b, &full_bar[stage], n0 + g * 64, k0, b);
          }
          if (++stage == C_::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1, 1, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, BM, BN);
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, num_kb, blockIdx.x, gridDim.x, BN);
      int tile, kb0, kb1;
      bool partial;
      for (; ok && wi.next(tile, kb0, kb1, partial); ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = mbar_wait(&tempty_bar[buf], acc_phase ^ 1u, abort_flag, p.status, 200);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * C_::kAccStride);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 201);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C_::kStageBytes);
          const uint32_t sb = sa + C_::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_f16_ss(tmem_d, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == C_::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int local = 0;
    bool ok = true;
    WorkIter wi;
    wi.init(p, num_kb, blockIdx.x, gridDim.x, BN);
    int tile, kb0, kb1;
    bool partial;
    for (; ok && wi.next(tile, kb0, kb1, partial); ++local) {
      int b, mi, nj;
      tile_coords<BN>(p, tile, b, mi, nj);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, 300);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM loads
      if (!ok) break;
      float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
      tc_fence_after();
      const int r = mi * BM + q * 32 + lane;
      const bool row_ok = r < p.M;
      if (p.row_scale != nullptr && row_ok) alpha *= __ldg(p.row_scale + (size_t)b * p.M + r);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * C_::kAccStride);
      uint8_t* cbase = reinterpret_cast<uint8_t*>(p.C) + (size_t)b * p.strideC * (p.c_fp32 ? 4 : 2);
      const uint8_t* cinbase =
          p.Cin ? reinterpret_cast<const uint8_t*>(p.Cin) + (size_t)b * p.strideCin * (p.cin_fp32 ? 4 : 2) : nullptr;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + ch * 32, v);
        tc_wait_ld();
        const int c0 = nj * BN + ch * 32;
        if (row_ok && c0 < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = alpha * __uint_as_float(v[j]);
          epilogue_store<BN>(p, f, r, c0, partial, cbase, cinbase);
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[buf]);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C_::kTmemCols);
  }
}

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int max_ctas, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes) !=
        cudaSuccess)
      return -4;
    configured = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  int per_batch = 0;
  if (p.sym) {
    for (int r = 0; r < p.tiles_m; ++r) per_batch += p.tiles_n - (r * BM) / BN;
  } else {
    per_batch = p.tiles_m * p.tiles_n;
  }
  p.num_tiles = per_batch * p.batch;
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (p.splitk) {
    const long long units = (long long)p.num_tiles * ((p.K + BK - 1) / BK);
    if (units < grid) grid = (int)units;
    if (p.num_tiles % grid == 0) p.splitk = 0;   // no partial wave: nothing to balance
  } else if (p.num_tiles < grid) {
    grid = p.num_tiles;
  }
  if (grid <= 0) return 0;
  gemm_bf16_kernel<BN><<<grid, kNumThreads, Cfg<BN>::kSmemBytes, stream>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

extern "C" int sr_gemm_bf16_pair(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                                 long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                                 long long strideB, long long strideC, long long strideCin, int a_mn, int b_mn,
                                 int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr,
                                 const float* row_scale, int sym, int splitk, int bn, int max_ctas, int* status,
                                 cudaStream_t stream);

// Process-wide handle of the driver's tensor-map encoder (see gemm_common.cuh). Resolved on first use and by
// sr_runtime_init(); returns null when the driver does not export it.
extern "C" void* sr_driver_encode_tiled(void) {
  static void* fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = ptr;
  }
  return fn;
}

// Called once by the loader, from the thread that opened the library, with the device it will use current: creates
// the runtime's context on that device and resolves the driver entry point there. Returns 0, or -1 when the tensor-map
// encoder is not available.
extern "C" int sr_runtime_init(void) {
  cudaFree(nullptr);
  return sr_driver_encode_tiled() != nullptr ? 0 : -1;
}

static int g_pair_mode = 1;
// 1 (default): eligible problems run on the CTA-pair kernel (gemm_tcgen05_pair.cu); 0: single-CTA kernel only.
extern "C" void sr_gemm_set_pair_mode(int on) { g_pair_mode = on; }

// out[b] = alpha * op(A[b]) op(B[b])^T + beta * Cin[b]; see the file header.
//   a_mn / b_mn : 0 = operand stored [rows, K] (K contiguous), 1 = stored [K, rows] (rows contiguous)
//   lda / ldb   : leading dimension (elements) of the stored 2-D array; stride* : per-batch element stride
//   alpha_ptr   : optional device fp32 scalar; the product is scaled by alpha * (*alpha_ptr)
//   row_scale   : optional device fp32 [batch, M]; row r of the product is also scaled by row_scale[r]
//   bn          : N tile (128 or 256), 0 = choose
//   status      : device int[4]; written only when a bounded wait ran out (see sm100_common.cuh)
// Returns 0 on successful launch, negative on bad arguments / launch failure.
extern "C" int sr_gemm_bf16(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                            long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                            long long strideB, long long strideC, long long strideCin, int a_mn, int b_mn,
                            int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr,
                            const float* row_scale, int sym, int bn, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (sym && M != N) return -6;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.strideC = strideC; p.c_fp32 = c_fp32;
  p.Cin = Cin; p.ldcin = ldcin; p.strideCin = strideCin; p.cin_fp32 = cin_fp32;
  p.alpha = alpha; p.beta = beta; p.alpha_ptr = alpha_ptr; p.row_scale = row_scale; p.sym = sym; p.status = status;
  // accumulate-into fp32 output (weight gradients): balance the k-loop over all SMs instead of whole tiles
  p.splitk = (c_fp32 && Cin == C && beta == 1.0f && !sym && ldcin == ldc && strideCin == strideC) ? 1 : 0;
  if (bn < 0) { p.splitk = 0; bn = -bn; }   // negative bn: caller forces the plain tile schedule
  // CTA pairs (256-row tiles over 74 pairs) for everything but single-tile-high problems; SR_GEMM_SYM_PAIR=0 (read
  // once) keeps symmetric outputs on the single-CTA kernel
  static const bool sym_pair = [] { const char* e = getenv("SR_GEMM_SYM_PAIR"); return e == nullptr || e[0] != '0'; }();
  const bool use_pair = g_pair_mode && M > BM && (!sym || sym_pair);
  const int rows = use_pair ? 2 * BM : BM;
  const int workers = use_pair ? num_sms() / 2 : num_sms();
  if (bn == 0 && p.splitk) bn = 256;
  if (bn == 0) {
    // prefer the 256-wide tile unless it leaves most of a wave idle
    const long long tm = (M + rows - 1) / rows;
    // tiles / (waves * workers); the pair kernel halves a last wave that at most half of the pairs would join
    auto eff = [&](long long tiles, bool splittable) {
      const long long full = tiles / workers, rem = tiles % workers;
      const double waves = (double)full + (rem == 0 ? 0.0 : (splittable && 2 * rem <= workers ? 0.5 : 1.0));
      return (double)tiles / (waves * workers);
    };
    // tiles of one matrix: all of them, or in symmetric mode only those that touch the upper triangle
    auto tiles_of = [&](int w) {
      const long long tn = (N + w - 1) / w;
      if (!sym) return tm * tn;
      long long t = 0;
      for (long long r = 0; r < tm; ++r) t += tn - (r * rows) / w;
      return t;
    };
    const double eff256 = eff(tiles_of(256) * batch, use_pair);
    const double eff128 = eff(tiles_of(128) * batch, false);
    bn = (eff256 + 0.08 >= eff128 && N > 128) ? 256 : 128;
    // 160-wide tiles when N is a multiple of 160 and they fill the waves better than both
    if (N % 160 == 0 && !b_mn && !sym) {
      const double eff160 = eff(tm * (N / 160) * batch, false);
      const double best = bn == 256 ? eff256 : eff128 * 0.92;
      if (eff160 * 0.97 > best + 0.03) bn = 160;
    }
  }
  if (bn != 128 && bn != 160 && bn != 256) return -7;
  if (use_pair && !(bn == 160 && b_mn))
    return sr_gemm_bf16_pair(A, B, C, Cin, M, N, K, batch, lda, ldb, ldc, ldcin, strideA, strideB, strideC, strideCin,
                             a_mn, b_mn, c_fp32, cin_fp32, alpha, beta, alpha_ptr, row_scale, sym, p.splitk, bn, max_ctas,
                             status, stream);
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = encode_bf16_map(&ma, A, K, M, batch, lda, strideA, BK, BM);
  else       rc = encode_bf16_map(&ma, A, M, K, batch, lda, strideA, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = encode_bf16_map(&mb, B, K, N, batch, ldb, strideB, BK, bn);
  else       rc = encode_bf16_map(&mb, B, N, K, batch, ldb, strideB, 64, BK);
  if (rc) return rc - 10;
  if (bn == 256) return launch<256>(ma, mb, p, max_ctas, stream);
  if (bn == 160) return launch<160>(ma, mb, p, max_ctas, stream);
  return launch<128>(ma, mb, p, max_ctas, stream);
}
