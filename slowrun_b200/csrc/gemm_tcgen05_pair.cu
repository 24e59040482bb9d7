// CTA-pair variant of the persistent bf16 GEMM: two CTAs on the two SMs of one TPC (a cluster of 2) compute one
// 256 x BN tile with tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and only HALF of the B tile
// (BN/2 rows); the instruction reads both halves. Against the single-CTA kernel this cuts the shared-memory traffic
// per tensor cycle by a third (operand reads 96 -> 64 B/clk, TMA writes likewise) and lets six to eight 32 KB stages
// fit instead of four 48 KB ones, which is what keeps the tensor pipe fed on the large training GEMMs.
//
// Protocol (rank 0 of the pair = leader, rank 1 = peer):
//   full[s]    lives in the leader. The leader's producer arms it with the bytes of BOTH CTAs' loads; both CTAs'
//              TMA loads complete their bytes on it (cp.async.bulk.tensor with .cta_group::2 may signal the other
//              CTA of the pair).
//   empty[s]   one per CTA; the leader's MMA thread releases a stage in both CTAs with one tcgen05.commit that
//              arrives on the barrier at the same offset in each CTA of the mask.
//   tfull[b]   one per CTA, same commit form: accumulator b is complete in both CTAs' TMEM.
//   tempty[b]  lives in the leader, count 256: the 128 epilogue threads of each CTA arrive on it (the peer's
//              through its cluster address) when they have drained their half of the accumulator.
// TMEM is allocated and freed by warp 1 of both CTAs with the cta_group::2 forms; a cluster barrier after the
// mbarrier initialisation and one before the teardown keep either CTA's shared memory alive while the other may
// still signal it. Every wait is bounded (see sm100_common.cuh); nothing here loads through the cluster.
//
// Same contract as the single-CTA kernel (gemm_tcgen05.cu) except: no symmetric-output mode.
#include "gemm_common.cuh"

namespace {

constexpr int PM = 256;  // rows of a pair tile

template <int BN>
struct PairCfg {
  static constexpr int kBHalf = BN / 2;                          // B rows staged by each CTA
  static constexpr int kBHalfLoad = ((kBHalf + 63) / 64) * 64;   // MN-major boxes are 64 wide
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = kBHalfLoad * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 6 : (BN == 160 ? 7 : 8);
  static constexpr int kTmemCols = (BN == 128) ? 256 : 512;
  static constexpr int kAccStride = (BN == 128) ? 128 : 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static_assert(kStageBytes % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted on an mbarrier that may sit in the other CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once all tcgen05.mma issued so far have completed) on the mbarrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
  using C_ = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C_::kStages * C_::kStageBytes);
  uint64_t* full_bar = bars;                      // [kStages]   (used in the leader)
  uint64_t* empty_bar = bars + C_::kStages;       // [kStages]
  uint64_t* tfull_bar = bars + 2 * C_::kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]         (used in the leader)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader, 1 = peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C_::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 256);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, C_::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything may signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, num_kb, pair, num_pairs, BN);
      int tile, kb0, kb1;
      bool partial;
      const uint32_t full0 = map_to_cta(smem_u32(&full_bar[0]), 0);   // the leader's full barriers
      constexpr uint32_t kBLoadBytes = C_::kBHalf * BK * 2;           // bytes actually loaded for B per CTA (K-major)
      while (ok && wi.next(tile, kb0, kb1, partial)) {
        int b, mi, nj;
        tile_coords<BN>(p, tile, b, mi, nj);
        const int m0 = mi * PM + (int)rank * BM;
        const int n0 = nj * BN + wi.n_off + (int)rank * (wi.n_w / 2);   // a column slice loads the same boxes, uses fewer rows
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 100);
          if (!ok) break;
          uint8_t* sa = smem + stage * C_::kStageBytes;
          uint8_t* sb = sa + C_::kABytes;
          if (rank == 0) {
            const uint32_t b_bytes = p.b_mn ? (uint32_t)((wi.n_w / 2 + 63) / 64) * (64 * BK * 2) : kBLoadBytes;
            mbar_arrive_expect_tx(&full_bar[stage], 2u * (C_::kABytes + b_bytes));
          }
          const uint32_t fb = full0 + stage * 8;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_3d_pair(sa, &map_a, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g) tma_load_3d_pair(sa + g * (BK * 128), &map_a, fb, m0 + g * 64, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d_pair(sb, &map_b, fb, k0, n0, b);
          } else {
#pragma unroll
            for (int g = 0; g < C_::kBHalfLoad / 64; ++g)
              if (g * 64 < wi.n_w / 2) tma_load_3d_pair(sb + g * (BK * 128), &map_b, fb, n0 + g * 64, k0, b);
          }
          if (++stage == C_::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      WorkIter wi;
      wi.init(p, num_kb, pair, num_pairs, BN);
      int tile, kb0, kb1;
      bool partial;
      for (; ok && wi.next(tile, kb0, kb1, partial); ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = mbar_wait(&tempty_bar[buf], acc_phase ^ 1u, abort_flag, p.status, 200);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * C_::kAccStride);
        const uint32_t idesc = make_idesc(1, 1, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, PM, (uint32_t)wi.n_w);
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
            umma_f16_ss_pair(tmem_d, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[stage]);   // frees this stage in both CTAs
          if (++stage == C_::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit_pair(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int local = 0;
    bool ok = true;
    WorkIter wi;
    wi.init(p, num_kb, pair, num_pairs, BN);
    int tile, kb0, kb1;
    bool partial;
    const uint32_t tempty0 = map_to_cta(smem_u32(&tempty_bar[0]), 0);
    for (; ok && wi.next(tile, kb0, kb1, partial); ++local) {
      int b, mi, nj;
      tile_coords<BN>(p, tile, b, mi, nj);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, 300);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
      tc_fence_after();
      const int r = mi * PM + (int)rank * BM + q * 32 + lane;
      const bool row_ok = r < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * C_::kAccStride);
      uint8_t* cbase = reinterpret_cast<uint8_t*>(p.C) + (size_t)b * p.strideC * (p.c_fp32 ? 4 : 2);
      const uint8_t* cinbase =
          p.Cin ? reinterpret_cast<const uint8_t*>(p.Cin) + (size_t)b * p.strideCin * (p.cin_fp32 ? 4 : 2) : nullptr;
      const int nch = (wi.n_w + 31) / 32;
#pragma unroll 1
      for (int ch = 0; ch < nch; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + ch * 32, v);
        tc_wait_ld();
        const int c0 = nj * BN + wi.n_off + ch * 32;
        if (row_ok && c0 < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = alpha * __uint_as_float(v[j]);
          epilogue_store<BN>(p, f, r, c0, partial, cbase, cinbase);
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(tempty0 + buf * 8);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves (or frees TMEM) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C_::kTmemCols);
  }
}

template <int BN>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int max_ctas, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             PairCfg<BN>::kSmemBytes) != cudaSuccess)
      return -4;
    configured = true;
  }
  p.tiles_m = (p.M + PM - 1) / PM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n * p.batch;
  int pairs = num_sms() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (pairs < 1) pairs = 1;
  p.tail_split = 1;
  if (p.splitk) {
    const long long units = (long long)p.num_tiles * ((p.K + BK - 1) / BK);
    if (units < pairs) pairs = (int)units;
    if (p.num_tiles % pairs == 0) p.splitk = 0;
  } else {
    // last, partial wave: when at most half of the pairs would have a tile, cut those tiles into two 128-wide
    // column slices so that the wave takes half as long
    const int rem = p.num_tiles % pairs;
    if (BN == 256 && rem > 0 && 2 * rem <= pairs) p.tail_split = 2;
    if (p.num_tiles < pairs) pairs = p.num_tiles * p.tail_split;
  }
  if (pairs <= 0) return 0;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<BN>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<BN>, ma, mb, p) == cudaSuccess ? 0 : -5;
}

}  // namespace

// CTA-pair GEMM; arguments as sr_gemm_bf16 (gemm_tcgen05.cu) without `sym`. bn in {128, 160, 256} (160 only with a
// K-major B), already chosen by the caller. Returns 0 on successful launch.
extern "C" int sr_gemm_bf16_pair(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                                 long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                                 long long strideB, long long strideC, long long strideCin, int a_mn, int b_mn,
                                 int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr, int splitk,
                                 int bn, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (bn != 128 && bn != 160 && bn != 256) return -7;
  if (bn == 160 && b_mn) return -7;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.strideC = strideC; p.c_fp32 = c_fp32;
  p.Cin = Cin; p.ldcin = ldcin; p.strideCin = strideCin; p.cin_fp32 = cin_fp32;
  p.alpha = alpha; p.beta = beta; p.alpha_ptr = alpha_ptr; p.sym = 0; p.status = status;
  p.splitk = splitk;
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = encode_bf16_map(&ma, A, K, M, batch, lda, strideA, BK, BM);
  else       rc = encode_bf16_map(&ma, A, M, K, batch, lda, strideA, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = encode_bf16_map(&mb, B, K, N, batch, ldb, strideB, BK, bn / 2);
  else       rc = encode_bf16_map(&mb, B, N, K, batch, ldb, strideB, 64, BK);
  if (rc) return rc - 10;
  if (bn == 256) return launch_pair<256>(ma, mb, p, max_ctas, stream);
  if (bn == 160) return launch_pair<160>(ma, mb, p, max_ctas, stream);
  return launch_pair<128>(ma, mb, p, max_ctas, stream);
}
