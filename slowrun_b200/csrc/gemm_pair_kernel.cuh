// CTA-pair tcgen05 GEMM kernel as a template over its epilogue, so that kernels which consume the accumulator tile
// in registers (the soft-capped cross-entropy of the lm-head, lmhead_ce.cu) share the TMA / MMA pipeline of the
// plain GEMM (gemm_tcgen05_pair.cu).
//
// Two CTAs on the two SMs of one TPC (a cluster of 2) compute one 256 x BN tile with tcgen05.mma.cta_group::2. Each
// CTA stages its own 128 rows of A and only HALF of the B tile (BN/2 rows); the instruction reads both halves. Against
// a single-CTA kernel this cuts the shared-memory traffic per tensor cycle by a third (operand reads 96 -> 64 B/clk,
// TMA writes likewise) and lets six to eight 32 KB stages fit instead of four 48 KB ones.
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
// Template parameters
//   BN   tile width (128, 160, 256)
//   EB   bytes per operand element: 2 = bf16 (kind::f16), 1 = fp8 e4m3/e5m2 (kind::f8f6f4, K-major operands only).
//        A k-block is always 128 bytes of K, so the shared-memory layout, the stage size and the 32-byte descriptor
//        step per MMA are the same for both; only the tensor maps, the instruction kind and the K coordinates differ.
//   Epi  epilogue policy, see EpiStore below.
#pragma once
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
template <int EB>
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  if (EB == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// Arrive (once all tcgen05.mma issued so far have completed) on the mbarrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

// Epilogue policy of the plain GEMM: alpha/beta, bf16 or fp32 store, accumulate-into reductions. A policy provides
//   Row                       per-thread state that lives across the 32-column chunks of one output row of one tile
//   begin(st, p, r, row_ok)   before the first chunk
//   chunk<BN>(st, p, f, r, c0, partial, cbase, cinbase)   f[] = alpha * accumulator for columns c0..c0+31 of row r
//   end(st, p, r, row_ok, nj) after the last chunk of the tile in tile column nj
struct EpiStore {
  struct Row {};
  static __device__ __forceinline__ void begin(Row&, const GemmParams&, int, bool) {}
  template <int BN>
  static __device__ __forceinline__ void chunk(Row&, const GemmParams& p, float (&f)[32], int r, int c0, bool partial,
                                               uint8_t* cbase, const uint8_t* cinbase) {
    epilogue_store<BN, PM>(p, f, r, c0, partial, cbase, cinbase);
  }
  static __device__ __forceinline__ void end(Row&, const GemmParams&, int, bool, int) {}
};

template <int BN, int EB, class Epi>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
  using C_ = PairCfg<BN>;
  constexpr int BKE = 128 / EB;   // elements of K per k-block (one 128-byte swizzle row)
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
  const int num_kb = (p.K + BKE - 1) / BKE;

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
        tile_coords<BN, PM>(p, tile, b, mi, nj);
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
          const int k0 = kb * BKE;
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
      const uint32_t a_fmt = EB == 2 ? 1u : (uint32_t)p.a_fmt, b_fmt = EB == 2 ? 1u : (uint32_t)p.b_fmt;
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
        const uint32_t idesc = make_idesc(a_fmt, b_fmt, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u, PM, (uint32_t)wi.n_w);
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
            umma_ss_pair<EB>(tmem_d, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
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
      tile_coords<BN, PM>(p, tile, b, mi, nj);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, 300);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int r = mi * PM + (int)rank * BM + q * 32 + lane;
      const bool row_ok = r < p.M;
      float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
      if (p.row_scale != nullptr && row_ok) alpha *= __ldg(p.row_scale + (size_t)b * p.M + r);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * C_::kAccStride);
      uint8_t* cbase = reinterpret_cast<uint8_t*>(p.C) + (size_t)b * p.strideC * (p.c_fp32 ? 4 : 2);
      const uint8_t* cinbase =
          p.Cin ? reinterpret_cast<const uint8_t*>(p.Cin) + (size_t)b * p.strideCin * (p.cin_fp32 ? 4 : 2) : nullptr;
      const int nch = (wi.n_w + 31) / 32;
      typename Epi::Row st;
      Epi::begin(st, p, r, row_ok);
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
          Epi::template chunk<BN>(st, p, f, r, c0, partial, cbase, cinbase);
        }
      }
      Epi::end(st, p, r, row_ok, nj);
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

// Fills in the tile counts and launches on clusters of two. `allow_tail_split` = 0 keeps every tile whole (policies
// that keep per-tile state, such as row sums, need that).
template <int BN, int EB, class Epi>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int max_ctas, int allow_tail_split,
                cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<BN, EB, Epi>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             PairCfg<BN>::kSmemBytes) != cudaSuccess)
      return -4;
    configured = true;
  }
  p.tiles_m = (p.M + PM - 1) / PM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n * p.batch;
  if (p.sym) {   // only the tiles that touch the upper triangle; the others are filled by mirrored stores
    int per_batch = 0;
    for (int r = 0; r < p.tiles_m; ++r) per_batch += p.tiles_n - (r * PM) / BN;
    p.num_tiles = per_batch * p.batch;
  }
  int pairs = num_sms() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (pairs < 1) pairs = 1;
  p.tail_split = 1;
  constexpr int BKE = 128 / EB;
  if (p.splitk) {
    const long long units = (long long)p.num_tiles * ((p.K + BKE - 1) / BKE);
    if (units < pairs) pairs = (int)units;
    if (p.num_tiles % pairs == 0) p.splitk = 0;
  } else {
    // last, partial wave: when at most half of the pairs would have a tile, cut those tiles into two 128-wide
    // column slices so that the wave takes half as long
    const int rem = p.num_tiles % pairs;
    if (allow_tail_split && !p.sym && BN == 256 && rem > 0 && 2 * rem <= pairs) p.tail_split = 2;
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
  return cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, EB, Epi>, ma, mb, p) == cudaSuccess ? 0 : -5;
}

}  // namespace
