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
#include "sm100_common.cuh"

namespace {

using namespace sr;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumThreads = 192;

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

struct GemmParams {
  int M, N, K, batch;
  int tiles_m, tiles_n, num_tiles;
  int a_mn, b_mn;
  void* C;
  long long ldc, strideC;
  int c_fp32;
  const void* Cin;
  long long ldcin, strideCin;
  int cin_fp32;
  float alpha, beta;
  const float* alpha_ptr;  // optional device scalar multiplied into alpha
  int sym;
  int splitk;              // fp32 accumulate-into output: CTAs own equal shares of (tile, k-block) units and add their
                           // partial tiles with vector reductions, so the last wave is never partly idle

  int* status;
};

// Tile index -> (batch, mi, nj). In sym mode rows only hold the tiles that touch the upper triangle.
template <int BN>
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& b, int& mi, int& nj) {
  if (!p.sym) {
    const int per_batch = p.tiles_m * p.tiles_n;
    b = tile / per_batch;
    int t = tile - b * per_batch;
    // groups of 8 M-tiles share their B tiles in L2
    constexpr int G = 8;
    const int group_sz = G * p.tiles_n;
    const int g = t / group_sz;
    const int first_m = g * G;
    const int gm = min(G, p.tiles_m - first_m);
    const int tt = t - g * group_sz;
    mi = first_m + tt % gm;
    nj = tt / gm;
  } else {
    int per_batch = 0;
    for (int r = 0; r < p.tiles_m; ++r) per_batch += p.tiles_n - (r * BM) / BN;
    b = tile / per_batch;
    int t = tile - b * per_batch;
    mi = 0;
    while (true) {
      const int first = (mi * BM) / BN;
      const int cnt = p.tiles_n - first;
      if (t < cnt) {
        nj = first + t;
        break;
      }
      t -= cnt;
      ++mi;
    }
  }
}

// Work items of one CTA. Full waves of tiles are strided over the grid (concurrent CTAs work on neighbouring tiles, which
// keeps their operand panels in L2). In splitk mode the tiles of the last, partial wave are cut along K instead: every
// CTA gets an equal share of their (tile, k-block) units and adds its partial tile with reductions.
struct WorkIter {
  int num_kb, stride, full_tiles;
  int t;                // cursor over the strided full-wave tiles
  long long u, u_end;   // cursor / end over the tail units
  __device__ __forceinline__ void init(const GemmParams& p, int nkb) {
    num_kb = nkb;
    stride = gridDim.x;
    t = blockIdx.x;
    if (p.splitk) {
      full_tiles = (p.num_tiles / stride) * stride;
      const long long units = (long long)(p.num_tiles - full_tiles) * nkb;
      u = units * blockIdx.x / stride;
      u_end = units * (blockIdx.x + 1) / stride;
    } else {
      full_tiles = p.num_tiles;
      u = u_end = 0;
    }
  }
  // partial = true: the item covers only part of K (or shares its tile with other CTAs) and must be added atomically
  __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1, bool& partial) {
    if (t < full_tiles) {
      tile = t;
      kb0 = 0;
      kb1 = num_kb;
      partial = false;
      t += stride;
      return true;
    }
    if (u >= u_end) return false;
    const int tt = (int)(u / num_kb);
    tile = full_tiles + tt;
    kb0 = (int)(u - (long long)tt * num_kb);
    const long long len = min((long long)(num_kb - kb0), u_end - u);
    kb1 = kb0 + (int)len;
    partial = true;
    u += len;
    return true;
  }
};

__device__ __forceinline__ bool sym_tile_skipped(int r, int c, int bn) {
  // the tile that would own element (r, c): mi = r / BM, nj = c / bn; skipped iff it lies below the diagonal band
  const int mi = r / BM, nj = c / bn;
  return nj * bn + bn <= mi * BM;
}

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
      wi.init(p, num_kb);
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
      wi.init(p, num_kb);
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
    wi.init(p, num_kb);
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
      const float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
      tc_fence_after();
      const int r = mi * BM + q * 32 + lane;
      const bool row_ok = r < p.M;
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
          const bool full = (c0 + 32 <= p.N);
          if (partial) {
            // partial tile of an accumulate-into fp32 output: add it with 16-byte reductions
            float* dst = reinterpret_cast<float*>(cbase) + (size_t)r * p.ldc + c0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(f[j]), "f"(f[j + 1]),
                             "f"(f[j + 2]), "f"(f[j + 3])
                             : "memory");
            } else {
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) atomicAdd(dst + j, f[j]);
            }
            continue;
          }
          if (cinbase) {
            if (p.cin_fp32) {
              const float* src = reinterpret_cast<const float*>(cinbase) + (size_t)r * p.ldcin + c0;
              if (full && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const float4 t = *reinterpret_cast<const float4*>(src + j);
                  f[j] += p.beta * t.x; f[j + 1] += p.beta * t.y; f[j + 2] += p.beta * t.z; f[j + 3] += p.beta * t.w;
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (c0 + j < p.N) f[j] += p.beta * src[j];
              }
            } else {
              const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(cinbase) + (size_t)r * p.ldcin + c0;
              if (full && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const uint4 t = *reinterpret_cast<const uint4*>(src + j);
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 ff = __bfloat1622float2(h[e]);
                    f[j + 2 * e] += p.beta * ff.x;
                    f[j + 2 * e + 1] += p.beta * ff.y;
                  }
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (c0 + j < p.N) f[j] += p.beta * __bfloat162float(src[j]);
              }
            }
          }
          if (p.c_fp32) {
            float* dst = reinterpret_cast<float*>(cbase) + (size_t)r * p.ldc + c0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) dst[j] = f[j];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cbase) + (size_t)r * p.ldc + c0;
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 t;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[j + 2 * e], f[j + 2 * e + 1]);
                *reinterpret_cast<uint4*>(dst + j) = t;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.N) dst[j] = __float2bfloat16(f[j]);
            }
          }
          if (p.sym) {
            // mirrored store for the tiles that were not computed; lanes hold consecutive rows, so each
            // store instruction writes 32 consecutive elements of one output row.
            for (int j = 0; j < 32; ++j) {
              const int c = c0 + j;
              if (c < p.N && c > r && sym_tile_skipped(c, r, BN)) {
                if (p.c_fp32)
                  reinterpret_cast<float*>(cbase)[(size_t)c * p.ldc + r] = f[j];
                else
                  reinterpret_cast<__nv_bfloat16*>(cbase)[(size_t)c * p.ldc + r] = __float2bfloat16(f[j]);
              }
            }
          }
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

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 3-D bf16 tensor map {inner, rows, batch}, 128B swizzle, zero fill outside the tensor.
int encode_bf16_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t ld,
                    uint64_t batch_stride, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((ld % 8) != 0 || (reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return -2;
  if (batch > 1 && (batch_stride % 8) != 0) return -2;
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {ld * 2, (batch > 1 ? batch_stride : rows * ld) * 2};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
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

// out[b] = alpha * op(A[b]) op(B[b])^T + beta * Cin[b]; see the file header.
//   a_mn / b_mn : 0 = operand stored [rows, K] (K contiguous), 1 = stored [K, rows] (rows contiguous)
//   lda / ldb   : leading dimension (elements) of the stored 2-D array; stride* : per-batch element stride
//   alpha_ptr   : optional device fp32 scalar; the product is scaled by alpha * (*alpha_ptr)
//   bn          : N tile (128 or 256), 0 = choose
//   status      : device int[4]; written only when a bounded wait ran out (see sm100_common.cuh)
// Returns 0 on successful launch, negative on bad arguments / launch failure.
extern "C" int sr_gemm_bf16(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                            long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                            long long strideB, long long strideC, long long strideCin, int a_mn, int b_mn,
                            int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr, int sym,
                            int bn, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (sym && M != N) return -6;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.strideC = strideC; p.c_fp32 = c_fp32;
  p.Cin = Cin; p.ldcin = ldcin; p.strideCin = strideCin; p.cin_fp32 = cin_fp32;
  p.alpha = alpha; p.beta = beta; p.alpha_ptr = alpha_ptr; p.sym = sym; p.status = status;
  // accumulate-into fp32 output (weight gradients): balance the k-loop over all SMs instead of whole tiles
  p.splitk = (c_fp32 && Cin == C && beta == 1.0f && !sym && ldcin == ldc && strideCin == strideC) ? 1 : 0;
  if (bn < 0) { p.splitk = 0; bn = -bn; }   // negative bn: caller forces the plain tile schedule
  if (bn == 0 && p.splitk) bn = 256;
  if (bn == 0) {
    // prefer the 256-wide tile unless it leaves most of a wave idle
    const long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256) * batch;
    const int sms = num_sms();
    const long long waves256 = (t256 + sms - 1) / sms;
    const double eff256 = (double)t256 / (double)(waves256 * sms);
    const long long t128 = (long long)((M + 127) / 128) * ((N + 127) / 128) * batch;
    const long long waves128 = (t128 + sms - 1) / sms;
    const double eff128 = (double)t128 / (double)(waves128 * sms);
    bn = (eff256 + 0.08 >= eff128 && N > 128) ? 256 : 128;
    // 160-wide tiles when N is a multiple of 160 and they fill the waves better than both
    if (N % 160 == 0 && !b_mn) {
      const long long t160 = (long long)((M + 127) / 128) * (N / 160) * batch;
      const long long waves160 = (t160 + sms - 1) / sms;
      const double eff160 = (double)t160 / (double)(waves160 * sms);
      const double best = bn == 256 ? eff256 : eff128 * 0.92;
      if (eff160 * 0.97 > best + 0.03) bn = 160;
    }
  }
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = encode_bf16_map(&ma, A, K, M, batch, lda, strideA, BK, BM);
  else       rc = encode_bf16_map(&ma, A, M, K, batch, lda, strideA, 64, BK);
  if (rc) return rc;
  if (bn != 128 && bn != 160 && bn != 256) return -7;
  if (!b_mn) rc = encode_bf16_map(&mb, B, K, N, batch, ldb, strideB, BK, bn);
  else       rc = encode_bf16_map(&mb, B, N, K, batch, ldb, strideB, 64, BK);
  if (rc) return rc - 10;
  if (bn == 256) return launch<256>(ma, mb, p, max_ctas, stream);
  if (bn == 160) return launch<160>(ma, mb, p, max_ctas, stream);
  return launch<128>(ma, mb, p, max_ctas, stream);
}
