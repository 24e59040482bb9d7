// Pieces shared by the single-CTA and the CTA-pair tcgen05 GEMM kernels: parameters, the work-item iterator, the
// per-chunk epilogue (alpha/beta, fp32 or bf16 output, accumulate-into reductions, mirrored store) and the TMA
// tensor-map encoder.
#pragma once
#include "sm100_common.cuh"
#include <stdio.h>

namespace {

using namespace sr;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumThreads = 192;

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
  int tail_split;          // >1: the tiles of the last, partial wave are cut into this many column slices (pair kernel)
  int splitk;              // fp32 accumulate-into output: CTAs own equal shares of (tile, k-block) units and add their
                           // partial tiles with vector reductions, so the last wave is never partly idle

  const float* row_scale;  // optional fp32 [batch, M]: output row r is scaled by row_scale[r] (before beta * Cin)
  int a_fmt, b_fmt;        // fp8 operands (kind::f8f6f4): 0 = e4m3, 1 = e5m2; ignored for bf16

  // Soft-capped cross-entropy epilogue (lmhead_ce.cu); unused by the plain GEMM.
  struct Ce {
    const long* targets;   // int64 [M]; row r is scored against targets[r + k], k < n_predict (flattened index)
    float* partials;       // fp32 [tiles_n, M]: per-tile row sums of exp(z - cap)
    float* ztgt;           // fp32 [M, 4]: soft-capped logit at each of the row's targets
    int n_predict, V;      // targets per row (<= 4); valid vocabulary (columns >= V do not enter the sum)
    float cap, inv_cap;
  } ce;

  int* status;
};

// Tile index -> (batch, mi, nj). In sym mode rows only hold the tiles that touch the upper triangle. TM = tile height
// (128 for one CTA, 256 for a CTA pair).
template <int BN, int TM = BM>
__host__ __device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& b, int& mi, int& nj) {
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
    for (int r = 0; r < p.tiles_m; ++r) per_batch += p.tiles_n - (r * TM) / BN;
    b = tile / per_batch;
    int t = tile - b * per_batch;
    mi = 0;
    while (true) {
      const int first = (mi * TM) / BN;
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

// (init/next, tile_coords and sym_tile_skipped also compile for the host: tests/native/sched_model_test.cu replays them for
// every worker of many problem shapes and checks that the work is covered exactly once.)
// Work items of one CTA. Full waves of tiles are strided over the grid (concurrent CTAs work on neighbouring tiles, which
// keeps their operand panels in L2). In splitk mode the tiles of the last, partial wave are cut along K instead: every
// CTA gets an equal share of their (tile, k-block) units and adds its partial tile with reductions.
struct WorkIter {
  int num_kb, stride, full_tiles;
  int t;                // cursor over the strided full-wave tiles
  long long u, u_end;   // cursor / end over the tail units
  int split, v, v_end;  // column-sliced tail (tail_split mode): slices per tile, cursor and end over the slices
  int n_off, n_w;       // column slice of the current item within its tile (set by next())
  int bn_full;
  // worker / nworkers: this CTA (or CTA pair) and how many of them share the problem
  __host__ __device__ __forceinline__ void init(const GemmParams& p, int nkb, int worker, int nworkers, int bn) {
    num_kb = nkb;
    stride = nworkers;
    t = worker;
    n_off = 0;
    n_w = bn;
    bn_full = bn;
    split = 1;
    v = v_end = 0;
    if (!p.splitk && p.tail_split > 1) {
      split = p.tail_split;
      full_tiles = (p.num_tiles / stride) * stride;
      v = worker;
      v_end = (p.num_tiles - full_tiles) * split;
      u = u_end = 0;
      return;
    }
    if (p.splitk) {
      full_tiles = (p.num_tiles / stride) * stride;
      const long long units = (long long)(p.num_tiles - full_tiles) * nkb;
      u = units * worker / stride;
      u_end = units * (worker + 1) / stride;
    } else {
      full_tiles = p.num_tiles;
      u = u_end = 0;
    }
  }
  // partial = true: the item covers only part of K (or shares its tile with other CTAs) and must be added atomically
  __host__ __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1, bool& partial) {
    if (t < full_tiles) {
      tile = t;
      kb0 = 0;
      kb1 = num_kb;
      partial = false;
      t += stride;
      return true;
    }
    if (split > 1) {
      if (v >= v_end) return false;
      tile = full_tiles + v / split;
      n_w = bn_full / split;
      n_off = (v % split) * n_w;
      kb0 = 0;
      kb1 = num_kb;
      partial = false;
      v += stride;
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

__host__ __device__ __forceinline__ bool sym_tile_skipped(int r, int c, int bn, int tm) {
  // the tile that would own element (r, c): mi = r / tm, nj = c / bn; skipped iff it lies below the diagonal band
  const int mi = r / tm, nj = c / bn;
  return nj * bn + bn <= mi * tm;
}


// One 32-column chunk of one output row: f[] holds alpha * accumulator for columns c0..c0+31 of row r.
template <int BN, int TM = BM>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, float (&f)[32], int r, int c0, bool partial,
                                               uint8_t* cbase, const uint8_t* cinbase) {
  const bool full = (c0 + 32 <= p.N);
  // debug build: the row must lie inside the output and the column chunk must start inside it
  if (!SR_DEBUG_CHECK(r >= 0 && r < p.M && c0 >= 0 && c0 < p.N, p.status, 4100, r)) return;
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
    return;
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
      if (c < p.N && c > r && sym_tile_skipped(c, r, BN, TM)) {
        if (p.c_fp32)
          reinterpret_cast<float*>(cbase)[(size_t)c * p.ldc + r] = f[j];
        else
          reinterpret_cast<__nv_bfloat16*>(cbase)[(size_t)c * p.ldc + r] = __float2bfloat16(f[j]);
      }
    }
  }
}

}  // namespace

namespace {
// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved once per process, by sr_runtime_init() (gemm_tcgen05.cu), which the Python
// loader calls from the main thread right after it has opened the library: every translation unit and every thread
// (autograd runs backward passes on its own) then shares the same pointer.
extern "C" void* sr_driver_encode_tiled(void);

// The encoder is a driver-API call and wants the device's context current on the calling thread. A thread whose first
// CUDA activity is one of these launchers (autograd's worker, when the loss is the direct output of an op of this
// library) has not bound it yet: one no-op runtime call per thread does.
inline EncodeTiledFn get_encode_fn() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  return reinterpret_cast<EncodeTiledFn>(sr_driver_encode_tiled());
}

inline int report_encode_failure(CUresult r, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                                 const cuuint32_t* box) {
  fprintf(stderr, "slowrun_b200: cuTensorMapEncodeTiled failed with CUresult %d (ptr %p, dims %llu x %llu x %llu, "
                  "strides %llu %llu, box %u x %u)\n", (int)r, ptr, (unsigned long long)dims[0],
          (unsigned long long)dims[1], (unsigned long long)dims[2], (unsigned long long)strides[0],
          (unsigned long long)strides[1], box[0], box[1]);
  return -3;
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
  return r == CUDA_SUCCESS ? 0 : report_encode_failure(r, ptr, dims, strides, box);
}

// Same for 1-byte (fp8) elements: {inner, rows, batch} with the leading dimension given in elements (= bytes).
int encode_u8_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t ld,
                  uint64_t batch_stride, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((ld % 16) != 0 || (reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return -2;
  if (batch > 1 && (batch_stride % 16) != 0) return -2;
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {ld, (batch > 1 ? batch_stride : rows * ld)};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : report_encode_failure(r, ptr, dims, strides, box);
}

inline int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}


}  // namespace
