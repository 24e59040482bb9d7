// Collectives fused with their consumers, over NVLink peer memory: plain P2P loads, or multimem.ld_reduce through the
// NVSwitch for the gradient sum when the buffer has a multicast mapping; never TMA on remote memory. Every rank maps
// every peer's symmetric buffers; kernels take a small device array of W base pointers.
//
//   peer_barrier          all-ranks barrier on symmetric flag words, monotonic epochs, bounded wait -> status word.
//                         When a wait runs out the status word becomes non-zero; every consumer kernel below reads
//                         it first and returns without writing, so a step whose barrier failed changes no state.
//   muon_pre_multi        gradient reduce-scatter fused with the Muon prologue: the owner of a matrix reads that
//                         matrix's gradient rows from all W ranks, sums and scales them, updates momentum, applies
//                         Nesterov + row normalisation and writes the bf16 Newton-Schulz input directly
//                         (reference: reduce_scatter_tensor then muon_step_fused, train.py:671-683, 603-613)
//   muon_apply_multi      all-gather of the orthogonalised update fused with the cautious-weight-decay apply: every
//                         rank reads each owner's bf16 update chunk in place and updates its own fp32 replica and
//                         bf16 shadow (reference: all_gather_into_tensor of fp32 parameters + copy, train.py:742-760)
//   bcast_multi           the other form of that all-gather, for buffers with a multicast mapping: the owner pushes its
//                         bf16 update chunk with multimem.st (one store, replicated by the switch into every rank's
//                         copy of the gathered buffer); after the barrier every rank applies from its own memory.
//                         Stores need no round trip, so the transfer is bound by the links and not by the number of
//                         loads an SM can keep in flight.
//   reduce_multi          out = sum over ranks of src_r[offset : offset+n]  (row-slice reduce-scatter for the AdamW
//                         parameters, and the one-shot all-reduce of the packed small-parameter gradients)
//   gather_multi          pull every other rank's slice of a sharded parameter into the local replica
#include "sm100_common.cuh"

namespace {

using namespace sr;

constexpr int kMaxWorld = 16;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct PtrTable {
  const void* p[kMaxWorld];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// flags: on every rank an array uint32[W]; slot s of rank d is written only by rank s.
// mode 0: announce `epoch` to every rank, then wait until every rank has announced it (a barrier);
// mode 1: announce only (a signal: "my work up to `epoch` is done and visible");  mode 2: wait only.
__global__ void peer_barrier_kernel(PtrTable flags, int rank, int world, uint32_t epoch, int* status,
                                    unsigned long long limit_ns, int mode) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  if (mode != 2) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(const_cast<void*>(flags.p[t])) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  if (mode == 1) return;
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + t;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((++it & 255u) == 0u && globaltimer_ns() - t0 > limit_ns) {
      report_error(status, SR_ERR_PEER_TIMEOUT, 900, t);
      break;
    }
  }
  __threadfence_system();
}

// One warp per row of the owned stack. G_r points at rank r's full gradient arena of this group; `base` is the element
// offset of the owned chunk inside it. Pass 1 pulls the row from every rank (two column steps of W independent 16-byte
// loads per lane are issued before any is consumed, so a warp keeps W KB in flight over NVLink), reduces it, updates the
// momentum and parks the Nesterov gradient in this rank's own copy of the row (dead once reduced; the other ranks only
// read the rows of their own chunks). Pass 2 rereads it from L2, applies the row norm and writes the bf16 input of the
// Newton-Schulz iteration.
constexpr int kPullWorld = 8;   // peers handled by the unrolled load stage; larger worlds take extra rounds

// sum over all ranks of the 16 bytes at this multicast address, reduced inside the NVSwitch (NVLS): one load returns
// what W peer loads would, and only 1/W of the bytes cross this GPU's links
__device__ __forceinline__ float4 multimem_sum_f32x4(const float* mc_addr) {
  float4 v;
  // no memory clobber: the data was published by the barrier that precedes the kernel, and the compiler is free
  // to keep several of these in flight around the surrounding arithmetic
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr));
  return v;
}

// same for a bf16 wire buffer: 16 bytes = eight gradients, summed in fp32 inside the switch, returned rounded to bf16
__device__ __forceinline__ void multimem_sum_bf16x8(const __nv_bfloat16* mc_addr, float (&f)[8]) {
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(mc_addr));
  const uint32_t w[4] = {a, b, c, d};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ void add_bf16x8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] += v.x;
    f[2 * i + 1] += v.y;
  }
}

// W16 = false: G_r are the ranks' fp32 gradient arenas. W16 = true: G_r (and mc) are bf16 copies of them (the wire
// format: half the bytes over NVLink); `park` is then this rank's own fp32 arena, used as scratch as before.
template <bool W16>
__global__ void __launch_bounds__(kThreads, 2)
muon_pre_multi_kernel(PtrTable G, const void* __restrict__ mc_v, float* __restrict__ park_base, int world, int rank,
                      long base, float* __restrict__ Mom,
                      __nv_bfloat16* __restrict__ X, float* __restrict__ sumsq, long rows_total, int r, int c, float mu,
                      float gscale, int row_norm, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;   // a barrier gave up: touch nothing
  // debug build: every peer's rows must start on a 16-byte boundary (the pulls are 16-byte vector loads)
  {
    const size_t esz = W16 ? 2 : 4;
    bool aligned = ((static_cast<size_t>(base) * esz) & 15) == 0 && ((static_cast<size_t>(c) * esz) & 15) == 0;
    for (int w = 0; w < world; ++w) aligned = aligned && (reinterpret_cast<uintptr_t>(G.p[w]) & 15) == 0;
    if (!SR_DEBUG_CHECK(aligned, const_cast<int*>(status), 4200, c)) return;
  }
  const int lane = threadIdx.x & 31;
  const float* mc = W16 ? nullptr : reinterpret_cast<const float*>(mc_v);
  const __nv_bfloat16* mc16 = W16 ? reinterpret_cast<const __nv_bfloat16*>(mc_v) : nullptr;
  // at most one CTA per SM (the launcher caps the grid): the kernel is meant to share the SMs with the Newton-Schulz
  // GEMMs of the neighbouring shape group, which need one CTA's worth of registers and shared memory on every SM
  for (long row = (long)blockIdx.x * kWarps + (threadIdx.x >> 5); row < rows_total; row += (long)gridDim.x * kWarps) {
    float* m = Mom + row * c;
    __nv_bfloat16* x = X + row * c;
    const long off = base + row * c;
    float* park = park_base + off;
    float ss = 0.f;
    // momentum update + Nesterov gradient of four reduced columns; the Nesterov value is parked in the local row
    auto consume = [&](int j, float4 gv) {
      gv.x *= gscale; gv.y *= gscale; gv.z *= gscale; gv.w *= gscale;
      float4 mv = *reinterpret_cast<const float4*>(m + j);
      mv.x += (1.f - mu) * (gv.x - mv.x); mv.y += (1.f - mu) * (gv.y - mv.y);
      mv.z += (1.f - mu) * (gv.z - mv.z); mv.w += (1.f - mu) * (gv.w - mv.w);
      *reinterpret_cast<float4*>(m + j) = mv;
      float4 nv;
      nv.x = gv.x + mu * (mv.x - gv.x); nv.y = gv.y + mu * (mv.y - gv.y);
      nv.z = gv.z + mu * (mv.z - gv.z); nv.w = gv.w + mu * (mv.w - gv.w);
      ss += nv.x * nv.x + nv.y * nv.y + nv.z * nv.z + nv.w * nv.w;
      *reinterpret_cast<float4*>(park + j) = nv;
    };
    if (W16) {
      auto consume8 = [&](int j, const float (&f)[8]) {
        consume(j, make_float4(f[0], f[1], f[2], f[3]));
        consume(j + 4, make_float4(f[4], f[5], f[6], f[7]));
      };
      if (mc16 != nullptr) {
        // NVLS: four in-switch reductions of eight gradients each in flight per lane
        for (int j0 = lane * 8; j0 < c; j0 += 1024) {
          float g[4][8];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + u * 256 < c) multimem_sum_bf16x8(mc16 + off + j0 + u * 256, g[u]);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (j0 + u * 256 < c) consume8(j0 + u * 256, g[u]);
        }
      } else {
        for (int j0 = lane * 8; j0 < c; j0 += 512) {
          const int j1 = j0 + 256;
          const bool has1 = j1 < c;
          float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int p0 = 0; p0 < world; p0 += kPullWorld) {
            uint4 t0[kPullWorld], t1[kPullWorld];
#pragma unroll
            for (int p = 0; p < kPullWorld; ++p) {
              if (p0 + p < world) {
                const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(G.p[p0 + p]) + off;
                t0[p] = *reinterpret_cast<const uint4*>(src + j0);
                if (has1) t1[p] = *reinterpret_cast<const uint4*>(src + j1);
              }
            }
#pragma unroll
            for (int p = 0; p < kPullWorld; ++p) {
              if (p0 + p < world) {
                add_bf16x8(t0[p], a0);
                if (has1) add_bf16x8(t1[p], a1);
              }
            }
          }
          consume8(j0, a0);
          if (has1) consume8(j1, a1);
        }
      }
    } else if (mc != nullptr) {
      // NVLS path: eight independent in-switch reductions in flight per lane
      for (int j0 = lane * 4; j0 < c; j0 += 1024) {
        float4 g[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (j0 + u * 128 < c) g[u] = multimem_sum_f32x4(mc + off + j0 + u * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (j0 + u * 128 < c) consume(j0 + u * 128, g[u]);
      }
    } else {
      for (int j0 = lane * 4; j0 < c; j0 += 256) {
        const int j1 = j0 + 128;
        const bool has1 = j1 < c;
        float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
        for (int p0 = 0; p0 < world; p0 += kPullWorld) {
          float4 t0[kPullWorld], t1[kPullWorld];
#pragma unroll
          for (int p = 0; p < kPullWorld; ++p) {
            if (p0 + p < world) {
              const float* src = reinterpret_cast<const float*>(G.p[p0 + p]) + off;
              t0[p] = *reinterpret_cast<const float4*>(src + j0);
              if (has1) t1[p] = *reinterpret_cast<const float4*>(src + j1);
            }
          }
#pragma unroll
          for (int p = 0; p < kPullWorld; ++p) {
            if (p0 + p < world) {
              g0.x += t0[p].x; g0.y += t0[p].y; g0.z += t0[p].z; g0.w += t0[p].w;
              if (has1) { g1.x += t1[p].x; g1.y += t1[p].y; g1.z += t1[p].z; g1.w += t1[p].w; }
            }
          }
        }
        consume(j0, g0);
        if (has1) consume(j1, g1);
      }
    }
    ss = warp_sum(ss);
    const float inv = row_norm ? 1.f / fmaxf(sqrtf(ss), 1e-7f) : 1.f;
    float xs = 0.f;
    for (int j = lane * 4; j < c; j += 128) {
      const float4 nv = *reinterpret_cast<const float4*>(park + j);   // written by this same lane above
      const __nv_bfloat162 lo = __floats2bfloat162_rn(nv.x * inv, nv.y * inv);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(nv.z * inv, nv.w * inv);
      *reinterpret_cast<__nv_bfloat162*>(x + j) = lo;
      *reinterpret_cast<__nv_bfloat162*>(x + j + 2) = hi;
      const float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
      xs += l.x * l.x + l.y * l.y + h.x * h.x + h.y * h.y;
    }
    xs = warp_sum(xs);
    if (lane == 0) atomicAdd(sumsq + row / r, xs);
  }
}

__global__ void fnorm_scale_kernel(__nv_bfloat16* __restrict__ X, const float* __restrict__ sumsq, long per_mat,
                                   long total, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < total; i += (long)gridDim.x * blockDim.x * 2) {
    const float s = 1.f / (1.02f * sqrtf(sumsq[i / per_mat]) + 1e-6f);
    const float2 v = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(X + i));
    *reinterpret_cast<__nv_bfloat162*>(X + i) = __floats2bfloat162_rn(v.x * s, v.y * s);
  }
}

// U_r points at rank r's update chunk [chunk_elems]; element i of the stack belongs to rank i / chunk_elems.
__global__ void muon_apply_multi_kernel(float* __restrict__ P, PtrTable U, long chunk_elems,
                                        __nv_bfloat16* __restrict__ shadow, float lr_b, float lrwd_b, long total,
                                        const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += (long)gridDim.x * blockDim.x * 4) {
    const long owner = i / chunk_elems;
    const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(U.p[owner]) + (i - owner * chunk_elems);
    float4 p = *reinterpret_cast<float4*>(P + i);
    const uint2 raw = *reinterpret_cast<const uint2*>(u);
    const float2 u0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 u1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    p.x -= bf16_round(lr_b * u0.x) + ((u0.x * p.x >= 0.f) ? lrwd_b * p.x : 0.f);
    p.y -= bf16_round(lr_b * u0.y) + ((u0.y * p.y >= 0.f) ? lrwd_b * p.y : 0.f);
    p.z -= bf16_round(lr_b * u1.x) + ((u1.x * p.z >= 0.f) ? lrwd_b * p.z : 0.f);
    p.w -= bf16_round(lr_b * u1.y) + ((u1.y * p.w >= 0.f) ? lrwd_b * p.w : 0.f);
    *reinterpret_cast<float4*>(P + i) = p;
    if (shadow != nullptr) {
      *reinterpret_cast<__nv_bfloat162*>(shadow + i) = __floats2bfloat162_rn(p.x, p.y);
      *reinterpret_cast<__nv_bfloat162*>(shadow + i + 2) = __floats2bfloat162_rn(p.z, p.w);
    }
  }
}

// Same update, eight elements per thread and two independent groups per iteration: 16-byte peer loads and four times
// the bytes in flight per thread (the kernel is bound by the latency of the remote reads otherwise).
__device__ __forceinline__ void apply8(float* __restrict__ P, const uint4& raw, __nv_bfloat16* __restrict__ shadow, long i,
                                       float lr_b, float lrwd_b) {
  float4 p0 = *reinterpret_cast<float4*>(P + i), p1 = *reinterpret_cast<float4*>(P + i + 4);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 u0 = __bfloat1622float2(h[0]), u1 = __bfloat1622float2(h[1]), u2 = __bfloat1622float2(h[2]),
               u3 = __bfloat1622float2(h[3]);
  p0.x -= bf16_round(lr_b * u0.x) + ((u0.x * p0.x >= 0.f) ? lrwd_b * p0.x : 0.f);
  p0.y -= bf16_round(lr_b * u0.y) + ((u0.y * p0.y >= 0.f) ? lrwd_b * p0.y : 0.f);
  p0.z -= bf16_round(lr_b * u1.x) + ((u1.x * p0.z >= 0.f) ? lrwd_b * p0.z : 0.f);
  p0.w -= bf16_round(lr_b * u1.y) + ((u1.y * p0.w >= 0.f) ? lrwd_b * p0.w : 0.f);
  p1.x -= bf16_round(lr_b * u2.x) + ((u2.x * p1.x >= 0.f) ? lrwd_b * p1.x : 0.f);
  p1.y -= bf16_round(lr_b * u2.y) + ((u2.y * p1.y >= 0.f) ? lrwd_b * p1.y : 0.f);
  p1.z -= bf16_round(lr_b * u3.x) + ((u3.x * p1.z >= 0.f) ? lrwd_b * p1.z : 0.f);
  p1.w -= bf16_round(lr_b * u3.y) + ((u3.y * p1.w >= 0.f) ? lrwd_b * p1.w : 0.f);
  *reinterpret_cast<float4*>(P + i) = p0;
  *reinterpret_cast<float4*>(P + i + 4) = p1;
  if (shadow != nullptr) {
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
    oh[0] = __floats2bfloat162_rn(p0.x, p0.y); oh[1] = __floats2bfloat162_rn(p0.z, p0.w);
    oh[2] = __floats2bfloat162_rn(p1.x, p1.y); oh[3] = __floats2bfloat162_rn(p1.z, p1.w);
    *reinterpret_cast<uint4*>(shadow + i) = o;
  }
}
__global__ void muon_apply_multi8_kernel(float* __restrict__ P, PtrTable U, long chunk_elems,
                                         __nv_bfloat16* __restrict__ shadow, float lr_b, float lrwd_b, long total,
                                         const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const long stride = (long)gridDim.x * blockDim.x * 8;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += 2 * stride) {
    const long i2 = i + stride;
    const bool has2 = i2 < total;
    const long o1 = i / chunk_elems;
    const uint4 r1 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(U.p[o1]) + (i - o1 * chunk_elems));
    uint4 r2 = make_uint4(0, 0, 0, 0);
    if (has2) {
      const long o2 = i2 / chunk_elems;
      r2 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(U.p[o2]) + (i2 - o2 * chunk_elems));
    }
    apply8(P, r1, shadow, i, lr_b, lrwd_b);
    if (has2) apply8(P, r2, shadow, i2, lr_b, lrwd_b);
  }
}

// Owner -> all ranks: src (this rank's memory, n 16-byte vectors) is written through the multicast address `mc_dst`, so
// the same bytes land at the same offset of the symmetric buffer on every rank, this one included.
__global__ void bcast_multi_kernel(const uint4* __restrict__ src, uint4* mc_dst, long n, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst + i), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
  }
}

template <bool BF16>
__global__ void reduce_multi_kernel(PtrTable src, int world, long offset, float* __restrict__ out, long n,
                                    const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long)gridDim.x * blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i + 3 < n) {
      for (int p = 0; p < world; ++p) {
        if (BF16) {
          const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(src.p[p]) + offset + i);
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
        } else {
          const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[p]) + offset + i);
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
      }
      *reinterpret_cast<float4*>(out + i) = acc;
    } else {
      for (long j = i; j < n; ++j) {
        float a = 0.f;
        for (int p = 0; p < world; ++p)
          a += BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src.p[p])[offset + j])
                    : reinterpret_cast<const float*>(src.p[p])[offset + j];
        out[j] = a;
      }
    }
  }
}

// bufs[r] = rank r's replica (same layout everywhere); copy slice s (bytes [s*slice, (s+1)*slice)) from rank s for all s != rank
__global__ void gather_multi_kernel(PtrTable bufs, int world, int rank, long slice_bytes, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const long vecs = slice_bytes / 16;
  const int s = blockIdx.y;
  if (s == rank) return;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(bufs.p[s]) + (long)s * slice_bytes);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(const_cast<void*>(bufs.p[rank])) + (long)s * slice_bytes);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long)gridDim.x * blockDim.x) dst[i] = src[i];
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}
inline int grid_for(long n, int per_block) {
  long b = (n + per_block - 1) / per_block;
  const long cap = (long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
inline int rc() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }

inline bool fill(PtrTable& t, const unsigned long long* ptrs, int world) {
  if (world < 1 || world > kMaxWorld) return false;
  for (int i = 0; i < world; ++i) t.p[i] = reinterpret_cast<const void*>(ptrs[i]);
  return true;
}

}  // namespace

// `ptrs` arguments are HOST arrays of `world` device addresses (one per rank, this rank's own included).
// `status` arguments are the device int[4] status word (sm100_common.cuh); consumer kernels return at once when it is
// non-zero. `limit_ns`: how long the barrier waits for each peer before it records SR_ERR_PEER_TIMEOUT (site 900,
// detail = the peer) and returns; 0 selects the library default.
extern "C" int sr_peer_barrier(const unsigned long long* flag_ptrs, int rank, int world, unsigned int epoch, int* status,
                               unsigned long long limit_ns, cudaStream_t s) {
  PtrTable t;
  if (!fill(t, flag_ptrs, world)) return -2;
  peer_barrier_kernel<<<1, 32, 0, s>>>(t, rank, world, epoch, status, limit_ns ? limit_ns : kWaitLimitNs, 0);
  return rc();
}
// The two halves of the barrier as separate launches, on a second flag array of monotonically growing progress
// counters: a rank signals "everything I enqueued before this on this stream is done" with a value, and a consumer on
// any stream waits (bounded, same status reporting, site 900) until every rank's counter has reached a value.
extern "C" int sr_peer_signal(const unsigned long long* flag_ptrs, int rank, int world, unsigned int value, cudaStream_t s) {
  PtrTable t;
  if (!fill(t, flag_ptrs, world)) return -2;
  peer_barrier_kernel<<<1, 32, 0, s>>>(t, rank, world, value, nullptr, 0, 1);
  return rc();
}
extern "C" int sr_peer_wait(const unsigned long long* flag_ptrs, int rank, int world, unsigned int value, int* status,
                            unsigned long long limit_ns, cudaStream_t s) {
  PtrTable t;
  if (!fill(t, flag_ptrs, world)) return -2;
  peer_barrier_kernel<<<1, 32, 0, s>>>(t, rank, world, value, status, limit_ns ? limit_ns : kWaitLimitNs, 2);
  return rc();
}

// `rank`: index of the calling rank in g_ptrs. `park`: this rank's own fp32 gradient arena of the group; its copy of the
// owned rows is overwritten (used as scratch). `wire_bf16`: g_ptrs / mc address bf16 copies of the arenas (c % 8 == 0).
// `mc`: multicast (NVLS) address of the same symmetric buffer, or null for plain peer loads.
// `shared_sms`: 1 = at most one CTA per SM (the kernel runs beside the Newton-Schulz GEMMs on another stream),
// 0 = two CTAs per SM (it has the GPU to itself).
extern "C" int sr_muon_pre_multi(const unsigned long long* g_ptrs, const void* mc, float* park, int wire_bf16, int world,
                                 int rank, long base, float* Mom, void* X,
                                 float* sumsq, int n, int r, int c, float mu, float gscale, int row_norm, int shared_sms,
                                 const int* status, cudaStream_t s) {
  if (n <= 0) return 0;
  if (c % 4 || rank < 0 || rank >= world || park == nullptr) return -2;
  if (wire_bf16 && c % 8) return -2;
  PtrTable t;
  if (!fill(t, g_ptrs, world)) return -2;
  const long rows = (long)n * r;
  cudaMemsetAsync(sumsq, 0, sizeof(float) * n, s);
  long pull_grid = (rows + kWarps - 1) / kWarps;
  const long cap = shared_sms ? sm_count() : 2L * sm_count();
  if (pull_grid > cap) pull_grid = cap;
  if (wire_bf16)
    muon_pre_multi_kernel<true><<<(unsigned)pull_grid, kThreads, 0, s>>>(
        t, mc, park, world, rank, base, Mom, reinterpret_cast<__nv_bfloat16*>(X), sumsq, rows, r, c, mu, gscale, row_norm, status);
  else
    muon_pre_multi_kernel<false><<<(unsigned)pull_grid, kThreads, 0, s>>>(
        t, mc, park, world, rank, base, Mom, reinterpret_cast<__nv_bfloat16*>(X), sumsq, rows, r, c, mu, gscale, row_norm, status);
  const long total = rows * c;
  fnorm_scale_kernel<<<grid_for(total / 2, kThreads), kThreads, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(X), sumsq, (long)r * c, total, status);
  return rc();
}

extern "C" int sr_muon_apply_multi(float* P, const unsigned long long* u_ptrs, int world, long chunk_elems, void* shadow,
                                   long total, float lr_b, float lrwd_b, const int* status, cudaStream_t s) {
  if (total <= 0) return 0;
  if (total % 4 || chunk_elems % 4) return -2;
  PtrTable t;
  if (!fill(t, u_ptrs, world)) return -2;
  if (total % 8 == 0 && chunk_elems % 8 == 0)
    muon_apply_multi8_kernel<<<grid_for(total / 16, kThreads), kThreads, 0, s>>>(P, t, chunk_elems, reinterpret_cast<__nv_bfloat16*>(shadow), lr_b, lrwd_b, total, status);
  else
    muon_apply_multi_kernel<<<grid_for(total / 4, kThreads), kThreads, 0, s>>>(P, t, chunk_elems, reinterpret_cast<__nv_bfloat16*>(shadow), lr_b, lrwd_b, total, status);
  return rc();
}

// Pushes `bytes` bytes (a multiple of 16, 16-byte aligned on both sides) from `src` into every rank's copy of a
// symmetric buffer through its multicast address `mc_dst`. `max_ctas` > 0 caps the grid (to leave SMs to a GEMM running
// beside it). The data is visible on the peers after the next peer barrier on the same stream.
extern "C" int sr_bcast_multi(const void* src, void* mc_dst, long bytes, int max_ctas, const int* status, cudaStream_t s) {
  if (bytes <= 0) return 0;
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(mc_dst) & 15) || mc_dst == nullptr)
    return -2;
  const long n = bytes / 16;
  long grid = (n + kThreads - 1) / kThreads;
  const long cap = max_ctas > 0 ? max_ctas : 4L * sm_count();
  if (grid > cap) grid = cap;
  bcast_multi_kernel<<<(unsigned)grid, kThreads, 0, s>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(mc_dst), n,
                                                         status);
  return rc();
}

extern "C" int sr_reduce_multi(const unsigned long long* src_ptrs, int world, long offset, float* out, long n,
                               int src_bf16, const int* status, cudaStream_t s) {
  if (n <= 0) return 0;
  if (offset % 4) return -2;
  PtrTable t;
  if (!fill(t, src_ptrs, world)) return -2;
  if (src_bf16)
    reduce_multi_kernel<true><<<grid_for((n + 3) / 4, kThreads), kThreads, 0, s>>>(t, world, offset, out, n, status);
  else
    reduce_multi_kernel<false><<<grid_for((n + 3) / 4, kThreads), kThreads, 0, s>>>(t, world, offset, out, n, status);
  return rc();
}

extern "C" int sr_gather_multi(const unsigned long long* buf_ptrs, int world, int rank, long slice_bytes,
                               const int* status, cudaStream_t s) {
  if (slice_bytes <= 0) return 0;
  if (slice_bytes % 16) return -2;
  PtrTable t;
  if (!fill(t, buf_ptrs, world)) return -2;
  dim3 grid(grid_for(slice_bytes / 16, kThreads) / 2 + 1, world);
  gather_multi_kernel<<<grid, kThreads, 0, s>>>(t, world, rank, slice_bytes, status);
  return rc();
}
