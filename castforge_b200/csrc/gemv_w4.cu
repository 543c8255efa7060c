// W4A16 decode GEMM (M <= 16): C[m,n] = sum_k A[m,k] * (q[n,k] - zp[n,g]) * s[n,g], HBM-bound on W.
//
// The packed INT4 weights are streamed exactly once with 128-bit loads; everything else is sized
// to stay out of the way of that stream.
//  * Tensor cores (mma.sync m16n8k16, bf16 -> f32) do the multiply-adds with the WEIGHT tile as
//    the 16-row operand (16 output channels) and the activations as the 8-column operand (8
//    tokens), so M = 1..8 costs one instruction per 16x16 weight block and M = 9..16 two.
//  * The k index a fragment slot stands for is free as long as both operands agree, so a lane
//    keeps the 32 consecutive k of its own 16-byte load: one LOP3 turns the nibbles (i, i+4) of
//    a word into a bf16 pair 128+q (0x4300 | q), one HSUB2 removes 128+zp exactly.  The group
//    scale is applied to the f32 partial sum of the 128-k group, so the dequantisation is exact.
//  * K is split over the 8 CTAs of a thread-block cluster, so a CTA stages only its own eighth of
//    the activations (a few KB, already permuted into fragment order and laid out so that a
//    quarter-warp reads 128 contiguous bytes) and reuses it for every output channel it owns.
//  * Each of a CTA's 4 warps owns up to 4 tiles of 16 output channels and keeps 4 work items
//    (16 rows x 128 k) of loads in flight; there is no block-wide barrier in the weight stream.
//  * The 8 partial sums of an output meet over distributed shared memory after one cluster
//    barrier: deterministic, no atomics, no workspace, one launch.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace cfb {
namespace {

constexpr int kWarps = 4;
constexpr int kThreadsGv = kWarps * 32;
constexpr int kChunk = 128;    // k per work item = one quantisation group
constexpr int kMaxTiles = 4;   // 16-channel tiles owned by one warp
constexpr int kMaxCluster = 8; // up to 8 CTAs of a cluster split K; their partial sums meet over DSMEM

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm(  // not volatile: independent accumulation chains may be interleaved by the scheduler
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two bf16 -> two f16 (round to nearest, saturating at +-65504; NaN stays NaN)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
  lo = (lo != lo) ? lo : fminf(fmaxf(lo, -65504.0f), 65504.0f);
  hi = (hi != hi) ? hi : fminf(fmaxf(hi, -65504.0f), 65504.0f);
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// nibbles (i, i+4) of w as the bf16 pair (128+q_i, 128+q_{i+4}) minus the pair (128+zp, 128+zp)
__device__ __forceinline__ uint32_t deq_pair(uint32_t w, int i, uint32_t zpc) {
  const uint32_t x = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
  const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x), *reinterpret_cast<const __nv_bfloat162*>(&zpc));
  return *reinterpret_cast<const uint32_t*>(&r);
}

struct GvArgs {
  const __nv_bfloat16* act;  // [M, K]
  const uint8_t* codes;      // [N, K/2]
  const uint16_t* scales;    // [N, K/128]
  const uint8_t* zps;        // nibbles, flat group index
  int M, N, K;
  void* C;                   // [M, N]
  int out_f32;
};

// Stage rows 0..8*MT-1 of the activations, chunks [c0, c0 + nchunks) of 128 k, into shared memory
// in fragment order: within each 8-group the elements are stored as (k0,k4)(k1,k5)(k2,k6)(k3,k7),
// and the 16 groups of a chunk are transposed 4x4 so that lane t, word j finds its group at slot
// 4j+t (a quarter-warp then reads 128 contiguous bytes; rows are 64 mod 128 bytes apart).
template <int MT, bool F16 = false>
__device__ __forceinline__ void stage_acts(const GvArgs& a, uint8_t* buf, int c0, int nchunks, int pitch) {
  const int groups = nchunks * 16;  // 8-groups per row
  for (int item = threadIdx.x; item < 8 * MT * groups; item += blockDim.x) {
    const int row = item / groups, grp = item % groups;
    const int k = c0 * kChunk + grp * 8;
    const uint4 r = (row < a.M && k < a.K) ? __ldg(reinterpret_cast<const uint4*>(a.act + (size_t)row * a.K + k)) : make_uint4(0, 0, 0, 0);
    const int chunk = grp >> 4, L = grp & 15;
    const int slot = ((L & 3) << 2) | (L >> 2);
    uint4 o;
    o.x = __byte_perm(r.x, r.z, 0x5410);
    o.y = __byte_perm(r.x, r.z, 0x7632);
    o.z = __byte_perm(r.y, r.w, 0x5410);
    o.w = __byte_perm(r.y, r.w, 0x7632);
    if (F16) {
      o.x = bf16x2_to_f16x2(o.x);
      o.y = bf16x2_to_f16x2(o.y);
      o.z = bf16x2_to_f16x2(o.z);
      o.w = bf16x2_to_f16x2(o.w);
    }
    *reinterpret_cast<uint4*>(buf + (size_t)row * pitch + chunk * 256 + slot * 16) = o;
  }
}

struct WItem {
  uint4 w[2];    // rows g and g+8 of the tile: 32 codes each
  float s[2];
  uint32_t z[2];
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const float* local, uint32_t rank) {
  const uint32_t la = (uint32_t)__cvta_generic_to_shared(local);
  uint32_t ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra));
  return v;
}

// grid.x = clusters * csize.  A cluster owns kWarps * tiles_per_warp tiles of 16 output channels;
// CTA `rank` of the cluster owns chunks [rank*cpc, rank*cpc + cpc) of K for all of them.
#ifdef CFB_GV_TRACE
// wall-clock stamps (%globaltimer, ns) of every CTA of the register-ring kernel, for builds made with -DCFB_GV_TRACE only
__device__ unsigned long long g_gvstamp[1024 * 4];
__device__ __forceinline__ void gv_stamp(int slot) {
  if (threadIdx.x == 0 && blockIdx.x < 1024) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_gvstamp[blockIdx.x * 4 + slot] = t;
  }
}
#define GV_STAMP(slot) gv_stamp(slot)
#else
#define GV_STAMP(slot) do { } while (0)
#endif

template <int MT>
__global__ void __launch_bounds__(kThreadsGv)
gemv_w4_kernel(const GvArgs a, int tiles_per_warp, int cpc /* chunks per CTA */, int pitch, int csize /* CTAs per cluster */) {
  extern __shared__ __align__(128) uint8_t smem[];
  GV_STAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t rank = cluster_rank();
  const int cluster_id = blockIdx.x / csize;
  const int gpr = a.K / kChunk;
  const int c0 = (int)rank * cpc;
  const int rows_per_cluster = kWarps * tiles_per_warp * 16;
  const int row0 = cluster_id * rows_per_cluster;  // first output channel of the cluster
  constexpr int kCols = 8 * MT;
  float* part = reinterpret_cast<float*>(smem + (size_t)8 * MT * pitch);  // [rows_per_cluster][kCols]

  float total[kMaxTiles][MT][4];
#pragma unroll
  for (int ti = 0; ti < kMaxTiles; ++ti)
#pragma unroll
    for (int mh = 0; mh < MT; ++mh)
#pragma unroll
      for (int i = 0; i < 4; ++i) total[ti][mh][i] = 0.0f;

  const int nitems = tiles_per_warp * cpc;
  auto fetch = [&](int it, WItem& wi) {
    const int ti = it / cpc, cc = it % cpc;
    const int c = c0 + cc;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = row0 + (ti * kWarps + warp) * 16 + h * 8 + g;
      if (it < nitems && n < a.N && c < gpr) {
        wi.w[h] = ld_stream16(a.codes + (size_t)n * (a.K / 2) + (size_t)c * (kChunk / 2) + t * 16);
        const size_t gi = (size_t)n * gpr + c;
        wi.s[h] = __half2float(__ushort_as_half(__ldg(a.scales + gi)));
        const uint32_t zp = (__ldg(a.zps + (gi >> 1)) >> ((gi & 1) * 4)) & 0xFu;
        wi.z[h] = (0x4300u | zp) * 0x00010001u;  // bf16 pair (128+zp, 128+zp)
      } else {
        wi.w[h] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
        wi.s[h] = 0.0f;
        wi.z[h] = 0x43084308u;  // q = zp = 8: exact zeros
      }
    }
  };
  constexpr int kDepth = 4;  // work items (16 rows x 128 k) in flight per warp
  WItem ring[kDepth];
#pragma unroll
  for (int d = 0; d < kDepth; ++d) fetch(d, ring[d]);
  // the first weights are on their way while the activations are staged
  stage_acts<MT>(a, smem, c0, cpc, pitch);
  __syncthreads();
  GV_STAMP(1);
  for (int it0 = 0; it0 < nitems; it0 += kDepth) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int it = it0 + d;
      const WItem cur = ring[d];
      fetch(it + kDepth, ring[d]);
      if (it >= nitems) continue;
      const int ti = it / cpc, cc = it % cpc;
      const uint8_t* abase = smem + (size_t)cc * 256;
      float accg[MT][4];
#pragma unroll
      for (int mh = 0; mh < MT; ++mh)
#pragma unroll
        for (int i = 0; i < 4; ++i) accg[mh][i] = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t wa = (&cur.w[0].x)[j], wb = (&cur.w[1].x)[j];
        const uint32_t ra0 = deq_pair(wa, 0, cur.z[0]), ra1 = deq_pair(wa, 1, cur.z[0]);
        const uint32_t ra2 = deq_pair(wa, 2, cur.z[0]), ra3 = deq_pair(wa, 3, cur.z[0]);
        const uint32_t rb0 = deq_pair(wb, 0, cur.z[1]), rb1 = deq_pair(wb, 1, cur.z[1]);
        const uint32_t rb2 = deq_pair(wb, 2, cur.z[1]), rb3 = deq_pair(wb, 3, cur.z[1]);
#pragma unroll
        for (int mh = 0; mh < MT; ++mh) {
          const uint4 x = *reinterpret_cast<const uint4*>(abase + (size_t)(mh * 8 + g) * pitch + (4 * j + t) * 16);
          mma_bf16_16816(accg[mh], ra0, rb0, ra1, rb1, x.x, x.y);
          mma_bf16_16816(accg[mh], ra2, rb2, ra3, rb3, x.z, x.w);
        }
      }
      // group scale on the f32 group sum (static switch keeps the totals in registers)
#pragma unroll
      for (int tt = 0; tt < kMaxTiles; ++tt)
        if (tt == ti) {
#pragma unroll
          for (int mh = 0; mh < MT; ++mh) {
            total[tt][mh][0] = __fmaf_rn(cur.s[0], accg[mh][0], total[tt][mh][0]);
            total[tt][mh][1] = __fmaf_rn(cur.s[0], accg[mh][1], total[tt][mh][1]);
            total[tt][mh][2] = __fmaf_rn(cur.s[1], accg[mh][2], total[tt][mh][2]);
            total[tt][mh][3] = __fmaf_rn(cur.s[1], accg[mh][3], total[tt][mh][3]);
          }
        }
    }
  }

  // Reduction over the cluster's K split.  Every CTA finishes `share` of the cluster's rows: the others PUSH their partial
  // sums for those rows into its shared memory (slot = sender's rank; posted stores over DSMEM), one cluster barrier makes
  // them visible, and the owner adds the slots up from its own memory.  (Pulling the partial sums instead took a second
  // barrier -- nobody may leave while its memory is still being read -- and a round trip per remote value.)
  GV_STAMP(2);
  const int share = rows_per_cluster / csize;  // rows this CTA finishes (rows_per_cluster is a multiple of 64)
  if (csize > 1) {
    const uint32_t part_addr = (uint32_t)__cvta_generic_to_shared(part);
#pragma unroll
    for (int ti = 0; ti < kMaxTiles; ++ti) {
      if (ti >= tiles_per_warp) break;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int r = (ti * kWarps + warp) * 16 + g + 8 * hh;  // row of the cluster
        const uint32_t owner = (uint32_t)(r / share);
        uint32_t base;  // owner's slot [rank][r % share][0]
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                     : "=r"(base)
                     : "r"(part_addr + (uint32_t)((((size_t)rank * share + (size_t)(r % share)) * kCols) * sizeof(float))), "r"(owner));
#pragma unroll
        for (int mh = 0; mh < MT; ++mh)
          asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(base + (uint32_t)((mh * 8 + 2 * t) * sizeof(float))),
                       "f"(total[ti][mh][2 * hh]), "f"(total[ti][mh][2 * hh + 1])
                       : "memory");
      }
    }
    cluster_sync_all();  // release / acquire at cluster scope: every slot of every CTA is complete and visible
  } else {
#pragma unroll
    for (int ti = 0; ti < kMaxTiles; ++ti) {
      if (ti >= tiles_per_warp) break;
#pragma unroll
      for (int mh = 0; mh < MT; ++mh) {
        float* base = part + (size_t)((ti * kWarps + warp) * 16) * kCols + mh * 8;
        base[(g)*kCols + 2 * t] = total[ti][mh][0];
        base[(g)*kCols + 2 * t + 1] = total[ti][mh][1];
        base[(g + 8) * kCols + 2 * t] = total[ti][mh][2];
        base[(g + 8) * kCols + 2 * t + 1] = total[ti][mh][3];
      }
    }
    __syncthreads();
  }
  for (int o = threadIdx.x; o < share * kCols; o += kThreadsGv) {
    const int m = o / share, rl = o % share;  // consecutive threads -> consecutive n
    const int n = row0 + (int)rank * share + rl;
    float sum = 0.0f;
    for (int q = 0; q < csize; ++q) sum += part[((size_t)q * share + rl) * kCols + m];  // csize == 1: slot 0 is the whole block
    if (m < a.M && n < a.N) {
      if (a.out_f32) reinterpret_cast<float*>(a.C)[(size_t)m * a.N + n] = sum;
      else reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)m * a.N + n] = __float2bfloat16_rn(sum);
    }
  }
  GV_STAMP(3);
}

// ---------------------------------------------------------------------------------------------------
// Large shapes: the same arithmetic, but the weights reach the tensor cores through shared memory.
// One CTA per SM, 8 warps.  Every warp owns a ring of kSlots slots in shared memory and feeds it
// itself: an item is 16 output channels x 512 k (16 bulk async copies of 256 B, one per row, issued
// by lanes 0..15 and counted by the slot's mbarrier), so two or three items per warp -- 64..96 KB per
// SM -- are in flight without holding a register, and the ring keeps running across tile and
// row-block boundaries.  The group scales / zero points of the NEXT item are fetched into registers
// while the current one is being multiplied.  A warp walks its tiles (one per row block of 128
// channels) over the CTA's share of K; with no K split it stores its tile straight from the
// accumulator registers, otherwise the cluster adds the shares up over DSMEM as in the small kernel.
static __device__ int g_gv_flag;  // sticky: a bounded wait of the ring kernel ran out
#ifndef CFB_GV_WARPS
#define CFB_GV_WARPS 12
#endif
#ifndef CFB_GV_SLOTS
#define CFB_GV_SLOTS 3
#endif
constexpr int kWarpsM8 = CFB_GV_WARPS;  // warps per CTA for M <= 8 (M = 9..16: 8 warps, the activations take twice the room)
#ifndef CFB_GV_M16_WARPS
#define CFB_GV_M16_WARPS 8
#endif
#ifndef CFB_GV_M16_SLOTS
#define CFB_GV_M16_SLOTS 2
#endif
constexpr int kWarpsM16 = CFB_GV_M16_WARPS, kSlotsM16 = CFB_GV_M16_SLOTS;  // M = 9..16
constexpr int kItemChunks = 4;               // 128-k groups per item
constexpr int kBoxBytes = 16 * 128;          // one TMA box: 16 rows x 128 bytes, 128-byte swizzle
constexpr int kSlotBytes = 2 * kBoxBytes;    // an item = two boxes side by side along K
constexpr int kSlotsM8 = CFB_GV_SLOTS;   // ring depth per warp for M <= 8; M = 9..16 stages twice the activations and takes 2

__device__ __forceinline__ bool mbar_wait_bounded_gv(uint32_t mbar, uint32_t parity) {
  for (unsigned it = 0; it < (1u << 22); ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

struct ItemMeta {  // group scales (4 x f16) and zero points (4 nibbles) of rows g and g+8 for one item
  uint2 s[2];
  uint32_t z[2];
};

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

template <int MT, int kSlots, int kW5>
__global__ void __launch_bounds__(kW5 * 32, 1)
gemv_w4_ring_kernel(const __grid_constant__ CUtensorMap tm_codes, const GvArgs a, int cpc /* chunks per CTA, multiple of 4 */,
                    int pitch, int csize, int n_rb, int n_clusters, int32_t* error_flag) {
  constexpr int kT5 = kW5 * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t rank = cluster_rank();
  const int cluster_id = blockIdx.x / csize;
  const int gpr = a.K / kChunk;
  const int c0 = (int)rank * cpc;
  constexpr int kCols = 8 * MT;
  constexpr int kRowsRb = kW5 * 16;  // output channels per row block
  float* part = reinterpret_cast<float*>(smem + (size_t)8 * MT * pitch);          // [kRowsRb][kCols]
  // [kW5][kSlots][kSlotBytes], on a 1024-byte boundary (the swizzle pattern follows the address)
  uint8_t* rings = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(part + kRowsRb * kCols) + 1023) & ~(uintptr_t)1023);
  uint64_t* mbars = reinterpret_cast<uint64_t*>(rings + (size_t)kW5 * kSlots * kSlotBytes);
  // per chunk and activation row: two combinations of the sums of the activations that meet low / high nibbles
  // [cpc][8 * MT], read two entries at a time with 16-byte loads: on a 16-byte boundary whatever kW5 * kSlots is
  float2* sums = reinterpret_cast<float2*>((reinterpret_cast<uintptr_t>(mbars + kW5 * kSlots) + 15) & ~(uintptr_t)15);
  const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(rings + (size_t)warp * kSlots * kSlotBytes);
  const uint32_t mbar0 = (uint32_t)__cvta_generic_to_shared(mbars + warp * kSlots);
  if (lane == 0) {
    for (int s = 0; s < kSlots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar0 + 8 * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int ipt = cpc / kItemChunks;  // items per tile
  const int n_my = cluster_id < n_rb ? (n_rb - cluster_id + n_clusters - 1) / n_clusters : 0;  // row blocks of this cluster
  const int n_items = n_my * ipt;
  const int n_step = n_clusters * kRowsRb;          // channels between this warp's consecutive tiles
  const int n_first = cluster_id * kRowsRb + warp * 16;

  // Three walkers over the same item sequence (tile by tile, item by item inside a tile), kept incrementally so that
  // no division is needed: the TMA issue runs kSlots - 1 items ahead, the scale / zero-point fetch 3 items ahead.
  struct Walker { int n0, ci; };
  auto advance = [&](Walker& w) {
    if (++w.ci == ipt) { w.ci = 0; w.n0 += n_step; }
  };
  Walker w_tma{n_first, 0}, w_meta{n_first, 0}, w_cur{n_first, 0};
  int issued = 0, fetched = 0;
  auto issue_next = [&]() {  // one lane asks the TMA unit for the item's two boxes; rows past N come back as zeros
    if (issued < n_items && lane == 0) {
      const int slot = issued % kSlots;
      const uint32_t bar = mbar0 + 8 * slot, dst = ring_addr + slot * kSlotBytes;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kSlotBytes) : "memory");
      const int x = (c0 + w_tma.ci * kItemChunks) * (kChunk / 2);  // byte offset along K: a multiple of 256
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(dst), "l"(&tm_codes), "r"(x), "r"(w_tma.n0), "r"(bar) : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(dst + kBoxBytes), "l"(&tm_codes), "r"(x + 128), "r"(w_tma.n0), "r"(bar) : "memory");
    }
    ++issued;
    advance(w_tma);
  };
  auto fetch_meta = [&](ItemMeta& m) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = w_meta.n0 + h * 8 + g;
      if (fetched < n_items && n < a.N) {
        const size_t gi = (size_t)n * gpr + c0 + w_meta.ci * kItemChunks;  // multiple of 4: 8-byte / 2-byte aligned loads
        m.s[h] = __ldg(reinterpret_cast<const uint2*>(a.scales + gi));
        m.z[h] = __ldg(reinterpret_cast<const unsigned short*>(a.zps + (gi >> 1)));
      } else {
        m.s[h] = make_uint2(0u, 0u);  // scale 0: whatever the slot holds contributes nothing
        m.z[h] = 0x8888u;
      }
    }
    ++fetched;
    advance(w_meta);
  };

  // the ring starts before the activations are staged
#pragma unroll
  for (int d = 0; d < kSlots - 1; ++d) issue_next();
  ItemMeta meta, meta1, meta2;  // scales / zero points of items it, it + 1, it + 2 (a rotating register ring)
  fetch_meta(meta);
  fetch_meta(meta1);
  fetch_meta(meta2);
  stage_acts<MT, true>(a, smem, c0, cpc, pitch);
  __syncthreads();
  for (int item = threadIdx.x; item < cpc * 8 * MT; item += kT5) {
    const int chunk = item / (8 * MT), row = item % (8 * MT);
    const uint4* p = reinterpret_cast<const uint4*>(smem + (size_t)row * pitch + chunk * 256);
    float s_lo = 0.0f, s_hi = 0.0f;  // words x, z of a group hold the k that meet nibbles 0, 4, 2, 6; words y, w the others
    for (int q = 0; q < 16; ++q) {
      const uint4 v = p[q];
      const float2 fx = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), fy = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      const float2 fz = __half22float2(*reinterpret_cast<const __half2*>(&v.z)), fw = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
      s_lo += (fx.x + fx.y) + (fz.x + fz.y);
      s_hi += (fy.x + fy.y) + (fw.x + fw.y);
    }
    // stored as (P, Q) with  -(1024 + zp) S_lo - (64 + zp) S_hi = P + zp * Q
    sums[item] = make_float2(-1024.0f * s_lo - 64.0f * s_hi, -(s_lo + s_hi));
  }
  __syncthreads();

  // per-lane shared-memory addresses (32-bit, shared state space) so that every access is a plain LDS
  const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t act_lane = smem_addr + (uint32_t)(g * pitch + t * 16);                      // + mh*8*pitch + chunk*256 + j*64
  const uint32_t sums_lane = (uint32_t)__cvta_generic_to_shared(sums) + (uint32_t)(2 * t) * 8;  // + (chunk*8*MT + mh*8) * 8
  // 16-byte unit u of row r sits at unit u ^ (r % 8) of the row (128-byte swizzle); rows g and g+8 share g
  const uint32_t w_even = (uint32_t)(g * 128 + ((t ^ g) << 4)), w_odd = (uint32_t)(g * 128 + (((4 + t) ^ g) << 4));

  // the two nibble masks and the f16 pattern of 1024 live in registers, so that (w & mask) | 1024 is ONE three-input
  // logic instruction (with immediates it takes two)
  uint32_t k_lo, k_hi, k_magic;
  asm("mov.u32 %0, 0x000F000F;" : "=r"(k_lo));
  asm("mov.u32 %0, 0x00F000F0;" : "=r"(k_hi));
  asm("mov.u32 %0, 0x64006400;" : "=r"(k_magic));

  float total[MT][4];
#pragma unroll
  for (int mh = 0; mh < MT; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) total[mh][i] = 0.0f;
  bool ok = true;
  int slot = 0;
  uint32_t parity = 0;

  for (int it = 0; it < n_items; ++it) {
    // refill the slot that the previous item used: its 16-byte loads have returned (their values were consumed
    // by the multiplies), and the whole warp is past them
    __syncwarp();
    issue_next();
    ItemMeta next;
    fetch_meta(next);
    // after a wait has run out the warp stops waiting but keeps walking, so that cluster barriers still pair up
    if (ok) ok = mbar_wait_bounded_gv(mbar0 + 8 * slot, parity);
    const uint32_t sl = ring_addr + slot * kSlotBytes;
    const uint32_t act_item = act_lane + (uint32_t)(w_cur.ci * kItemChunks) * 256u;
    const uint32_t sums_item = sums_lane + (uint32_t)(w_cur.ci * kItemChunks) * (8 * MT * 8);
#pragma unroll
    for (int jc = 0; jc < kItemChunks; ++jc) {
      const uint32_t woff = sl + (jc >> 1) * kBoxBytes + ((jc & 1) ? w_odd : w_even);
      const uint4 w0 = lds128(woff), w1 = lds128(woff + 8 * 128);
      const uint32_t sb0 = (jc < 2 ? meta.s[0].x : meta.s[0].y) >> ((jc & 1) * 16);
      const uint32_t sb1 = (jc < 2 ? meta.s[1].x : meta.s[1].y) >> ((jc & 1) * 16);
      const float s0 = __half2float(__ushort_as_half((unsigned short)(sb0 & 0xffffu)));
      const float s1 = __half2float(__ushort_as_half((unsigned short)(sb1 & 0xffffu)));
      const float z0 = (float)((meta.z[0] >> (4 * jc)) & 0xFu), z1 = (float)((meta.z[1] >> (4 * jc)) & 0xFu);
      // Nibbles go to the tensor cores without a subtraction and with one shift per word: masked onto the f16
      // pattern of 1024, a low nibble reads 1024 + q and a high nibble 1024 + 16 q.  Low-nibble pairs feed one
      // accumulator, high-nibble pairs the other:  lo = sum a q + 1024 S_lo,  hi = 16 sum a q + 1024 S_hi, so
      //   sum a (q - zp) = lo + hi / 16 - (1024 + zp) S_lo - (64 + zp) S_hi      (S = activation sums, staged above).
      float accg[MT][2][4];
#pragma unroll
      for (int mh = 0; mh < MT; ++mh)
#pragma unroll
        for (int i = 0; i < 4; ++i) accg[mh][0][i] = accg[mh][1][i] = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t wa = (&w0.x)[j], wb = (&w1.x)[j], wa8 = wa >> 8, wb8 = wb >> 8;
        const uint32_t ra0 = and_or(wa, k_lo, k_magic), ra1 = and_or(wa, k_hi, k_magic);
        const uint32_t ra2 = and_or(wa8, k_lo, k_magic), ra3 = and_or(wa8, k_hi, k_magic);
        const uint32_t rb0 = and_or(wb, k_lo, k_magic), rb1 = and_or(wb, k_hi, k_magic);
        const uint32_t rb2 = and_or(wb8, k_lo, k_magic), rb3 = and_or(wb8, k_hi, k_magic);
#pragma unroll
        for (int mh = 0; mh < MT; ++mh) {
          const uint4 x = lds128(act_item + (uint32_t)(mh * 8) * (uint32_t)pitch + (uint32_t)(jc * 256 + j * 64));
          mma_f16_16816(accg[mh][0], ra0, rb0, ra2, rb2, x.x, x.z);  // nibbles (0,4) and (2,6): low nibbles
          mma_f16_16816(accg[mh][1], ra1, rb1, ra3, rb3, x.y, x.w);  // nibbles (1,5) and (3,7): high nibbles
        }
      }
#pragma unroll
      for (int mh = 0; mh < MT; ++mh) {
        // columns 2t, 2t+1 of this lane: (S_lo, S_hi) of activation rows mh*8 + 2t and + 1
        const float4 sv = lds128f(sums_item + (uint32_t)((jc * 8 * MT + mh * 8) * 8));  // (P, Q) of columns 2t and 2t+1
        const float c00 = __fmaf_rn(z0, sv.y, sv.x), c01 = __fmaf_rn(z0, sv.w, sv.z);
        const float c10 = __fmaf_rn(z1, sv.y, sv.x), c11 = __fmaf_rn(z1, sv.w, sv.z);
        total[mh][0] = __fmaf_rn(s0, __fmaf_rn(accg[mh][1][0], 0.0625f, accg[mh][0][0]) + c00, total[mh][0]);
        total[mh][1] = __fmaf_rn(s0, __fmaf_rn(accg[mh][1][1], 0.0625f, accg[mh][0][1]) + c01, total[mh][1]);
        total[mh][2] = __fmaf_rn(s1, __fmaf_rn(accg[mh][1][2], 0.0625f, accg[mh][0][2]) + c10, total[mh][2]);
        total[mh][3] = __fmaf_rn(s1, __fmaf_rn(accg[mh][1][3], 0.0625f, accg[mh][0][3]) + c11, total[mh][3]);
      }
    }
    meta = meta1;
    meta1 = meta2;
    meta2 = next;
    if (++slot == kSlots) { slot = 0; parity ^= 1u; }
    if (w_cur.ci == ipt - 1) {  // the tile's K share is complete
      const int n0 = w_cur.n0;
      if (csize == 1) {
#pragma unroll
        for (int mh = 0; mh < MT; ++mh)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n = n0 + g + (q >> 1) * 8, m = mh * 8 + 2 * t + (q & 1);
            if (n < a.N && m < a.M) {
              if (a.out_f32) reinterpret_cast<float*>(a.C)[(size_t)m * a.N + n] = total[mh][q];
              else reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)m * a.N + n] = __float2bfloat16_rn(total[mh][q]);
            }
          }
      } else {
#pragma unroll
        for (int mh = 0; mh < MT; ++mh) {
          float* base = part + (size_t)(warp * 16) * kCols + mh * 8;
          base[g * kCols + 2 * t] = total[mh][0];
          base[g * kCols + 2 * t + 1] = total[mh][1];
          base[(g + 8) * kCols + 2 * t] = total[mh][2];
          base[(g + 8) * kCols + 2 * t + 1] = total[mh][3];
        }
        cluster_sync_all();  // every warp of every CTA of the cluster finishes a row block at the same item
        const int share = kRowsRb / csize;
        const int row0 = n0 - warp * 16;
        for (int o = threadIdx.x; o < share * kCols; o += kT5) {
          const int m = o / share, r = (int)rank * share + o % share;
          const int n = row0 + r;
          float sum = 0.0f;
          for (uint32_t q = 0; q < (uint32_t)csize; ++q) sum += ld_dsmem_f32(part + (size_t)r * kCols + m, q);
          if (m < a.M && n < a.N) {
            if (a.out_f32) reinterpret_cast<float*>(a.C)[(size_t)m * a.N + n] = sum;
            else reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)m * a.N + n] = __float2bfloat16_rn(sum);
          }
        }
        cluster_sync_all();  // the partial sums may be overwritten from here on
      }
#pragma unroll
      for (int mh = 0; mh < MT; ++mh)
#pragma unroll
        for (int q = 0; q < 4; ++q) total[mh][q] = 0.0f;
    }
    advance(w_cur);
  }
  if (!ok && lane == 0) {
    g_gv_flag = 1;
    if (error_flag) *error_flag = 1;
  }
}

template <int MT>
int32_t launch_gv(const GvArgs& a, cudaStream_t st) {
  const int gpr = a.K / kChunk;
  const int ntiles = (a.N + 15) / 16;
  const int sms = sm_count();
  // Split K over `csize` CTAs of a cluster only as far as it takes to put about 3 CTAs on every SM:
  // every halving of a warp's stream shortens the part of its life in which weights are in flight.
  // The activations of a CTA's K share must fit in shared memory beside the partial sums.
  static thread_local int attr_dev = -1;
  static thread_local size_t occ_smem[8];
  static thread_local int occ_per_sm[8], occ_n = 0;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    CFB_CUDA(cudaFuncSetAttribute(gemv_w4_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_dev = dev;
    occ_n = 0;
  }
  int csize = 1, tpw = kMaxTiles;
  auto ctas = [&](int cs, int t) { return (long long)((ntiles + kWarps * t - 1) / (kWarps * t)) * cs; };
  auto smem_of = [&](int cs, int t) {
    const int cpc = (gpr + cs - 1) / cs;
    return (size_t)8 * MT * (cpc * kChunk * 2 + 64) + (size_t)kWarps * t * 16 * 8 * MT * sizeof(float);
  };
  while (smem_of(csize, tpw) > 96 * 1024 && csize < kMaxCluster) csize *= 2;
  int prev_csize = csize, prev_tpw = tpw;
  while (ctas(csize, tpw) < 3LL * sms) {
    prev_csize = csize;
    prev_tpw = tpw;
    if (tpw > 2) tpw /= 2;                       // fewer tiles per warp first (keeps K streams long) ...
    else if (csize < kMaxCluster && gpr / (csize * 2) >= 4) csize *= 2;  // ... then split K, down to 4 chunks per CTA
    else if (tpw > 1) tpw /= 2;
    else break;
  }
  // The grid must be resident at once: a second wave of a kernel this short doubles its time.  If the last step went
  // past what the registers and shared memory of the device hold, take it back.
  {
    const size_t sm_bytes = smem_of(csize, tpw);
    int per_sm = 0;
    for (int i = 0; i < occ_n; ++i)
      if (occ_smem[i] == sm_bytes) per_sm = occ_per_sm[i];
    if (per_sm == 0 && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_w4_kernel<MT>, kThreadsGv, sm_bytes) == cudaSuccess &&
        per_sm > 0 && occ_n < 8) {  // remembered per shared-memory size: the query is not free and this runs per call
      occ_smem[occ_n] = sm_bytes;
      occ_per_sm[occ_n++] = per_sm;
    }
    if (per_sm > 0 && ctas(csize, tpw) > (long long)per_sm * sms && ctas(prev_csize, prev_tpw) >= sms &&
        smem_of(prev_csize, prev_tpw) <= 96 * 1024) {
      csize = prev_csize;
      tpw = prev_tpw;
    }
  }
  const int cpc = (gpr + csize - 1) / csize;
  const int pitch = cpc * kChunk * 2 + 64;
  const int rows_per_cluster = kWarps * tpw * 16;
  const size_t smem = smem_of(csize, tpw);
  if (smem > 200 * 1024) return set_error(CFB200_ERR_UNSUPPORTED, "K = %d is too large for the decode kernel", a.K);
  const int clusters = (a.N + rows_per_cluster - 1) / rows_per_cluster;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * csize));
  cfg.blockDim = dim3(kThreadsGv);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CFB_CUDA(cudaLaunchKernelEx(&cfg, gemv_w4_kernel<MT>, a, tpw, cpc, pitch, csize));
  return CFB200_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Ring kernel launch; returns CFB200_ERR_UNSUPPORTED when the shape does not fit it.
template <int MT, int kW5>
int32_t launch_gv_ring(const GvArgs& a, cudaStream_t st) {
  constexpr int kSlots = MT == 1 ? kSlotsM8 : kSlotsM16;
  constexpr int kT5 = kW5 * 32;
  const int gpr = a.K / kChunk;
  if (gpr % kItemChunks != 0) return CFB200_ERR_UNSUPPORTED;
  const int sms = sm_count();
  const int n_rb = (a.N + kW5 * 16 - 1) / (kW5 * 16);
  auto smem_of = [&](int cs) {
    const int cpc = gpr / cs;
    return (size_t)8 * MT * (cpc * kChunk * 2 + 64) + (size_t)kW5 * 16 * 8 * MT * sizeof(float) + 1024 /* alignment */ +
           (size_t)kW5 * kSlots * kSlotBytes + (size_t)kW5 * kSlots * 8 + 16 /* alignment */ + (size_t)cpc * 8 * MT * sizeof(float2);
  };
  int csize = 0;
  for (int cs = 1; cs <= kMaxCluster; cs *= 2) {
    if (gpr % (cs * kItemChunks) != 0 || smem_of(cs) > 226 * 1024) continue;
    const long long min_rounds = tunable(kTuneGemvRingRounds) > 0 ? tunable(kTuneGemvRingRounds) : 1;
    if ((long long)n_rb * cs >= min_rounds * sms) {  // the first split that gives every cluster enough row blocks
      csize = cs;
      break;
    }
  }
  if (csize == 0) return CFB200_ERR_UNSUPPORTED;  // too few row blocks even with the deepest K split: the register-ring kernel
  const int cpc = gpr / csize;
  const int pitch = cpc * kChunk * 2 + 64;
  int n_clusters = sms / csize;
  if (n_clusters > n_rb) n_clusters = n_rb;
  static thread_local int attr_dev = -1;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    CFB_CUDA(cudaFuncSetAttribute(gemv_w4_ring_kernel<MT, kSlots, kW5>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr_dev = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_clusters * csize));
  cfg.blockDim = dim3(kT5);
  cfg.dynamicSmemBytes = smem_of(csize);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUtensorMap tm;
  {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return CFB200_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)(a.K / 2), (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)(a.K / 2)};
    const cuuint32_t box[2] = {128, 16};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.codes), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(CFB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
  }
  int32_t* no_flag = nullptr;
  CFB_CUDA(cudaLaunchKernelEx(&cfg, gemv_w4_ring_kernel<MT, kSlots, kW5>, tm, a, cpc, pitch, csize, n_rb, n_clusters, no_flag));
  return CFB200_OK;
}

int32_t read_gv_flag(int* out) {
  CFB_CUDA(cudaMemcpyFromSymbol(out, g_gv_flag, sizeof(int)));
  return CFB200_OK;
}

}  // namespace
}  // namespace cfb

using namespace cfb;

#ifdef CFB_GV_TRACE
extern "C" int32_t cfb200_debug_gv_trace(unsigned long long* out, int reset) {
  if (out && cudaMemcpyFromSymbol(out, g_gvstamp, sizeof(g_gvstamp)) != cudaSuccess) return 1;
  if (reset) {
    static unsigned long long z[1024 * 4];
    if (cudaMemcpyToSymbol(g_gvstamp, z, sizeof(z)) != cudaSuccess) return 1;
  }
  return 0;
}
#endif

extern "C" int32_t cfb200_gemv_w4a16(const void* A, const uint8_t* w_codes, const uint16_t* w_scales, const uint8_t* w_zps,
                                     size_t M, size_t N, size_t K, size_t group, void* C, int32_t out_f32, void* stream) {
  CFB_CHECK_ARG(A && w_codes && w_scales && w_zps && C, "NULL buffer");
  CFB_CHECK_ARG(M >= 1 && M <= 16, "decode kernel takes 1..16 rows of activations (got %zu); use cfb200_gemm_w4a16", M);
  CFB_CHECK_ARG(group == 128, "decode kernel needs group 128 (got %zu)", group);
  CFB_CHECK_ARG(N > 0 && K > 0 && K % 128 == 0, "K must be a positive multiple of 128 (got %zu)", K);
  CFB_CHECK_ARG(N < (1u << 30) && K < (1u << 30), "dimension too large");
  CFB_CHECK_ALIGNED(A, 16);
  CFB_CHECK_ALIGNED(w_codes, 16);
  GvArgs a;
  a.act = reinterpret_cast<const __nv_bfloat16*>(A);
  a.codes = w_codes; a.scales = w_scales; a.zps = w_zps;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.C = C; a.out_f32 = out_f32;
  cudaStream_t st = (cudaStream_t)stream;
  // weights of 16 MB and more go through the shared-memory ring; small ones (launch-latency territory) and shapes the
  // ring does not take through the register-ring kernel
  const long long ring_knob = tunable(kTuneGemvRing);  // 0 = never, 1 = from 16 MB of packed weights, n > 1 = from n MB
  if (ring_knob != 0 && N * K / 2 >= ((size_t)(ring_knob == 1 ? 16 : ring_knob) << 20)) {
    int32_t rc;
    if (M <= 8) {
      // 10, 11 or 12 warps per CTA: whichever leaves the fewest idle warps in the last round of 16-channel tiles
      const long long tiles = ((long long)N + 15) / 16, sms = sm_count();
      int best_w = kWarpsM8;
      double best_eff = 0.0;
      for (int w = kWarpsM8; w >= kWarpsM8 - 2; --w) {
        const long long per_round = (long long)w * sms, rounds = (tiles + per_round - 1) / per_round;
        const double eff = (double)tiles / (double)(rounds * per_round);
        if (eff > best_eff + 0.02) { best_eff = eff; best_w = w; }
      }
      rc = best_w == kWarpsM8 ? launch_gv_ring<1, kWarpsM8>(a, st)
           : best_w == kWarpsM8 - 1 ? launch_gv_ring<1, kWarpsM8 - 1>(a, st) : launch_gv_ring<1, kWarpsM8 - 2>(a, st);
    } else {
      rc = launch_gv_ring<2, kWarpsM16>(a, st);
    }
    if (rc != CFB200_ERR_UNSUPPORTED) return rc;
  }
  return M <= 8 ? launch_gv<1>(a, st) : launch_gv<2>(a, st);
}

// 0 = no kernel of this file has reported a bounded wait that ran out (sticky, per device); synchronises.
extern "C" int32_t cfb200_gemv_w4a16_status(int32_t* flag_host) {
  CFB_CHECK_ARG(flag_host != nullptr, "NULL argument");
  int v = 0;
  const int32_t rc = read_gv_flag(&v);
  *flag_host = v;
  return rc;
}
