// A1: per-tensor symmetric INT8/INT4 quantization (quantize_symmetric_f32, formats.rs:664-698) of
// one tensor or of a whole list of tensors resident in HBM.
//
// A per-tensor scale needs the absmax of the whole tensor before the first code exists, so every
// tensor is read twice: pass 1 folds |v| into one 32-bit word per tensor (integer atomicMax on the
// bit pattern of a non-negative float), pass 2 turns elements into codes.  The two passes of a
// list of tensors are software-pipelined through ONE kernel, the "stage":
//
//     stage k  =  pass 2 of tensor group k-1   followed by   pass 1 of tensor group k
//
// A stage needs no grid-wide barrier (its two halves touch different tensors) and a list of G
// groups takes G+1 launches instead of 2G, which halves the ramp-up/tail cost that dominates
// tensors of a few tens of MB.  Pass 2 walks its tensors BACK TO FRONT so that it meets the
// lines pass 1 (the previous launch) left in the 126 MB L2 before they are evicted, and writes
// codes with streaming stores.  Groups are consecutive tensors whose bytes fit an L2 budget.
//
// Pass 2, per element, common path (4 FP32 instructions, no conversion, no division):
//   s = fma(v, 1/scale, 1.5*2^23)   low mantissa byte of s = two's complement of rne(v/scale)
//   n = s - 1.5*2^23
//   r = fma(-n, scale, v)           proves n == roundf(v/scale) when |r| < 0.5*scale*(1-2^-10)
// (see DivRound in common.cuh).  If any element of a 16-byte vector fails the proof (a near tie,
// NaN, infinity, a quotient beyond the code range) the vector takes the exact path: IEEE division,
// roundf, clamp, NaN -> 0.
#include <atomic>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common.cuh"

namespace cfb {
namespace {

#ifndef CFB_A1_UNROLL
#define CFB_A1_UNROLL 4
#endif
#ifndef CFB_A1_MINB
#define CFB_A1_MINB 1
#endif
constexpr int kThreads = 256;
constexpr int kUnroll = CFB_A1_UNROLL;  // 16-byte loads in flight per thread
constexpr int kMaxSeg = 8;

struct Seg {
  const void* src;
  size_t n;
  int8_t* codes;        // pass 2 only
  unsigned* acc;        // absmax accumulator (bit pattern), = scale_absmax + 1
  float* scale_absmax;  // pass 2 writes [0] = scale, [1] = absmax
};

struct StageArgs {
  Seg apply[kMaxSeg];
  Seg amax[kMaxSeg];
  int n_apply, n_amax;
  float qmin, qmax;
  int check_range;  // pass 2 verifies |code| <= qmax per element (absmax supplied by the caller)
  int keep;         // pass 1 loads allocate normally in L2 (pass 2 is about to re-read them)
  int demote;       // pass 2 loads with an L2 evict_first policy
  int merge;        // advance the two passes in lockstep instead of one after the other
};

// One 16-byte vector -> VE codes.  TRUSTED: the absmax is this tensor's own, so |v/scale| < 127.5
// and the branch-free path of common.cuh applies; otherwise every element takes the reference
// formula literally (IEEE division, roundf, clamp, NaN -> 0).
template <int DT, bool TRUSTED, bool FINITE = false>
__device__ __forceinline__ void apply_vec(uint4 raw, size_t i, int8_t* __restrict__ codes, float scale,
                                          float inv, float qmin, float qmax) {
  constexpr int VE = Vec16<DT>::kElems;
  float f[VE];
  Vec16<DT>::unpack(raw, f);
  uint32_t packed[VE / 4];
  if constexpr (TRUSTED) {
    float a[VE];
#pragma unroll
    for (int k = 0; k < VE; ++k) a[k] = quant_mag_fixed<DT == CFB200_F32, FINITE>(f[k], scale, inv);
    if constexpr (DT == CFB200_F32) {
      packed[0] = negate_bytes(pack_mag4(a[0], a[1], a[2], a[3]), sign_mask_32(raw.x, raw.y, raw.z, raw.w));
    } else {
      packed[0] = negate_bytes(pack_mag4(a[0], a[1], a[2], a[3]), sign_mask_16(raw.x, raw.y));
      packed[1] = negate_bytes(pack_mag4(a[4], a[5], a[6], a[7]), sign_mask_16(raw.z, raw.w));
    }
  } else {
#pragma unroll
    for (int w = 0; w < VE / 4; ++w) {
      uint32_t acc = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        int q = clamp_to_int(roundf(__fdiv_rn(f[4 * w + b], scale)), qmin, qmax);
        acc |= ((uint32_t)q & 0xffu) << (8 * b);
      }
      packed[w] = acc;
    }
  }
  if constexpr (VE == 8) st_stream8(codes + i * VE, make_uint2(packed[0], packed[1]));
  else st_stream4(codes + i * VE, packed[0]);
}

// One 16-byte vector -> VE E4M3FN codes: x = v * (1 / scale), round to nearest even, saturating at +-448, NaN -> 0x7F
// (the arithmetic of cast_e4m3_tensor_kernel in quant_tensor.cu).
template <int DT>
__device__ __forceinline__ void apply_vec_e4m3(uint4 raw, size_t i, uint8_t* __restrict__ codes, float inv) {
  constexpr int VE = Vec16<DT>::kElems;
  float f[VE];
  Vec16<DT>::unpack(raw, f);
  auto pair = [&](float a, float b) -> uint32_t {  // a -> low byte
    unsigned short pk;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(__fmul_rn(b, inv)), "f"(__fmul_rn(a, inv)));
    return pk;
  };
  uint32_t packed[VE / 4];
#pragma unroll
  for (int w = 0; w < VE / 4; ++w) packed[w] = pair(f[4 * w], f[4 * w + 1]) | (pair(f[4 * w + 2], f[4 * w + 3]) << 16);
  if constexpr (VE == 8) st_stream8(codes + i * VE, make_uint2(packed[0], packed[1]));
  else st_stream4(codes + i * VE, packed[0]);
}

template <int DT, bool TRUSTED>
__device__ __forceinline__ void apply_part(const Seg& sg, float qmin, float qmax, bool demote) {
  constexpr int VE = Vec16<DT>::kElems;
  const float amax = __uint_as_float(*reinterpret_cast<const volatile unsigned*>(sg.acc));
  const float scale = (amax < 1e-12f) ? 1.0f : __fdiv_rn(amax, qmax);
  const float inv = __fdiv_rn(1.0f, scale);
  const size_t nvec = sg.n / VE;
  const uint4* p = reinterpret_cast<const uint4*>(sg.src);
  const size_t stride = (size_t)gridDim.x * kThreads;
  const uint64_t pol = l2_policy_evict_first();
  size_t j = (size_t)blockIdx.x * kThreads + threadIdx.x;
  // vector index i = nvec-1-j: back to front
  for (; j + (kUnroll - 1) * stride < nvec; j += kUnroll * stride) {
    uint4 r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint4* q = p + (nvec - 1 - (j + u * stride));
      r[u] = demote ? ld_stream16_policy(q, pol) : ld_stream16(q);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      apply_vec<DT, TRUSTED>(r[u], nvec - 1 - (j + u * stride), sg.codes, scale, inv, qmin, qmax);
  }
  for (; j < nvec; j += stride) {
    const size_t i = nvec - 1 - j;
    apply_vec<DT, TRUSTED>(demote ? ld_stream16_policy(p + i, pol) : ld_stream16(p + i), i, sg.codes, scale, inv, qmin, qmax);
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x < (unsigned)(sg.n - nvec * VE)) {
      const size_t i = nvec * VE + threadIdx.x;
      sg.codes[i] = (int8_t)clamp_to_int(roundf(__fdiv_rn(load_elem<DT>(sg.src, i), scale)), qmin, qmax);
    }
    if (threadIdx.x == 0) {
      sg.scale_absmax[0] = scale;
      sg.scale_absmax[1] = amax;  // same bits as the accumulator it aliases
    }
  }
}

template <int DT>
__device__ __forceinline__ void absmax_part(const Seg& sg, bool keep, float* s_part) {
  constexpr int VE = Vec16<DT>::kElems;
  using H2 = typename std::conditional<DT == CFB200_BF16, __nv_bfloat162, __half2>::type;
  const size_t nvec = sg.n / VE;
  const uint4* p = reinterpret_cast<const uint4*>(sg.src);
  const size_t stride = (size_t)gridDim.x * kThreads;
  float m = 0.0f;
  H2 hm;
  *reinterpret_cast<uint32_t*>(&hm) = 0u;
  auto fold = [&](uint4 r) {
    if constexpr (DT == CFB200_F32) {
      m = fmaxf(m, fabsf(__uint_as_float(r.x)));
      m = fmaxf(m, fabsf(__uint_as_float(r.y)));
      m = fmaxf(m, fabsf(__uint_as_float(r.z)));
      m = fmaxf(m, fabsf(__uint_as_float(r.w)));
    } else {
      // two lanes per instruction; __hmax2 drops a NaN operand like Rust's f32::max
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) hm = __hmax2(hm, __habs2(*reinterpret_cast<const H2*>(&w[i])));
    }
  };
  size_t j = (size_t)blockIdx.x * kThreads + threadIdx.x;
  for (; j + (kUnroll - 1) * stride < nvec; j += kUnroll * stride) {
    uint4 r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) r[u] = keep ? ld_cached16(p + j + u * stride) : ld_stream16(p + j + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) fold(r[u]);
  }
  for (; j < nvec; j += stride) fold(keep ? ld_cached16(p + j) : ld_stream16(p + j));
  if constexpr (DT != CFB200_F32) {
    const uint32_t bits = *reinterpret_cast<uint32_t*>(&hm);
    float lo, hi;
    if constexpr (DT == CFB200_BF16) {
      lo = __uint_as_float(bits << 16);
      hi = __uint_as_float(bits & 0xffff0000u);
    } else {
      const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&bits));
      lo = t2.x;
      hi = t2.y;
    }
    m = fmaxf(lo, hi);
  }
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(sg.n - nvec * VE))
    m = fmaxf(m, fabsf(load_elem<DT>(sg.src, nvec * VE + threadIdx.x)));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? s_part[threadIdx.x] : 0.0f;
    v = warp_max(v);
    if (threadIdx.x == 0 && v > 0.0f) atomicMax(sg.acc, __float_as_uint(v));
  }
  __syncthreads();
}

// Merged stage: pass 2 of the previous group (issue-bound once its reads hit in L2) and pass 1 of the
// next group (pure HBM streaming) advance in lockstep, kUnroll vectors of each per trip, so the
// memory pipe and the FP32 pipe are busy at the same time.  Trip counts are uniform over the
// grid (loads are predicated), which keeps the per-segment block reduction convergent.
template <int DT, bool TRUSTED, int U>
__device__ __forceinline__ void stage_body(const StageArgs& a, float* s_part) {
  constexpr int VE = Vec16<DT>::kElems;
  using H2 = typename std::conditional<DT == CFB200_BF16, __nv_bfloat162, __half2>::type;
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t j_first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const uint64_t pol = l2_policy_evict_first();
  const bool demote = a.demote != 0, keep = a.keep != 0;

  int ai = 0, mi = 0;        // current pass-2 / pass-1 segment
  size_t aj = j_first, mj = j_first;
  // pass-2 state of segment ai
  float scale = 1.0f, inv = 1.0f, amax_a = 0.0f;
  size_t nvec_a = 0, nvec_m = 0;
  const uint4* pa = nullptr;
  const uint4* pm = nullptr;
  bool a_open = false, m_open = false;
  float m = 0.0f;
  H2 hm;
  *reinterpret_cast<uint32_t*>(&hm) = 0u;

  while (ai < a.n_apply || mi < a.n_amax) {
    if (ai < a.n_apply && !a_open) {
      const Seg& sg = a.apply[ai];
      amax_a = __uint_as_float(*reinterpret_cast<const volatile unsigned*>(sg.acc));
      scale = (amax_a < 1e-12f) ? 1.0f : __fdiv_rn(amax_a, a.qmax);
      inv = __fdiv_rn(1.0f, scale);
      nvec_a = sg.n / VE;
      pa = reinterpret_cast<const uint4*>(sg.src);
      aj = j_first;
      a_open = true;
    }
    if (mi < a.n_amax && !m_open) {
      const Seg& sg = a.amax[mi];
      nvec_m = sg.n / VE;
      pm = reinterpret_cast<const uint4*>(sg.src);
      mj = j_first;
      m = 0.0f;
      *reinterpret_cast<uint32_t*>(&hm) = 0u;
      m_open = true;
    }
    // ---- issue the loads of both streams ----
    uint4 ra[U], rm[U];
    if (a_open) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t j = aj + u * stride;
        if (j < nvec_a) {
          const uint4* q = pa + (nvec_a - 1 - j);  // back to front
          ra[u] = demote ? ld_stream16_policy(q, pol) : ld_stream16(q);
        }
      }
    }
    if (m_open) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t j = mj + u * stride;
        rm[u] = j < nvec_m ? (keep ? ld_cached16(pm + j) : ld_stream16(pm + j)) : make_uint4(0, 0, 0, 0);
      }
    }
    // ---- consume ----
    if (a_open) {
      const Seg& sg = a.apply[ai];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t j = aj + u * stride;
        if (j < nvec_a) apply_vec<DT, TRUSTED>(ra[u], nvec_a - 1 - j, sg.codes, scale, inv, a.qmin, a.qmax);
      }
      aj += (size_t)U * stride;
      if (aj - threadIdx.x - (size_t)blockIdx.x * kThreads >= nvec_a || nvec_a == 0) {  // uniform over the grid
        if (blockIdx.x == 0) {
          if (threadIdx.x < (unsigned)(sg.n - nvec_a * VE)) {
            const size_t i = nvec_a * VE + threadIdx.x;
            sg.codes[i] = (int8_t)clamp_to_int(roundf(__fdiv_rn(load_elem<DT>(sg.src, i), scale)), a.qmin, a.qmax);
          }
          if (threadIdx.x == 0) {
            sg.scale_absmax[0] = scale;
            sg.scale_absmax[1] = amax_a;  // same bits as the accumulator it may alias
          }
        }
        a_open = false;
        ++ai;
      }
    }
    if (m_open) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if constexpr (DT == CFB200_F32) {
          m = fmaxf(m, fabsf(__uint_as_float(rm[u].x)));
          m = fmaxf(m, fabsf(__uint_as_float(rm[u].y)));
          m = fmaxf(m, fabsf(__uint_as_float(rm[u].z)));
          m = fmaxf(m, fabsf(__uint_as_float(rm[u].w)));
        } else {
          // two lanes per instruction; __hmax2 drops a NaN operand like Rust's f32::max
          const uint32_t w[4] = {rm[u].x, rm[u].y, rm[u].z, rm[u].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) hm = __hmax2(hm, __habs2(*reinterpret_cast<const H2*>(&w[i])));
        }
      }
      mj += (size_t)U * stride;
      if (mj - threadIdx.x - (size_t)blockIdx.x * kThreads >= nvec_m || nvec_m == 0) {
        const Seg& sg = a.amax[mi];
        if constexpr (DT != CFB200_F32) {
          const uint32_t bits = *reinterpret_cast<uint32_t*>(&hm);
          float lo, hi;
          if constexpr (DT == CFB200_BF16) {
            lo = __uint_as_float(bits << 16);
            hi = __uint_as_float(bits & 0xffff0000u);
          } else {
            const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&bits));
            lo = t2.x;
            hi = t2.y;
          }
          m = fmaxf(lo, hi);
        }
        if (blockIdx.x == 0 && threadIdx.x < (unsigned)(sg.n - nvec_m * VE))
          m = fmaxf(m, fabsf(load_elem<DT>(sg.src, nvec_m * VE + threadIdx.x)));
        m = warp_max(m);
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x < 32) {
          float v = threadIdx.x < kThreads / 32 ? s_part[threadIdx.x] : 0.0f;
          v = warp_max(v);
          if (threadIdx.x == 0 && v > 0.0f) atomicMax(sg.acc, __float_as_uint(v));
        }
        __syncthreads();
        m_open = false;
        ++mi;
      }
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(kThreads, CFB_A1_MINB) a1_stage_kernel(const __grid_constant__ StageArgs a) {
  __shared__ float s_part[kThreads / 32];
  if (a.check_range) {
    for (int s = 0; s < a.n_apply; ++s) apply_part<DT, false>(a.apply[s], a.qmin, a.qmax, a.demote != 0);
  } else {
    for (int s = 0; s < a.n_apply; ++s) apply_part<DT, true>(a.apply[s], a.qmin, a.qmax, a.demote != 0);
  }
  for (int s = 0; s < a.n_amax; ++s) absmax_part<DT>(a.amax[s], a.keep != 0, s_part);
}

template <int DT, int U>
__global__ void __launch_bounds__(kThreads) a1_stage_merged_kernel(const __grid_constant__ StageArgs a) {
  __shared__ float s_part[kThreads / 32];
  stage_body<DT, true, U>(a, s_part);
}

// ---------------------------------------------------------------------------------------------------
// Persistent variant: ONE cooperative launch (one CTA per SM) walks the whole list.  Per group of
// tensors: pass 1, a grid-wide barrier, pass 2.  Both passes move the weights through a ring of
// 32 KB shared-memory buffers filled by bulk async copies (one thread issues them, an mbarrier per
// buffer counts the bytes), so close to the whole shared memory of the SM is in flight and the
// loads cost no registers.  A CTA's items are the 32 KB chunks c, c + G, c + 2G, ... of the
// group's tensors laid end to end.  Pass 2 walks them in REVERSE: the last ring-full of pass 1 is
// still in shared memory and is quantized from there without touching memory again (34 MB over
// the 148 SMs), and the chunks before it are re-read newest first, while L2 still holds them.
#ifndef CFB_A1_CONSUMERS
#define CFB_A1_CONSUMERS 256
#endif
constexpr int kPConsumers = CFB_A1_CONSUMERS;  // threads that fold and quantize
constexpr int kPThreads = kPConsumers + 32;    // + one warp that only issues the bulk copies
constexpr int kPMaxTensors = 1024;
constexpr int kPSlots = 8;
#ifndef CFB_A1_ITEM_KB
#define CFB_A1_ITEM_KB 32
#endif
constexpr int kPItemBytes = CFB_A1_ITEM_KB * 1024;
constexpr int kPItemVecs = kPItemBytes / 16;
constexpr int kPBufs = 224 / CFB_A1_ITEM_KB;
constexpr int kPSmemBytes = kPBufs * kPItemBytes;

struct PSeg {
  const void* src;
  size_t n;
  int8_t* codes;
  float* scale_absmax;  // [0] scale, [1] absmax (doubles as the atomicMax accumulator)
  uint32_t flags;       // bit 0: last tensor of its group
  uint32_t pad;
};

static __device__ PSeg g_pseg[kPSlots][kPMaxTensors];
static __device__ unsigned g_pbar[kPSlots * 32];  // one barrier counter per slot, 128 bytes apart
static __device__ int g_pflag;                    // sticky: a bounded wait ran out
#ifdef CFB_A1_TRACE
// Phase time stamps (globaltimer ns) of three CTAs, for builds made with -DCFB_A1_TRACE only.
constexpr int kTracePhases = 200, kTraceSlots = 8;
static __device__ unsigned long long g_ptrace[3][kTracePhases][kTraceSlots];
__device__ __forceinline__ void trace_stamp(uint32_t bid, uint32_t G, int phase, int slot) {
  const int c = bid == 0 ? 0 : bid == G / 2 ? 1 : bid == G - 1 ? 2 : -1;
  if (c >= 0 && phase >= 0 && phase < kTracePhases) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_ptrace[c][phase][slot] = t;
  }
}
static __device__ unsigned long long g_ptrace_all[160][32][2];  // every CTA: barrier arrival and barrier completion
__device__ __forceinline__ void trace_all(uint32_t bid, int phase, int which) {
  if (bid < 160 && phase >= 0 && phase < 32) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_ptrace_all[bid][phase][which] = t;
  }
}
#define CFB_TRACE(slot) do { trace_stamp(bid, G, p + 1, slot); if ((slot) == 3) trace_all(bid, p + 1, 0); if ((slot) == 4) trace_all(bid, p + 1, 1); } while (0)
#else
#define CFB_TRACE(slot) do {} while (0)
#endif

// Absmax of a stream of 16-byte vectors, one instruction per 32-bit word for each of two
// accumulators (max.xorsign.abs takes |a|, |b| itself; the sign it leaves is dropped at the end):
//   hm: NaN operands are ignored, like Rust's f32::max in the reference fold;
//   hn: NaN operands win (.NaN), so it tells afterwards whether the tensor held a NaN.
template <int DT>
struct AbsFold {
  uint32_t hm, hn;  // bf16x2 / f16x2 / f32 bit patterns
  __device__ __forceinline__ AbsFold() { reset(); }
  __device__ __forceinline__ void reset() { hm = 0u; hn = 0u; }
  __device__ __forceinline__ void add1(uint32_t w) {
    if constexpr (DT == CFB200_BF16) {
      asm("max.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(hm) : "r"(w));
      asm("max.NaN.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(hn) : "r"(w));
    } else if constexpr (DT == CFB200_F16) {
      asm("max.xorsign.abs.f16x2 %0, %0, %1;" : "+r"(hm) : "r"(w));
      asm("max.NaN.xorsign.abs.f16x2 %0, %0, %1;" : "+r"(hn) : "r"(w));
    } else {
      asm("max.xorsign.abs.f32 %0, %0, %1;" : "+r"(hm) : "r"(w));
      asm("max.NaN.xorsign.abs.f32 %0, %0, %1;" : "+r"(hn) : "r"(w));
    }
  }
  __device__ __forceinline__ void add(const uint4& r) { add1(r.x); add1(r.y); add1(r.z); add1(r.w); }
  // a NaN or an infinity went by
  __device__ __forceinline__ bool nonfinite() const {
    if constexpr (DT == CFB200_F32) return (hn & 0x7fffffffu) >= 0x7f800000u;
    constexpr uint32_t kInf = DT == CFB200_BF16 ? 0x7f80u : 0x7c00u;
    return (hn & 0x7fffu) >= kInf || ((hn >> 16) & 0x7fffu) >= kInf;
  }
  __device__ __forceinline__ float finish() const {
    if constexpr (DT == CFB200_F32) return __uint_as_float(hm & 0x7fffffffu);
    const uint32_t bits = hm & 0x7fff7fffu;
    float lo, hi;
    if constexpr (DT == CFB200_BF16) {
      lo = __uint_as_float(bits << 16);
      hi = __uint_as_float(bits & 0xffff0000u);
    } else {
      const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&bits));
      lo = t2.x;
      hi = t2.y;
    }
    return fmaxf(lo, hi);
  }
};

// All CTAs of a cooperative launch meet here.  Bounded: about a second of polling, then false.
__device__ __forceinline__ bool grid_barrier_bounded(unsigned* ctr, unsigned target, unsigned sleep_ns) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");  // orders this CTA's earlier atomics before the count
    int ok = 0;
    for (unsigned it = 0; it < (1u << 24); ++it) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
      if (v >= target) { ok = 1; break; }
      if (sleep_ns) __nanosleep(sleep_ns);
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity, unsigned limit = 1u << 22) {
  for (unsigned it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

struct PGroup {  // one group's tensors, in shared memory (three copies rotate: current, next, the one being set up)
  const uint8_t* src[kMaxSeg];
  int8_t* codes[kMaxSeg];
  float* scale_absmax[kMaxSeg];
  size_t n[kMaxSeg];
  size_t nvec[kMaxSeg];
  uint32_t first_chunk[kMaxSeg + 1];  // chunks of the group before tensor s
  unsigned amax[kMaxSeg];
  float scale[kMaxSeg], inv[kMaxSeg];
  unsigned odd[kMaxSeg];              // non-zero: the tensor holds a NaN or an infinity
  int nseg, end;                      // tensors in the group (0 = no such group); index one past its last tensor
};
struct PItem {  // what a ring buffer holds
  uint32_t seg, chunk, vecs;
  uint32_t kind;  // bit 0: 1 = quantize (pass 2), 0 = absmax (pass 1); bit 1: keep the buffer (a pass-1 item that stays)
};

// Lanes of ONE warp fill grp with the group that starts at tensor `first` (at most kMaxSeg tensors).
template <int VE>
__device__ __forceinline__ void setup_group(PGroup& grp, const PSeg* __restrict__ segs, int count, int first, int lane) {
  int e = first;
  if (first < count) {
    while (e + 1 < count && !(segs[e].flags & 1u)) ++e;
    ++e;
  }
  const int nseg = e - first;
  if (lane < nseg) {
    const PSeg sg = segs[first + lane];
    grp.src[lane] = reinterpret_cast<const uint8_t*>(sg.src);
    grp.codes[lane] = sg.codes;
    grp.scale_absmax[lane] = sg.scale_absmax;
    grp.n[lane] = sg.n;
    grp.nvec[lane] = sg.n / VE;
    grp.amax[lane] = 0u;
    grp.odd[lane] = 0u;
  }
  __syncwarp();
  if (lane == 0) {
    uint32_t acc = 0;
    for (int s2 = 0; s2 < nseg; ++s2) {
      grp.first_chunk[s2] = acc;
      acc += (uint32_t)((grp.nvec[s2] * 16 + kPItemBytes - 1) / kPItemBytes);
    }
    grp.first_chunk[nseg] = acc;
    grp.nseg = nseg;
    grp.end = e;
  }
  __syncwarp();
}

// Items of this CTA in a group: chunks bid, bid + G, ... of the group's tensors laid end to end.
__device__ __forceinline__ uint32_t items_of(const PGroup& grp, uint32_t bid, uint32_t G) {
  if (grp.nseg == 0) return 0;
  const uint32_t total = grp.first_chunk[grp.nseg];
  return total > bid ? (total - bid - 1) / G + 1 : 0;
}

// The kernel runs in phases, one per grid barrier.  Phase p quantizes group p (pass 2) and, under it,
// folds the absmax of group p+1 (pass 1): pass 2 keeps the integer pipe busy and reads mostly from
// shared memory and L2, pass 1 is pure HBM streaming, so the two overlap.  Every item goes through
// the ring in ONE sequence (buffer = sequence number mod kPBufs) that the producer warp issues and
// the consumers follow:
//   * the items of group p that pass 1 left in the ring are quantized first, oldest first, which
//     frees the buffers in the order the producer reuses them;
//   * then pass-2 reloads of group p (oldest chunk first: the lines L2 gives up first) alternate with
//     the pass-1 items of group p+1 in proportion to their counts;
//   * the last kPBufs pass-1 items of group p+1 close the phase and stay in the ring.
// OUT: 0 = symmetric integer codes (A1), 1 = E4M3FN codes with scale = absmax / 448 (the per-tensor FP8 weight cast)
template <int DT, int OUT = 0>
__global__ void __launch_bounds__(kPThreads, 1)
a1_persist_kernel(const PSeg* __restrict__ segs, int count, unsigned* bar, float qmin, float qmax, uint32_t retain_items,
                  uint32_t bar_sleep_ns, uint32_t tail_first) {
  constexpr int VE = Vec16<DT>::kElems;
  constexpr int VPT = kPItemVecs / kPConsumers;  // vectors per consumer thread per item
  static_assert(kPItemVecs % kPConsumers == 0 && VPT % 4 == 0, "the unrolled quantize loop reads four vectors per thread per trip");
  extern __shared__ __align__(128) uint8_t p_ring[];
  __shared__ __align__(8) uint64_t s_full[kPBufs], s_empty[kPBufs];
  __shared__ PGroup s_grp[3];
  __shared__ PItem s_item[kPBufs];
  __shared__ int s_fail;
  __shared__ uint32_t s_issued;  // producer: items issued so far (read only on the failure path)
  const int tid = threadIdx.x, lane = tid & 31;
  const bool producer = tid >= kPConsumers;  // the last warp only moves data
  const uint32_t G = gridDim.x, bid = blockIdx.x;
  const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(p_ring);
  const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(&s_full[0]);
  const uint32_t empty0 = (uint32_t)__cvta_generic_to_shared(&s_empty[0]);
  if (tid == 0) {
    for (int b = 0; b < kPBufs; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * b) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * b), "r"(kPConsumers / 32) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_fail = 0;
    s_issued = 0;
    s_grp[2].nseg = 0;  // "group -1": nothing to quantize in the first phase
    s_grp[2].end = 0;
  }
  if (producer) {
    setup_group<VE>(s_grp[0], segs, count, 0, lane);
    setup_group<VE>(s_grp[1], segs, count, s_grp[0].end, lane);
  }
  __syncthreads();
  uint32_t full_par = 0;             // consumers: bit b = parity of buffer b's next fill
  uint32_t empty_par = 0, used = 0;  // producer lane 0: parity of buffer b's next release; buffers filled before
  uint32_t seq = 0;                  // items issued (producer) / consumed (consumers) so far; buffer = seq % kPBufs
  unsigned nbar = 0;
  const uint64_t pol_first = l2_policy_evict_first();

  // item k of this CTA in group grp: its tensor, chunk, address and length
  auto locate = [&](const PGroup& grp, uint32_t k, int& sidx, uint32_t& ch, uint32_t& bytes) -> const uint8_t* {
    const uint32_t g = bid + k * G;
    sidx = 0;
    while (sidx + 1 < grp.nseg && grp.first_chunk[sidx + 1] <= g) ++sidx;
    ch = g - grp.first_chunk[sidx];
    const size_t left = grp.nvec[sidx] * 16 - (size_t)ch * kPItemBytes;
    bytes = (uint32_t)(left < (size_t)kPItemBytes ? left : (size_t)kPItemBytes);
    return grp.src[sidx] + (size_t)ch * kPItemBytes;
  };
  // producer lane 0: item k of this CTA in group grp -> ring buffer seq % kPBufs
  auto issue = [&](const PGroup& grp, uint32_t k, uint32_t kind, bool evict_first) -> bool {
    const int b = (int)(seq % kPBufs);
    if (used & (1u << b)) {
      if (!mbar_wait_bounded(empty0 + 8 * b, (empty_par >> b) & 1u)) return false;
      empty_par ^= 1u << b;
    }
    ++seq;
    used |= 1u << b;
    int sidx;
    uint32_t ch, bytes;
    const uint8_t* src = locate(grp, k, sidx, ch, bytes);
    s_item[b] = PItem{(uint32_t)sidx, ch, bytes / 16, kind};
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * b), "r"(bytes) : "memory");
    if (evict_first)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                   ::"r"(ring_addr + b * kPItemBytes), "l"(src), "r"(bytes), "r"(full0 + 8 * b), "l"(pol_first) : "memory");
    else
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(ring_addr + b * kPItemBytes), "l"(src), "r"(bytes), "r"(full0 + 8 * b) : "memory");
    return true;
  };
  // consumers: one pass-2 item out of buffer b
  auto quantize_item = [&](const PGroup& grp, int b) {
    const PItem it = s_item[b];
    const uint4* buf = reinterpret_cast<const uint4*>(p_ring + (size_t)b * kPItemBytes);
    const float scale = grp.scale[it.seg], inv = grp.inv[it.seg];
    int8_t* codes = grp.codes[it.seg];
    const size_t v0 = (size_t)it.chunk * kPItemVecs;
    if constexpr (OUT == 1) {
      uint8_t* c8 = reinterpret_cast<uint8_t*>(codes);
      if (it.vecs == (uint32_t)kPItemVecs) {
#pragma unroll
        for (int h = 0; h < VPT; h += 4) {
          uint4 r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) r[u] = buf[tid + (h + u) * kPConsumers];
#pragma unroll
          for (int u = 0; u < 4; ++u) apply_vec_e4m3<DT>(r[u], v0 + tid + (h + u) * kPConsumers, c8, inv);
        }
      } else {
        for (uint32_t v = tid; v < it.vecs; v += kPConsumers) apply_vec_e4m3<DT>(buf[v], v0 + v, c8, inv);
      }
    } else if (it.vecs == (uint32_t)kPItemVecs && grp.odd[it.seg] == 0u) {
#pragma unroll
      for (int h = 0; h < VPT; h += 4) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = buf[tid + (h + u) * kPConsumers];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          apply_vec<DT, true, true>(r[u], v0 + tid + (h + u) * kPConsumers, codes, scale, inv, qmin, qmax);
      }
    } else {
      for (uint32_t v = tid; v < it.vecs; v += kPConsumers) apply_vec<DT, true>(buf[v], v0 + v, codes, scale, inv, qmin, qmax);
    }
  };
  auto release = [&](int b) {
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * b) : "memory");
  };

  // A bounded wait ran out: copies already issued still write into this CTA's shared memory, so wait (bounded again)
  // for each of them before the CTA returns, and report through the sticky device flag.
  auto fail_exit = [&]() {
    if (tid == 0) {
      g_pflag = 1;
      for (uint32_t j = seq; j < s_issued; ++j) {
        const int b = (int)(j % kPBufs);
        if (!mbar_wait_bounded(full0 + 8 * b, (full_par >> b) & 1u)) break;
        full_par ^= 1u << b;
      }
    }
    __syncthreads();
  };

  // phase p: quantize group p (s_grp[(p + 3) % 3], absent for p == -1) under the absmax pass of group p + 1
  for (int p = -1;; ++p) {
    PGroup& cur = s_grp[(p + 3) % 3];
    PGroup& nxt = s_grp[(p + 1) % 3];
    if (cur.nseg == 0 && nxt.nseg == 0) break;
    const uint32_t Tc = items_of(cur, bid, G), Tn = items_of(nxt, bid, G);
    const uint32_t Rc = Tc < (uint32_t)kPBufs ? Tc : (uint32_t)kPBufs;  // items of cur still in the ring
    const uint32_t A = Tc - Rc;                                        // pass-2 reloads
    const uint32_t Bfree = Tn > (uint32_t)kPBufs ? Tn - kPBufs : 0;    // pass-1 items that do not stay

    if (producer) {
      if (lane == 0) {
        bool ok = true;
        uint32_t a = 0, b2 = 0;
        CFB_TRACE(5);
        // Reload order: the last `retain_items` reloads are the lines pass 1 left in L2 at normal priority.  They go
        // first (oldest of them first), while L2 still holds them; the lines that were let go follow.
        const uint32_t Rk = tail_first ? (retain_items < A ? retain_items : A) : A;
        while (ok && (a < A || b2 < Bfree)) {  // proportional interleave
          if (a < A && (b2 >= Bfree || (uint64_t)a * Bfree <= (uint64_t)b2 * A)) {
            ok = issue(cur, a < Rk ? A - Rk + a : a - Rk, 1u, true);
            ++a;
          }
          else {  // early items would be gone from L2 before their second read anyway: let them go first
            const bool early = b2 + retain_items < Bfree;
            ok = issue(nxt, b2++, 0u, early);
          }
        }
        for (; ok && b2 < Tn; ++b2) ok = issue(nxt, b2, 2u, true);  // the items that stay
        s_issued = seq;
        CFB_TRACE(6);
        if (!ok) s_fail = 1;
      }
      __syncwarp();
      // the group after next, for the following phase (its slot held group p - 1, which is done)
      setup_group<VE>(s_grp[(p + 2) % 3], segs, count, nxt.nseg ? nxt.end : count, lane);
    } else {
      // tails of both groups: elements past the last whole vector (CTA 0)
      if (bid == 0) {
        for (int s2 = 0; s2 < nxt.nseg; ++s2) {
          const size_t nv = nxt.nvec[s2];
          if (tid < (int)(nxt.n[s2] - nv * VE)) {
            const float x = fabsf(load_elem<DT>(nxt.src[s2], nv * VE + tid));
            atomicMax(&nxt.amax[s2], __float_as_uint(fmaxf(0.0f, x)));  // fmaxf drops a NaN
            if (!(x <= 3.4028234e38f)) nxt.odd[s2] = 1u;
          }
        }
        for (int s2 = 0; s2 < cur.nseg; ++s2) {
          const size_t nv = cur.nvec[s2];
          const float scale = cur.scale[s2];
          if (tid < (int)(cur.n[s2] - nv * VE)) {
            const size_t k = nv * VE + tid;
            if constexpr (OUT == 1) {
              unsigned short pk;
              asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(__fmul_rn(load_elem<DT>(cur.src[s2], k), cur.inv[s2])));
              cur.codes[s2][k] = (int8_t)(pk & 0xffu);
            } else {
              cur.codes[s2][k] = (int8_t)clamp_to_int(roundf(__fdiv_rn(load_elem<DT>(cur.src[s2], k), scale)), qmin, qmax);
            }
          }
        }
      }
      bool ok = true;
      if (tid == 0) CFB_TRACE(0);
      // 1. what pass 1 left in the ring, oldest first
      for (uint32_t r = 0; r < Rc; ++r) {
        const int b = (int)((seq - Rc + r) % kPBufs);
        quantize_item(cur, b);
        release(b);
      }
      if (tid == 0) CFB_TRACE(1);
      // 2. the merged stream
      AbsFold<DT> f;
      int fseg = -1;
      auto flush = [&]() {
        if (fseg >= 0) {
          const bool odd = __any_sync(kFullMask, f.nonfinite());
          const float m = warp_max(f.finish());
          if (lane == 0 && m > 0.0f) atomicMax(&nxt.amax[fseg], __float_as_uint(m));
          if (lane == 0 && odd) nxt.odd[fseg] = 1u;
        }
        f.reset();
      };
      const uint32_t n_items = A + Tn;
      for (uint32_t j = 0; j < n_items; ++j) {
        const int b = (int)(seq % kPBufs);
        if (!mbar_wait_bounded(full0 + 8 * b, (full_par >> b) & 1u)) { ok = false; break; }
        ++seq;
        full_par ^= 1u << b;
        const uint32_t kind = s_item[b].kind;
        if (kind & 1u) {
          quantize_item(cur, b);
          release(b);
        } else {
          const PItem it = s_item[b];
          if ((int)it.seg != fseg) { flush(); fseg = (int)it.seg; }
          const uint4* buf = reinterpret_cast<const uint4*>(p_ring + (size_t)b * kPItemBytes);
          if (it.vecs == (uint32_t)kPItemVecs) {
#pragma unroll
            for (int u = 0; u < VPT; ++u) f.add(buf[tid + u * kPConsumers]);
          } else {
            for (uint32_t v = tid; v < it.vecs; v += kPConsumers) f.add(buf[v]);
          }
          if (!(kind & 2u)) release(b);
        }
      }
      if (tid == 0) CFB_TRACE(2);
      flush();
      if (!ok) s_fail = 1;
    }
    __syncthreads();
    if (s_fail) {
      fail_exit();
      return;
    }
    if (bid == 0 && tid < cur.nseg) cur.scale_absmax[tid][0] = cur.scale[tid];  // group p is done: publish its scale
    if (nxt.nseg == 0) continue;  // last phase: nothing was folded, no barrier needed
    if (tid < nxt.nseg) {
      if (nxt.amax[tid] != 0u) atomicMax(reinterpret_cast<unsigned*>(nxt.scale_absmax[tid] + 1), nxt.amax[tid]);
      // slot [0] is zero until CTA 0 writes the scale one phase later: it carries the flag meanwhile
      if (nxt.odd[tid] != 0u) atomicOr(reinterpret_cast<unsigned*>(nxt.scale_absmax[tid]), 1u);
    }
    ++nbar;
    if (tid == 0) CFB_TRACE(3);
    if (!grid_barrier_bounded(bar, nbar * G, bar_sleep_ns)) {
      fail_exit();
      return;
    }
    if (tid < nxt.nseg) {
      unsigned abits, obits;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(abits) : "l"(nxt.scale_absmax[tid] + 1) : "memory");
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(obits) : "l"(nxt.scale_absmax[tid]) : "memory");
      const float amax = __uint_as_float(abits);
      const float scale = (amax < 1e-12f) ? 1.0f : __fdiv_rn(amax, qmax);
      nxt.scale[tid] = scale;
      nxt.inv[tid] = __fdiv_rn(1.0f, scale);
      nxt.odd[tid] = obits;
    }
    if (tid == 0) CFB_TRACE(4);
    __syncthreads();
  }
}

// Self-test of the give-up path: a wait on a barrier that nothing ever completes, with a short limit, reported the way
// the persistent kernel reports it (the sticky device flag).  No memory is touched, nothing is left in flight.
__global__ void a1_wait_probe_kernel(unsigned limit) {
  __shared__ __align__(8) uint64_t s_bar;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&s_bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait_bounded(bar, 0u, limit)) g_pflag = 1;
  }
}

void bounds_of(int32_t bits, float* qmin, float* qmax) {  // formats.rs:654-660
  if (bits == 4) { *qmin = -8.0f; *qmax = 7.0f; }
  else { *qmin = -128.0f; *qmax = 127.0f; }
}

// resident CTAs (occupancy x SMs) of a kernel on the current device
template <typename K>
int resident_grid(K kernel, int* cache /* [64], zero-initialised */) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cache[dev] == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 2;
    cache[dev] = per_sm * sm_count();
  }
  return cache[dev];
}

template <int DT>
int32_t launch_stage_dt(const StageArgs& a, size_t chunks, cudaStream_t st) {
  static int c_seq[64], c_m2[64], c_m4[64];
  const bool merged = a.merge != 0 && !a.check_range;
  int cap;
  if (!merged) cap = resident_grid(a1_stage_kernel<DT>, c_seq);
  else if (a.merge == 1) cap = resident_grid(a1_stage_merged_kernel<DT, 2>, c_m2);
  else cap = resident_grid(a1_stage_merged_kernel<DT, 4>, c_m4);
  int grid = (int)(chunks < (size_t)cap ? chunks : (size_t)cap);
  if (grid < 1) grid = 1;
  if (!merged) a1_stage_kernel<DT><<<grid, kThreads, 0, st>>>(a);
  else if (a.merge == 1) a1_stage_merged_kernel<DT, 2><<<grid, kThreads, 0, st>>>(a);
  else a1_stage_merged_kernel<DT, 4><<<grid, kThreads, 0, st>>>(a);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

int32_t launch_stage(int32_t dt, const StageArgs& a, cudaStream_t st) {
  size_t chunks = 0;
  for (int s = 0; s < a.n_apply; ++s) chunks = max(chunks, a.apply[s].n / (dt == CFB200_F32 ? 4 : 8) / kThreads + 1);
  for (int s = 0; s < a.n_amax; ++s) chunks = max(chunks, a.amax[s].n / (dt == CFB200_F32 ? 4 : 8) / kThreads + 1);
  switch (dt) {
    case CFB200_F32: return launch_stage_dt<CFB200_F32>(a, chunks, st);
    case CFB200_F16: return launch_stage_dt<CFB200_F16>(a, chunks, st);
    default: return launch_stage_dt<CFB200_BF16>(a, chunks, st);
  }
}

// The persistent kernel wins for 16-bit sources; an f32 source needs an IEEE division per element, which the
// launch-per-group kernel hides better behind its 8 CTAs per SM.  Knob: 0 = never, 1 = 16-bit sources (default), 2 = always.
bool use_persist(int32_t src_dtype) {
  const long long k = tunable(kTuneA1Persist);
  return k >= 2 || (k == 1 && src_dtype != CFB200_F32);
}

size_t default_group_bytes() {
  const long long mb = tunable(kTuneA1GroupMB);
  return (size_t)(mb > 0 ? mb : 64) << 20;
}

// consecutive tensors are grouped while their bytes fit the budget (a larger tensor is alone)
int plan_groups(int32_t count, const size_t* ns, int32_t dt, size_t budget, int* group_end /* count entries */) {
  if (budget == 0) budget = default_group_bytes();
  const size_t eb = dtype_size(dt);
  int ng = 0, i = 0;
  while (i < count) {
    size_t bytes = 0;
    int k = 0;
    while (i < count && k < kMaxSeg && (k == 0 || bytes + ns[i] * eb <= budget)) {
      bytes += ns[i] * eb;
      ++i;
      ++k;
    }
    group_end[ng++] = i;
  }
  return ng;
}

template <int DT, int OUT>
int32_t launch_persist_dt(const PSeg* table, int count, unsigned* bar, float qmin, float qmax, cudaStream_t st) {
  static int ready[64];
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ready[dev]) {
    CFB_CUDA(cudaFuncSetAttribute(a1_persist_kernel<DT, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmemBytes));
    int per_sm = 0;
    CFB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a1_persist_kernel<DT, OUT>, kPThreads, kPSmemBytes));
    if (per_sm < 1) return set_error(CFB200_ERR_UNSUPPORTED, "the persistent A1 kernel does not fit this device");
    ready[dev] = 1;
  }
  const long long retain_mb = tunable(kTuneA1RetainMB);
  uint32_t retain_items = retain_mb >= 0 ? (uint32_t)(((size_t)retain_mb << 20) / ((size_t)kPItemBytes * sm_count())) : 0xffffffffu / 2;
  const long long bs = tunable(kTuneA1BarSleep);
  uint32_t bar_sleep_ns = (uint32_t)(bs < 0 ? 0 : bs > 1000 ? 1000 : bs);
  uint32_t tail_first = tunable(kTuneA1TailFirst) != 0;
  void* args[] = {(void*)&table, (void*)&count, (void*)&bar, (void*)&qmin, (void*)&qmax, (void*)&retain_items,
                  (void*)&bar_sleep_ns, (void*)&tail_first};
  CFB_CUDA(cudaLaunchCooperativeKernel((const void*)a1_persist_kernel<DT, OUT>, dim3((unsigned)sm_count()), dim3(kPThreads), args,
                                       (size_t)kPSmemBytes, st));
  return CFB200_OK;
}

// The whole list through the persistent kernel, kPMaxTensors tensors per launch.
int32_t run_persist(int32_t count, const void* const* srcs, int32_t dt, const size_t* ns, float qmin, float qmax,
                    int8_t* const* codes, float* scale_absmax, const int* group_end, int ng, size_t budget, void* const* stage_events,
                    cudaStream_t st, int out_kind = 0) {
  // Descriptor tables and barrier words are handed out round-robin, per device.  A slot is reused only after the launch
  // that last read it has finished (an event per slot, waited for on the host), so any number of calls may be in
  // flight on any streams and host threads.
  static std::mutex slot_mutex;
  static unsigned next_slot[64];
  static cudaEvent_t slot_done[64][kPSlots];
  int launch = 0;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CFB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  PSeg* dev_table = nullptr;
  unsigned* dev_bar = nullptr;
  CFB_CUDA(cudaGetSymbolAddress((void**)&dev_table, g_pseg));
  CFB_CUDA(cudaGetSymbolAddress((void**)&dev_bar, g_pbar));
  const size_t eb = dtype_size(dt);
  std::vector<PSeg> host;
  int g = 0;
  while (g < ng) {
    // as many whole groups as fit one table
    host.clear();
    const int first = g > 0 ? group_end[g - 1] : 0;
    int g_hi = g;
    while (g_hi < ng && group_end[g_hi] - first <= kPMaxTensors) ++g_hi;
    if (g_hi == g) return set_error(CFB200_ERR_INVALID, "tensor group larger than the descriptor table");
    for (int gg = g; gg < g_hi; ++gg) {
      const int lo = gg > 0 ? group_end[gg - 1] : 0, hi = group_end[gg];
      for (int i = lo; i < hi; ++i) {
        PSeg sg{srcs[i], ns[i], codes[i], scale_absmax + 2 * i, 0u, 0u};
        if (i == hi - 1) sg.flags |= 1u;
        host.push_back(sg);
      }
    }
    std::lock_guard<std::mutex> lock(slot_mutex);
    const unsigned slot = next_slot[dev]++ % kPSlots;
    if (!slot_done[dev][slot]) CFB_CUDA(cudaEventCreateWithFlags(&slot_done[dev][slot], cudaEventDisableTiming));
    else CFB_CUDA(cudaEventSynchronize(slot_done[dev][slot]));
    PSeg* table = dev_table + (size_t)slot * kPMaxTensors;
    unsigned* bar = dev_bar + (size_t)slot * 32;
    CFB_CUDA(cudaMemcpyAsync(table, host.data(), host.size() * sizeof(PSeg), cudaMemcpyHostToDevice, st));
    CFB_CUDA(cudaMemsetAsync(bar, 0, sizeof(unsigned), st));
    if (stage_events && stage_events[launch]) CFB_CUDA(cudaEventRecord((cudaEvent_t)stage_events[launch], st));
    ++launch;
    int32_t rc;
    const int n = (int)host.size();
    switch (dt) {
      case CFB200_F32: rc = out_kind ? launch_persist_dt<CFB200_F32, 1>(table, n, bar, qmin, qmax, st) : launch_persist_dt<CFB200_F32, 0>(table, n, bar, qmin, qmax, st); break;
      case CFB200_F16: rc = out_kind ? launch_persist_dt<CFB200_F16, 1>(table, n, bar, qmin, qmax, st) : launch_persist_dt<CFB200_F16, 0>(table, n, bar, qmin, qmax, st); break;
      default: rc = out_kind ? launch_persist_dt<CFB200_BF16, 1>(table, n, bar, qmin, qmax, st) : launch_persist_dt<CFB200_BF16, 0>(table, n, bar, qmin, qmax, st); break;
    }
    if (rc) return rc;
    CFB_CUDA(cudaEventRecord(slot_done[dev][slot], st));
    g = g_hi;
  }
  if (stage_events && stage_events[launch]) CFB_CUDA(cudaEventRecord((cudaEvent_t)stage_events[launch], st));
  return CFB200_OK;
}

}  // namespace
}  // namespace cfb

using namespace cfb;

// 0 = no bounded wait of the persistent kernel has run out on the current device (sticky); synchronises the device.
extern "C" int32_t cfb200_quant_sym_status(int32_t* flag_host) {
  CFB_CHECK_ARG(flag_host != nullptr, "NULL argument");
  CFB_CUDA(cudaDeviceSynchronize());
  int v = 0;
  CFB_CUDA(cudaMemcpyFromSymbol(&v, g_pflag, sizeof(int)));
  *flag_host = v;
  return CFB200_OK;
}

#ifdef CFB_A1_TRACE
extern "C" int32_t cfb200_debug_a1_trace(unsigned long long* host_out /* 3 * 200 * 8 */) {
  CFB_CUDA(cudaDeviceSynchronize());
  CFB_CUDA(cudaMemcpyFromSymbol(host_out, g_ptrace, sizeof(unsigned long long) * 3 * kTracePhases * kTraceSlots));
  return CFB200_OK;
}
extern "C" int32_t cfb200_debug_a1_trace_all(unsigned long long* host_out /* 160 * 32 * 2 */) {
  CFB_CUDA(cudaDeviceSynchronize());
  CFB_CUDA(cudaMemcpyFromSymbol(host_out, g_ptrace_all, sizeof(unsigned long long) * 160 * 32 * 2));
  return CFB200_OK;
}
#endif

namespace cfb {
// Runs the probe, returns what cfb200_quant_sym_status reports afterwards, and clears the flag again.
int32_t a1_expired_wait_selftest(int32_t* observed) {
  a1_wait_probe_kernel<<<1, 32>>>(1u << 12);
  CFB_LAUNCH_CHECK();
  int32_t rc = cfb200_quant_sym_status(observed);
  const int zero = 0;
  CFB_CUDA(cudaMemcpyToSymbol(g_pflag, &zero, sizeof(int)));
  return rc;
}
}  // namespace cfb

extern "C" int32_t cfb200_quant_sym_apply(const void* src, int32_t src_dtype, size_t n, int32_t bits,
                                          const float* absmax, int8_t* codes, float* scale_absmax, void* stream) {
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ARG(scale_absmax != nullptr && absmax != nullptr, "scale_absmax or absmax is NULL");
  CFB_CHECK_ARG(n == 0 || (src && codes), "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 16);
  StageArgs a = {};
  bounds_of(bits, &a.qmin, &a.qmax);
  a.n_apply = 1;
  a.apply[0] = Seg{src, n, codes, reinterpret_cast<unsigned*>(const_cast<float*>(absmax)), scale_absmax};
  a.check_range = 1;  // the absmax is the caller's: it may be smaller than this shard's
  a.demote = tunable(kTuneA1Demote) != 0;
  return launch_stage(src_dtype, a, (cudaStream_t)stream);
}

extern "C" int32_t cfb200_quant_sym_tensor(const void* src, int32_t src_dtype, size_t n, int32_t bits,
                                           int8_t* codes, float* scale_absmax, void* stream) {
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ARG(scale_absmax != nullptr, "scale_absmax is NULL");
  CFB_CHECK_ARG(n == 0 || (src && codes), "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 16);
  CFB_CHECK_ALIGNED(scale_absmax, 8);
  cudaStream_t st = (cudaStream_t)stream;
  // scale_absmax[1] doubles as the atomicMax accumulator (bit pattern of a non-negative float)
  CFB_CUDA(cudaMemsetAsync(scale_absmax, 0, 2 * sizeof(float), st));
  StageArgs a = {};
  bounds_of(bits, &a.qmin, &a.qmax);
  // A large tensor goes through the persistent kernel (bulk-copy ring, tail kept on chip).  That path copies a
  // descriptor from host memory, which a stream under graph capture cannot do: those calls keep the two launches.
  if (use_persist(src_dtype) && n * dtype_size(src_dtype) >= ((size_t)32 << 20)) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
      const void* srcs[1] = {src};
      int8_t* outs[1] = {codes};
      const int ge[1] = {1};
      return run_persist(1, srcs, src_dtype, &n, a.qmin, a.qmax, outs, scale_absmax, ge, 1, default_group_bytes(), nullptr, st);
    }
  }
  a.keep = tunable(kTuneA1KeepMB) == 0;  // knob value 0 (default) = keep pass 1's lines in L2
  a.merge = (int)tunable(kTuneA1Merge);
  a.demote = tunable(kTuneA1Demote) != 0;
  const Seg sg{src, n, codes, reinterpret_cast<unsigned*>(scale_absmax + 1), scale_absmax};
  a.n_amax = 1;
  a.amax[0] = sg;
  int32_t rc = launch_stage(src_dtype, a, st);
  if (rc) return rc;
  a.n_amax = 0;
  a.n_apply = 1;
  a.apply[0] = sg;
  return launch_stage(src_dtype, a, st);
}

extern "C" int32_t cfb200_quant_sym_tensors_plan(int32_t count, const size_t* ns, int32_t src_dtype,
                                                 size_t l2_group_bytes, int32_t* n_stages) {
  CFB_CHECK_ARG(count >= 0 && (count == 0 || ns) && n_stages, "bad arguments");
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  if (count == 0) { *n_stages = 0; return CFB200_OK; }
  int* ge = new int[count];
  const int ng = plan_groups(count, ns, src_dtype, l2_group_bytes, ge);
  if (use_persist(src_dtype)) {  // launches = descriptor tables
    int launches = 0, g = 0;
    while (g < ng) {
      const int first = g > 0 ? ge[g - 1] : 0;
      int g_hi = g;
      while (g_hi < ng && ge[g_hi] - first <= kPMaxTensors) ++g_hi;
      if (g_hi == g) break;
      g = g_hi;
      ++launches;
    }
    *n_stages = launches;
  } else {
    *n_stages = ng + 1;
  }
  delete[] ge;
  return CFB200_OK;
}

extern "C" int32_t cfb200_quant_sym_tensors(int32_t count, const void* const* srcs, int32_t src_dtype,
                                            const size_t* ns, int32_t bits, int8_t* const* codes,
                                            float* scale_absmax, size_t l2_group_bytes,
                                            void* const* stage_events, void* stream) {
  CFB_CHECK_ARG(count >= 0, "negative count");
  if (count == 0) return CFB200_OK;
  CFB_CHECK_ARG(srcs && ns && codes && scale_absmax, "NULL argument");
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ALIGNED(scale_absmax, 8);
  for (int i = 0; i < count; ++i) {
    CFB_CHECK_ARG(ns[i] == 0 || (srcs[i] && codes[i]), "tensor %d: NULL buffer", i);
    CFB_CHECK_ALIGNED(srcs[i], 16);
    CFB_CHECK_ALIGNED(codes[i], 16);
  }
  cudaStream_t st = (cudaStream_t)stream;
  int* ge = new int[count];
  const int ng = plan_groups(count, ns, src_dtype, l2_group_bytes, ge);
  CFB_CUDA(cudaMemsetAsync(scale_absmax, 0, (size_t)count * 2 * sizeof(float), st));
  StageArgs a = {};
  bounds_of(bits, &a.qmin, &a.qmax);
  a.keep = tunable(kTuneA1KeepMB) == 0;  // knob value 0 (default) = keep pass 1's lines in L2
  a.merge = (int)tunable(kTuneA1Merge);
  a.demote = tunable(kTuneA1Demote) != 0;
  int32_t rc = CFB200_OK;
  if (use_persist(src_dtype)) {
    // one cooperative launch per table of tensors; stage_events[k] precedes launch k, the last one follows
    rc = run_persist(count, srcs, src_dtype, ns, a.qmin, a.qmax, codes, scale_absmax, ge, ng,
                     l2_group_bytes ? l2_group_bytes : default_group_bytes(), stage_events, st);
    delete[] ge;
    return rc;
  }
  for (int stage = 0; stage <= ng && rc == CFB200_OK; ++stage) {
    a.n_apply = a.n_amax = 0;
    if (stage > 0)
      for (int i = stage > 1 ? ge[stage - 2] : 0; i < ge[stage - 1]; ++i)
        a.apply[a.n_apply++] = Seg{srcs[i], ns[i], codes[i], reinterpret_cast<unsigned*>(scale_absmax + 2 * i + 1), scale_absmax + 2 * i};
    if (stage < ng)
      for (int i = stage > 0 ? ge[stage - 1] : 0; i < ge[stage]; ++i)
        a.amax[a.n_amax++] = Seg{srcs[i], ns[i], codes[i], reinterpret_cast<unsigned*>(scale_absmax + 2 * i + 1), scale_absmax + 2 * i};
    if (stage_events && stage_events[stage]) {
      if (cudaEventRecord((cudaEvent_t)stage_events[stage], st) != cudaSuccess) rc = set_error(CFB200_ERR_CUDA, "cudaEventRecord failed");
    }
    if (rc == CFB200_OK) rc = launch_stage(src_dtype, a, st);
  }
  if (rc == CFB200_OK && stage_events && stage_events[ng + 1]) {
    if (cudaEventRecord((cudaEvent_t)stage_events[ng + 1], st) != cudaSuccess) rc = set_error(CFB200_ERR_CUDA, "cudaEventRecord failed");
  }
  delete[] ge;
  return rc;
}


// E4: the per-tensor E4M3FN weight cast over a whole list of tensors, through the same cooperative launch as A1 (absmax
// pass of a group under the cast pass of the previous one, tails kept on chip): scale = absmax < 1e-12 ? 1 : absmax / 448,
// codes = e4m3(v * (1 / scale)), identical to cfb200_cast_e4m3_tensor tensor by tensor.
extern "C" int32_t cfb200_cast_e4m3_tensors(int32_t count, const void* const* srcs, int32_t src_dtype, const size_t* ns,
                                            uint8_t* const* codes, float* scale_absmax, size_t l2_group_bytes, void* stream) {
  CFB_CHECK_ARG(count >= 0, "negative count");
  if (count == 0) return CFB200_OK;
  CFB_CHECK_ARG(srcs && ns && codes && scale_absmax, "NULL argument");
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ALIGNED(scale_absmax, 8);
  for (int i = 0; i < count; ++i) {
    CFB_CHECK_ARG(ns[i] == 0 || (srcs[i] && codes[i]), "tensor %d: NULL buffer", i);
    CFB_CHECK_ALIGNED(srcs[i], 16);
    CFB_CHECK_ALIGNED(codes[i], 16);
  }
  cudaStream_t st = (cudaStream_t)stream;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
    return set_error(CFB200_ERR_UNSUPPORTED, "cfb200_cast_e4m3_tensors copies a descriptor table from host memory: not under stream capture");
  int* ge = new int[count];
  const int ng = plan_groups(count, ns, src_dtype, l2_group_bytes, ge);
  int32_t rc = CFB200_OK;
  if (cudaMemsetAsync(scale_absmax, 0, (size_t)count * 2 * sizeof(float), st) != cudaSuccess) rc = set_error(CFB200_ERR_CUDA, "cudaMemsetAsync failed");
  if (rc == CFB200_OK)
    rc = run_persist(count, srcs, src_dtype, ns, -448.0f, 448.0f, reinterpret_cast<int8_t* const*>(codes), scale_absmax, ge, ng,
                     l2_group_bytes ? l2_group_bytes : default_group_bytes(), nullptr, st, 1);
  delete[] ge;
  return rc;
}
