// Shared device/host helpers for the sm_100a kernels of the quantize-and-execute path.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/cfb200.h"

namespace cfb {

// ---------------------------------------------------------------------------------------------
// host side: status + last-error text (thread local), device properties
// ---------------------------------------------------------------------------------------------
int32_t set_error(int32_t code, const char* fmt, ...);
int sm_count();  // SMs of the current device (cached per device)

// Performance knobs (never change results).  Read with tunable(), set with cfb200_tune().
enum Tunable {
  kTuneA1KeepMB = 0,   // non-zero: pass 1 of A1 streams (no L2 retention) -- for experiments
  kTuneA1Demote = 1,   // pass 2 of A1 reads with an evict_first policy (releases the kept lines)
  kTuneA1Merge = 2,    // A1 stage kernel advances its two passes in lockstep
  kTuneA1Persist = 3,  // A1 list entry point runs as one cooperative launch that keeps tensor heads on chip
  kTuneA1GroupMB = 4,  // L2 budget of a tensor group in MB (0 = default)
  kTuneA1RetainMB = 5, // persistent A1: MB of a group's tail that pass 1 leaves in L2 at normal priority (0 = all)
  kTuneGemvRing = 6,   // decode W4A16: large shapes go through the shared-memory ring kernel
  kTuneGemvRingRounds = 7,  // row blocks per cluster the ring kernel asks for before it splits K further (0 = default 1)
  kTuneW4SplitK = 8,   // W4A16 prefill: 0 = automatic split-K for M <= 256, 1 = never, n > 1 = at most n slices
  kTuneA1BarSleep = 9, // persistent A1: nanoseconds between two polls of the grid barrier (0 = poll back to back)
  kTuneA1TailFirst = 10, // persistent A1: the quantize pass re-reads the lines kept in L2 before the ones that were let go
  kTuneGemmPair = 11,  // tensor-core GEMMs: two CTAs (a cluster, two SMs) per 256 x 256 tile where the shape has one
  kTuneColparP2P = 12, // column-parallel products: 1 = blocks rejoined by this library's peer-load kernel where the ranks can map each other's memory, 0 = always NCCL all-gather
  kTuneCount
};
long long tunable(int id);
// Give-up-path self-tests (a short bounded wait on a barrier nothing completes): what the host then observes.
int32_t a1_expired_wait_selftest(int32_t* observed);
int32_t tc_expired_wait_selftest(int32_t* observed, int which);

#define CFB_CHECK_ARG(cond, ...)                                        \
  do {                                                                  \
    if (!(cond)) return cfb::set_error(CFB200_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define CFB_CHECK_ALIGNED(ptr, a)                                                            \
  do {                                                                                       \
    if ((reinterpret_cast<uintptr_t>(ptr) & ((a) - 1)) != 0)                                 \
      return cfb::set_error(CFB200_ERR_MISALIGNED, "%s must be %d-byte aligned", #ptr, (int)(a)); \
  } while (0)

#define CFB_CUDA(call)                                                                      \
  do {                                                                                      \
    cudaError_t e__ = (call);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return cfb::set_error(CFB200_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

#define CFB_LAUNCH_CHECK()                                                                  \
  do {                                                                                      \
    cudaError_t e__ = cudaGetLastError();                                                   \
    if (e__ != cudaSuccess)                                                                 \
      return cfb::set_error(CFB200_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e__)); \
  } while (0)

inline size_t dtype_size(int32_t dt) { return dt == CFB200_F32 ? 4 : 2; }
inline bool dtype_ok(int32_t dt) { return dt == CFB200_F32 || dt == CFB200_F16 || dt == CFB200_BF16; }

// ---------------------------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned kFullMask = 0xffffffffu;

// 128-bit read-only load that does not allocate in L1 (every input byte is used exactly once
// per pass; L2 keeps it for a second pass).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 128-bit read-only load with default L2 allocation: for data a following launch re-reads.
// (On B200 the L1::no_allocate form above is also first in line for L2 eviction: a second pass
// over data read that way misses.)
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// 256-bit streaming load (sm_100): 32 contiguous bytes per lane in one instruction
struct Raw32 { uint32_t w[8]; };
__device__ __forceinline__ Raw32 ld_stream32(const void* p) {
  Raw32 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
               : "l"(p));
  return r;
}
// 32 bytes from an address that is only known to be 16-byte aligned: the 256-bit form needs 32-byte alignment, which a
// caller's buffer (aligned to 16 as the entry points ask) need not have.  The test is uniform over a launch.
__device__ __forceinline__ Raw32 ld_stream32_any(const void* p) {
  if ((reinterpret_cast<uintptr_t>(p) & 31u) == 0) return ld_stream32(p);
  Raw32 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]) : "l"(p));
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
               : "l"(static_cast<const char*>(p) + 16));
  return r;
}
__device__ __forceinline__ uint2 ld_stream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
// The same load with an explicit L2 eviction policy (createpolicy.fractional.*).
__device__ __forceinline__ uint4 ld_stream16_policy(const void* p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// Streaming stores: results are never read back by the producing kernel.
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream8(void* p, uint2 v) {
#if defined(CFB_ST_VARIANT) && CFB_ST_VARIANT == 1
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
#elif defined(CFB_ST_VARIANT) && CFB_ST_VARIANT == 2
  if (v.x == 0x12345678u && v.y == 0x9abcdef0u) asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
#elif defined(CFB_ST_VARIANT) && CFB_ST_VARIANT == 3
  asm volatile("st.global.cg.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
#else
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
#endif
}
__device__ __forceinline__ void st_stream4(void* p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Widening of one stored element to f32, bit-identical to the reference's converters
// (tensor_store.rs:58-82 for f16 incl. subnormals, :104-106 for bf16).
template <int DT> struct Elem;
template <> struct Elem<CFB200_F32> {
  using type = float;
  static constexpr int kBytes = 4;
  static __device__ __forceinline__ float widen(float v) { return v; }
};
template <> struct Elem<CFB200_F16> {
  using type = __half;
  static constexpr int kBytes = 2;
  static __device__ __forceinline__ float widen(__half v) { return __half2float(v); }
};
template <> struct Elem<CFB200_BF16> {
  using type = __nv_bfloat16;
  static constexpr int kBytes = 2;
  static __device__ __forceinline__ float widen(__nv_bfloat16 v) {
    return __uint_as_float(((uint32_t)__bfloat16_as_ushort(v)) << 16);
  }
};

// Unpack a 16-byte vector into 16/sizeof(elem) floats.
template <int DT> struct Vec16;
template <> struct Vec16<CFB200_F32> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void unpack(uint4 r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
};
template <> struct Vec16<CFB200_BF16> {
  static constexpr int kElems = 8;
  typedef __nv_bfloat162 Pair2;  // two elements of a 32-bit word (low half = the earlier element)
  static __device__ __forceinline__ Pair2 zero2() { return __floats2bfloat162_rn(0.0f, 0.0f); }
  static __device__ __forceinline__ float low_f32(Pair2 p) { return __uint_as_float(*reinterpret_cast<const uint32_t*>(&p) << 16); }
  static __device__ __forceinline__ float high_f32(Pair2 p) { return __uint_as_float(*reinterpret_cast<const uint32_t*>(&p) & 0xffff0000u); }
  static __device__ __forceinline__ void unpack(uint4 r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Vec16<CFB200_F16> {
  static constexpr int kElems = 8;
  typedef __half2 Pair2;
  static __device__ __forceinline__ Pair2 zero2() { return __floats2half2_rn(0.0f, 0.0f); }
  static __device__ __forceinline__ float low_f32(Pair2 p) { return __low2float(p); }
  static __device__ __forceinline__ float high_f32(Pair2 p) { return __high2float(p); }
  static __device__ __forceinline__ void unpack(uint4 r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};

template <int DT>
__device__ __forceinline__ float load_elem(const void* base, size_t i) {
  return Elem<DT>::widen(reinterpret_cast<const typename Elem<DT>::type*>(base)[i]);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

// max over aligned sub-groups of LANES lanes (LANES a power of two <= 32)
template <int LANES>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}
template <int LANES>
__device__ __forceinline__ float group_min(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
// Exact round(v / scale) without an IEEE division on the common path.
//
// The reference computes `(v / scale).round()` with a correctly rounded division and
// round-half-away-from-zero.  An IEEE division costs ~10 instructions, which would make the
// packing kernels issue-bound before they are HBM-bound, so the quotient is first estimated as
// n = rne(v * (1/scale)) with the add-magic-number trick, and proven right with one FMA:
// r = v - n*scale (single rounding).  If |r| < 0.5*scale*(1 - 2^-10) then the true quotient is
// further than 2^-11 from a rounding tie, which is more than the rounding error of the exact
// division for |quotient| <= 2048, so roundf(v/scale) == n.  Otherwise (a near-tie, |n| large,
// NaN or infinity anywhere: the comparison is false) the slow path does the real division.
// ---------------------------------------------------------------------------------------------
struct DivRound {
  float scale, inv, half_lo;
  __device__ __forceinline__ explicit DivRound(float s) {
    scale = s;
    inv = __fdiv_rn(1.0f, s);
    half_lo = 0.5f * s * (1.0f - 0.0009765625f);
  }
  // Returns roundf(v / scale) as a float (may be NaN, as in the reference, when v or the
  // quotient is NaN).  Requires the caller to clamp afterwards.
  __device__ __forceinline__ float operator()(float v) const {
    const float magic = 12582912.0f;  // 1.5 * 2^23
    float n = __fadd_rn(__fmaf_rn(v, inv, magic), -magic);
    float r = __fmaf_rn(-n, scale, v);
    if (fabsf(r) < half_lo && fabsf(n) <= 2048.0f) return n;
    return roundf(__fdiv_rn(v, scale));
  }
};

// ---------------------------------------------------------------------------------------------
// Branch-free exact |round_half_away(v / scale)| for quotients below 127.5.
//
// 16-bit sources (EXACT_DIV = false): D = fma(fma(-scale, q0, v), inv, q0) with q0 = v*inv and
// inv = RN(1/scale) is one Newton correction of the quotient.  It is not always RN(v/scale), but
// an exhaustive host check over every (absmax, v) pair of bf16 and of f16 patterns with
// |v| <= absmax, scale = absmax/127 or absmax/7, shows that the rounded code below is always the
// one the reference gets from the IEEE division (tests/test_fastpath_exhaustive.py).
// f32 sources (EXACT_DIV = true) use the IEEE division itself.
// Rounding: a = RZ(|D| * 2^16 + 2^23 + 2^15) holds floor(|D|*2^16 + 2^15) in its mantissa, so
// byte 2 of a's bit pattern is floor(|D| + 0.5) -- round half away from zero of the magnitude,
// with no second rounding because the truncation can never reach a tie from below.
// NaN (from a NaN element, or inf/inf) becomes magnitude 0, like `NaN as i8` in the reference.
// ---------------------------------------------------------------------------------------------
// FINITE: the caller knows that no element is NaN or infinite, so the quotient needs no NaN guard.
template <bool EXACT_DIV, bool FINITE = false>
__device__ __forceinline__ float quant_mag_fixed(float v, float scale, float inv) {
  float D;
  if (EXACT_DIV) D = __fdiv_rn(v, scale);
  else {
    const float q0 = __fmul_rn(v, inv);
    D = __fmaf_rn(__fmaf_rn(-scale, q0, v), inv, q0);
  }
  if (FINITE) return __fmaf_rz(fabsf(D), 65536.0f, 8388608.0f + 32768.0f);
  return __fmaf_rz(fmaxf(fabsf(D), 0.0f), 65536.0f, 8388608.0f + 32768.0f);
}
// the rounding step alone, for a quotient the caller has already made NaN-free and < 127.5
__device__ __forceinline__ float round_mag_fixed(float D) {
  return __fmaf_rz(fabsf(D), 65536.0f, 8388608.0f + 32768.0f);
}
template <bool EXACT_DIV>
__device__ __forceinline__ float quotient(float v, float scale, float inv) {
  if (EXACT_DIV) return __fdiv_rn(v, scale);
  const float q0 = __fmul_rn(v, inv);
  return __fmaf_rn(__fmaf_rn(-scale, q0, v), inv, q0);
}
// byte 2 of four fixed-point values -> one word of magnitudes
__device__ __forceinline__ uint32_t pack_mag4(float a0, float a1, float a2, float a3) {
  return __byte_perm(__byte_perm(__float_as_uint(a0), __float_as_uint(a1), 0x0062),
                     __byte_perm(__float_as_uint(a2), __float_as_uint(a3), 0x0062), 0x5410);
}
// per-byte two's-complement negation of the bytes of P (each 0..128) selected by M (0x00 / 0xFF)
__device__ __forceinline__ uint32_t negate_bytes(uint32_t P, uint32_t M) {
  const uint32_t x = P ^ M;
  return (((x & 0x7f7f7f7fu) + (M & 0x01010101u)) ^ (x & 0x80808080u));
}
// prmt.b32 with full selector nibbles: bit 3 of a nibble replicates the selected byte's sign bit
// over the result byte (the __byte_perm intrinsic drops that bit).
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// 0xFF per negative element: sign bytes of four consecutive 16-bit elements held in w0, w1 ...
__device__ __forceinline__ uint32_t sign_mask_16(uint32_t w0, uint32_t w1) { return prmt_raw(w0, w1, 0xFDB9u); }
// ... and of four f32 elements
__device__ __forceinline__ uint32_t sign_mask_32(uint32_t f0, uint32_t f1, uint32_t f2, uint32_t f3) {
  return __byte_perm(prmt_raw(f0, f1, 0x00FBu), prmt_raw(f2, f3, 0x00FBu), 0x5410);
}

// f32 -> f16 bit pattern the way the reference stores it: mantissa truncated, subnormal results flushed to +-0,
// overflow to infinity, NaN kept as a quiet NaN.
__host__ __device__ inline uint16_t f32_to_f16_bits_trunc(float val) {  // tensor_store.rs:85-101
#ifdef __CUDA_ARCH__
  const uint32_t bits = __float_as_uint(val);
#else
  uint32_t bits;
  memcpy(&bits, &val, 4);
#endif
  const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  const int exp = (int)((bits >> 23) & 0xffu);
  const uint32_t mant = bits & 0x007fffffu;
  if (exp == 255) return (uint16_t)(sign | 0x7c00u | (mant != 0 ? 0x0200u : 0u));
  const int ne = exp - 127 + 15;
  if (ne >= 31) return (uint16_t)(sign | 0x7c00u);
  if (ne <= 0) return sign;
  return (uint16_t)(sign | ((uint16_t)ne << 10) | (uint16_t)(mant >> 13));
}

// Rust `clamp` then `as i8`/`as u8`: NaN -> 0.
__device__ __forceinline__ int clamp_to_int(float x, float lo, float hi) {
  if (x != x) return 0;
  return __float2int_rz(fminf(fmaxf(x, lo), hi));
}

// State of the exact k-th-largest-|v| radix select (three passes of 11 + 10 + 10 bits, MSB first; kernels in quant_group.cu).
constexpr int kSelectBins = 2048;
struct SelectState {
  unsigned long long hist[kSelectBins];
  unsigned long long k;          // rank still to find inside the current prefix (1 = largest); after the last pass: the
                                 // rank inside the elements equal to the threshold
  unsigned long long bin_count;  // elements in the bin chosen by the latest pass; after the last pass: how many equal the threshold
  unsigned prefix;               // bits fixed so far (in place)
  unsigned mask;                 // which bits are fixed
  unsigned ticket;               // CTAs that have delivered their histogram in the running pass (the last one scans)
  unsigned pad;
};
// sub != NULL: select over src - sub, which the first pass also writes to diff_out (n floats, 16-byte aligned).
// fast_ws / fast_bytes: optional extra workspace (select_fast_workspace_bytes(n)); with it, and for ranks in the top
// 5 % of a tensor of a million elements or more, the tensor is read ONCE: a sample brackets the threshold, one pass counts
// what lies above the bracket and collects what lies inside it, and the exact rank is found among those candidates.
// The bracket is verified on the device (count above < k <= count above + candidates); if it does not hold, the
// three full passes run instead, so the result is exact either way.
size_t select_fast_workspace_bytes(size_t n);
int32_t select_kth_abs_rank(const float* src, size_t n, unsigned long long k, float* thr_out, SelectState* state, cudaStream_t st,
                            const float* sub = nullptr, float* diff_out = nullptr, void* fast_ws = nullptr, size_t fast_bytes = 0);

#endif  // __CUDACC__

}  // namespace cfb
