// KV-cache page codecs on the device.
//
//   K16/V8  (AsymK16V8Codec, src/passes/serving/kv_attention.rs:52-222): keys become f16 bit patterns through the
//           truncating f32_to_f16_bits (src/ir/tensor_store.rs:85-101); values become INT8 codes
//           clamp(round(v / scale), -127, 127) with scale = absmax / 127 (1.0 when the absmax is 0) taken per tensor,
//           per kv head, or per (page, kv head).  Layout [num_pages, page_tokens, num_kv_heads, head_dim], contiguous.
//   E4M3FN slice codec (quantize_f32_slice_to_fp8_e4m3fn / dequantize_fp8_e4m3fn_slice_to_f32,
//           src/passes/serving/mutable_loads.rs:431-441): one byte per element, no scale.
//
// All of it is byte traffic bound by HBM.  The per-(page, head) scope runs as ONE launch: a CTA owns a page, takes
// the per-head absmax of its values into shared memory, and re-reads the page (64 KB for 16 tokens x 8 heads x 128,
// so the second read is served by L1 / L2) to emit the codes; the keys ride along in the same pass.  The two wider
// scopes need every page before the first code can be written: absmax launch (shared-memory maxima per CTA, one
// atomic per head per CTA), a one-block scale launch, then the same encode pass.
#include <math.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace cfb {
namespace {

constexpr int kThreadsKv = 256;
constexpr int kMaxHeads = 1024;

enum { kScopeTensor = 0, kScopeLayerHead = 1, kScopePageHead = 2 };

struct KvGeom {
  size_t num_pages;
  uint32_t page_vecs;     // 16-byte source vectors per page
  uint32_t vecs_per_row;  // head_dim / elements per vector
  uint32_t heads;
  uint32_t row_shift, head_mask;  // set when vecs_per_row and heads are powers of two (head_mask = heads - 1), else 0xffffffff
};

__device__ __forceinline__ uint32_t head_of(const KvGeom& g, uint32_t v) {
  if (g.row_shift != 0xffffffffu) return (v >> g.row_shift) & g.head_mask;
  return (v / g.vecs_per_row) % g.heads;
}

__device__ __forceinline__ float scale_of_absmax(float amax) {  // kv_attention.rs:139-144
  return amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
}

// Two keys -> two truncated f16 bit patterns.  For 2^-14 <= |x| < 65536 truncating the mantissa is the hardware's
// round-toward-zero conversion; below (flush to +-0), above (infinity) and NaN (quiet NaN 0x7e00) the reference's
// converter differs from it and the scalar restatement is used.
__device__ __forceinline__ uint32_t f16_bits_trunc_pair(float a, float b) {
  const uint32_t ua = (__float_as_uint(a) & 0x7fffffffu) - 0x38800000u, ub = (__float_as_uint(b) & 0x7fffffffu) - 0x38800000u;
  if (max(ua, ub) < 0x47800000u - 0x38800000u) {
    uint32_t d;
    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));  // first source operand lands in the upper half
    return d;
  }
  return (uint32_t)f32_to_f16_bits_trunc(a) | ((uint32_t)f32_to_f16_bits_trunc(b) << 16);
}

// absmax of one page's values into smax[heads] (positive floats order like their bit patterns)
template <int DT>
__device__ __forceinline__ void page_absmax(const KvGeom& g, const uint8_t* vp, unsigned* smax, bool per_head) {
  constexpr int VE = Vec16<DT>::kElems;
  constexpr int U = 4;  // loads in flight per thread
  for (uint32_t i0 = threadIdx.x; i0 < g.page_vecs; i0 += U * kThreadsKv) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = i0 + u * kThreadsKv;
      r[u] = i < g.page_vecs ? ld_cached16(vp + (size_t)i * 16) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = i0 + u * kThreadsKv;
      if (i >= g.page_vecs) break;
      float f[VE];
      Vec16<DT>::unpack(r[u], f);
      float m = 0.0f;
#pragma unroll
      for (int k = 0; k < VE; ++k) m = fmaxf(m, fabsf(f[k]));  // fmaxf drops a NaN operand, like f32::max
      const uint32_t h = per_head ? head_of(g, i) : 0u;
      if (__float_as_uint(m) > smax[h]) atomicMax(&smax[h], __float_as_uint(m));
    }
  }
}

// keys -> f16 bit patterns, values -> codes, for one page; sscale[h] / sinv[h] hold the scale of head h and its
// reciprocal (or [0] for all).  Every |v| is at most the absmax its scale was made from, so the quotient stays below
// 127.5 and the clamp never acts: the branch-free rounding of common.cuh applies.  Its division-free quotient is
// proven for 16-bit sources with a finite absmax >= 1e-12 only; scales outside of that (sinv[h] == 0) take the
// reference formula literally.
template <int DT>
__device__ __forceinline__ void page_encode(const KvGeom& g, const uint8_t* kp, const uint8_t* vp, uint16_t* ko, int8_t* vo,
                                            const float* sscale, const float* sinv, bool per_head) {
  constexpr int VE = Vec16<DT>::kElems;
  constexpr int U = 2;  // (value, key) vector pairs in flight per thread
  for (uint32_t i0 = threadIdx.x; i0 < g.page_vecs; i0 += U * kThreadsKv) {
    uint4 rvs[U], rks[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = i0 + u * kThreadsKv;
      if (i < g.page_vecs) {
        rvs[u] = ld_stream16(vp + (size_t)i * 16);
        rks[u] = ld_stream16(kp + (size_t)i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
    const uint32_t i = i0 + u * kThreadsKv;
    if (i >= g.page_vecs) break;
    const uint4 rv = rvs[u];
    float fv[VE], fk[VE];
    Vec16<DT>::unpack(rv, fv);
    Vec16<DT>::unpack(rks[u], fk);
    const uint32_t h = per_head ? head_of(g, i) : 0u;
    const float sc = sscale[h], inv = sinv[h];
    uint32_t codes[VE / 4], kb[VE / 2];
    if (inv != 0.0f) {
      float a[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) a[e] = quant_mag_fixed<DT == CFB200_F32, false>(fv[e], sc, inv);
      if constexpr (DT == CFB200_F32) {
        codes[0] = negate_bytes(pack_mag4(a[0], a[1], a[2], a[3]), sign_mask_32(rv.x, rv.y, rv.z, rv.w));
      } else {
        codes[0] = negate_bytes(pack_mag4(a[0], a[1], a[2], a[3]), sign_mask_16(rv.x, rv.y));
        codes[1] = negate_bytes(pack_mag4(a[4], a[5], a[6], a[7]), sign_mask_16(rv.z, rv.w));
      }
    } else {
#pragma unroll
      for (int w = 0; w < VE / 4; ++w) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b)
          acc |= ((uint32_t)clamp_to_int(roundf(__fdiv_rn(fv[4 * w + b], sc)), -127.0f, 127.0f) & 0xffu) << (8 * b);
        codes[w] = acc;
      }
    }
#pragma unroll
    for (int w = 0; w < VE / 2; ++w) kb[w] = f16_bits_trunc_pair(fk[2 * w], fk[2 * w + 1]);
    if constexpr (VE == 8) {
      st_stream8(vo + (size_t)i * VE, make_uint2(codes[0], codes[1]));
      st_stream16(ko + (size_t)i * VE, make_uint4(kb[0], kb[1], kb[2], kb[3]));
    } else {
      st_stream4(vo + (size_t)i * VE, codes[0]);
      st_stream8(ko + (size_t)i * VE, make_uint2(kb[0], kb[1]));
    }
    }
  }
}
// reciprocal of a scale for the branch-free path, 0 where that path is not proven (see page_encode)
template <int DT>
__device__ __forceinline__ float fast_inv(float scale) {
  // f32 sources divide exactly, so only the flag matters; a scale that underflowed to 0 or near it must not get here
  if (DT == CFB200_F32) return (scale >= 1e-30f && scale < __uint_as_float(0x7f800000u)) ? 1.0f : 0.0f;
  return (scale >= 1e-14f && scale < __uint_as_float(0x7f800000u)) ? __fdiv_rn(1.0f, scale) : 0.0f;
}

// scope = per (page, head): one launch, a CTA per page
template <int DT>
__global__ void __launch_bounds__(kThreadsKv, 5)
kv_encode_page_scope_kernel(KvGeom g, const uint8_t* __restrict__ k, const uint8_t* __restrict__ v, uint16_t* __restrict__ ko,
                            int8_t* __restrict__ vo, float* __restrict__ v_scales) {
  __shared__ unsigned smax[kMaxHeads];
  __shared__ float sscale[kMaxHeads], sinv[kMaxHeads];
  const size_t page_bytes = (size_t)g.page_vecs * 16, page_elems = (size_t)g.page_vecs * Vec16<DT>::kElems;
  for (size_t p = blockIdx.x; p < g.num_pages; p += gridDim.x) {
    for (uint32_t h = threadIdx.x; h < g.heads; h += kThreadsKv) smax[h] = 0u;
    __syncthreads();
    page_absmax<DT>(g, v + p * page_bytes, smax, true);
    __syncthreads();
    for (uint32_t h = threadIdx.x; h < g.heads; h += kThreadsKv) {
      const float s = scale_of_absmax(__uint_as_float(smax[h]));
      sscale[h] = s;
      sinv[h] = fast_inv<DT>(s);
      v_scales[p * g.heads + h] = s;
    }
    __syncthreads();
    page_encode<DT>(g, k + p * page_bytes, v + p * page_bytes, ko + p * page_elems, vo + p * page_elems, sscale, sinv, true);
    __syncthreads();
  }
}

// the wider scopes, launch 1: absmax per head (or of everything) into amax_bits (zeroed by the caller)
template <int DT>
__global__ void __launch_bounds__(kThreadsKv)
kv_absmax_kernel(KvGeom g, const uint8_t* __restrict__ v, unsigned* __restrict__ amax_bits, int per_head) {
  __shared__ unsigned smax[kMaxHeads];
  const uint32_t slots = per_head ? g.heads : 1u;
  for (uint32_t h = threadIdx.x; h < slots; h += kThreadsKv) smax[h] = 0u;
  __syncthreads();
  const size_t page_bytes = (size_t)g.page_vecs * 16;
  for (size_t p = blockIdx.x; p < g.num_pages; p += gridDim.x) page_absmax<DT>(g, v + p * page_bytes, smax, per_head != 0);
  __syncthreads();
  for (uint32_t h = threadIdx.x; h < slots; h += kThreadsKv)
    if (smax[h] != 0u) atomicMax(&amax_bits[h], smax[h]);
}
// launch 2: absmax bit patterns -> scales, in place
__global__ void kv_scales_kernel(float* scales, uint32_t slots) {
  for (uint32_t h = threadIdx.x; h < slots; h += blockDim.x) scales[h] = scale_of_absmax(scales[h]);
}
// launch 3: encode
template <int DT>
__global__ void __launch_bounds__(kThreadsKv, 5)
kv_encode_kernel(KvGeom g, const uint8_t* __restrict__ k, const uint8_t* __restrict__ v, uint16_t* __restrict__ ko,
                 int8_t* __restrict__ vo, const float* __restrict__ v_scales, int per_head) {
  __shared__ float sscale[kMaxHeads], sinv[kMaxHeads];
  const uint32_t slots = per_head ? g.heads : 1u;
  for (uint32_t h = threadIdx.x; h < slots; h += kThreadsKv) {
    sscale[h] = v_scales[h];
    sinv[h] = fast_inv<DT>(sscale[h]);
  }
  __syncthreads();
  const size_t page_bytes = (size_t)g.page_vecs * 16, page_elems = (size_t)g.page_vecs * Vec16<DT>::kElems;
  // back to front: the absmax launch walked the pages front to back, so the last ones are the values L2 still holds
  for (size_t q = blockIdx.x; q < g.num_pages; q += gridDim.x) {
    const size_t p = g.num_pages - 1 - q;
    page_encode<DT>(g, k + p * page_bytes, v + p * page_bytes, ko + p * page_elems, vo + p * page_elems, sscale, sinv, per_head != 0);
  }
}

// decode: four elements per thread; k_out = widen(f16 bits), v_out = (code as f32) * scale (kv_attention.rs:186-221)
__global__ void __launch_bounds__(kThreadsKv)
kv_decode_kernel(const uint16_t* __restrict__ kb, const int8_t* __restrict__ vc, const float* __restrict__ v_scales, size_t nquads,
                 uint32_t quads_per_row, uint32_t heads, uint32_t rows_per_page, int scope, float* __restrict__ k_out,
                 float* __restrict__ v_out) {
  const size_t stride = (size_t)gridDim.x * kThreadsKv;
  constexpr int U = 4;  // quads in flight per thread
  for (size_t i0 = (size_t)blockIdx.x * kThreadsKv + threadIdx.x; i0 < nquads; i0 += U * stride) {
    uint2 kws[U];
    uint32_t cws[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + u * stride;
      if (i < nquads) {
        kws[u] = ld_stream8(kb + i * 4);
        asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(cws[u]) : "l"(vc + i * 4));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= nquads) break;
      const uint2 kw = kws[u];
      const uint32_t cw = cws[u];
      const size_t row = i / quads_per_row;  // (page, token, head) index
      const uint32_t h = (uint32_t)(row % heads);
      const size_t slot = scope == kScopeTensor ? 0 : scope == kScopeLayerHead ? h : (row / rows_per_page) * heads + h;
      const float s = v_scales[slot];
      const __half2 k01 = *reinterpret_cast<const __half2*>(&kw.x), k23 = *reinterpret_cast<const __half2*>(&kw.y);
      const float2 a = __half22float2(k01), b = __half22float2(k23);
      st_stream16(k_out + i * 4, make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(b.x), __float_as_uint(b.y)));
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __fmul_rn((float)(int8_t)((cw >> (8 * j)) & 0xffu), s);
      st_stream16(v_out + i * 4, make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3])));
    }
  }
}

// E4M3FN slice codec: four elements per thread.
// REF: reproduce the reference codec (src/passes/serving/mutable_loads.rs:367-410) where it departs from round-to-
// nearest-even.  It takes the exponent as floor(log2f(|v|)); for a value a few ulp below a power of two 2^k the f32
// logarithm rounds up to k, the mantissa term comes out slightly negative, `floor` gives -1, the round-up step adds one
// to a mantissa that `as u8` clamped to 0, and the byte encodes 1.125 * 2^k instead of 2^k.  Which of the eight values
// below each 2^k do this depends on the host's log2f, so the host evaluates it once (c_slip: bit t-1 of entry k+5 set =
// 2^k * (1 - t * 2^-24) slips) and the kernel patches exactly those inputs.
__constant__ uint8_t c_e4m3_slip[16];

template <bool REF>
__device__ __forceinline__ uint32_t e4m3_fix(uint32_t code, uint32_t bits) {
  if constexpr (!REF) return code;
  const uint32_t mant = bits & 0x7fffffu, ex = (bits >> 23) & 0xffu;
  if (mant < 0x7ffff8u) return code;                    // not within 8 ulp below a power of two
  const int k = (int)ex - 127 + 1;                      // the value lies just below 2^k
  if (k < -5 || k > 8) return code;                     // below the normal range (other branch of the codec) or saturated
  const uint32_t t = 0x800000u - mant;                  // 1..8
  if (!((c_e4m3_slip[k + 5] >> (t - 1)) & 1u)) return code;
  return (bits >> 24 & 0x80u) | (uint32_t)((k + 7) << 3) | 1u;   // k + 7 <= 15 and mantissa 1 < 7: never the NaN / saturation byte
}

template <bool REF>
__global__ void __launch_bounds__(kThreadsKv) e4m3_slice_encode_kernel(const float* __restrict__ src, size_t n, uint8_t* __restrict__ out) {
  const size_t nq = n / 4;
  for (size_t i = (size_t)blockIdx.x * kThreadsKv + threadIdx.x; i < nq; i += (size_t)gridDim.x * kThreadsKv) {
    const uint4 r = ld_stream16(src + i * 4);
    unsigned short lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(__uint_as_float(r.y)), "f"(__uint_as_float(r.x)));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(__uint_as_float(r.w)), "f"(__uint_as_float(r.z)));
    uint32_t word = (uint32_t)lo | ((uint32_t)hi << 16);
    if constexpr (REF) {
      word = e4m3_fix<true>(word & 0xffu, r.x) | (e4m3_fix<true>((word >> 8) & 0xffu, r.y) << 8) |
             (e4m3_fix<true>((word >> 16) & 0xffu, r.z) << 16) | (e4m3_fix<true>(word >> 24, r.w) << 24);
    }
    st_stream4(out + i * 4, word);
  }
  if (blockIdx.x == 0)
    for (size_t i = nq * 4 + threadIdx.x; i < n; i += kThreadsKv) {
      unsigned short pk;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(src[i]));
      out[i] = (uint8_t)e4m3_fix<REF>(pk & 0xffu, __float_as_uint(src[i]));
    }
}
__device__ __forceinline__ float e4m3_value(uint32_t b) {  // mutable_loads.rs:413-429
  const uint32_t exp = (b >> 3) & 0xfu, mant = b & 7u;
  float mag;
  if (exp == 0xfu && mant == 7u) return __uint_as_float(0x7fc00000u);  // f32::NAN
  if (exp == 0) mag = (float)mant * (1.0f / 512.0f);
  else mag = __uint_as_float(((exp + 120u) << 23) | (mant << 20));  // (1 + mant/8) * 2^(exp-7), exact
  return (b & 0x80u) ? -mag : mag;
}
__global__ void __launch_bounds__(kThreadsKv) e4m3_slice_decode_kernel(const uint8_t* __restrict__ codes, size_t n, float* __restrict__ out) {
  const size_t nq = n / 4, stride = (size_t)gridDim.x * kThreadsKv;
  constexpr int U = 4;  // words in flight per thread; a warp's loads and stores stay contiguous
  for (size_t i0 = (size_t)blockIdx.x * kThreadsKv + threadIdx.x; i0 < nq; i0 += U * stride) {
    uint32_t cw[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < nq) asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(cw[u]) : "l"(codes + (i0 + u * stride) * 4));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= nq) break;
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = e4m3_value((cw[u] >> (8 * j)) & 0xffu);
      st_stream16(out + i * 4, make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3])));
    }
  }
  if (blockIdx.x == 0)
    for (size_t i = nq * 4 + threadIdx.x; i < n; i += kThreadsKv) out[i] = e4m3_value(codes[i]);
}

unsigned kv_grid(size_t work_items) {
  const size_t cap = (size_t)sm_count() * 8;
  return (unsigned)std::max<size_t>(1, std::min(work_items, cap));
}

template <int DT>
int32_t kv_encode_dt(const KvGeom& g, const void* k, const void* v, int32_t scope, uint16_t* ko, int8_t* vo, float* v_scales,
                     cudaStream_t st) {
  const uint8_t* kp = static_cast<const uint8_t*>(k);
  const uint8_t* vp = static_cast<const uint8_t*>(v);
  const unsigned grid = kv_grid(g.num_pages);
  if (scope == kScopePageHead) {
    kv_encode_page_scope_kernel<DT><<<grid, kThreadsKv, 0, st>>>(g, kp, vp, ko, vo, v_scales);
    CFB_LAUNCH_CHECK();
    return CFB200_OK;
  }
  const int per_head = scope == kScopeLayerHead;
  const uint32_t slots = per_head ? g.heads : 1u;
  CFB_CUDA(cudaMemsetAsync(v_scales, 0, slots * sizeof(float), st));
  kv_absmax_kernel<DT><<<grid, kThreadsKv, 0, st>>>(g, vp, reinterpret_cast<unsigned*>(v_scales), per_head);
  CFB_LAUNCH_CHECK();
  kv_scales_kernel<<<1, 256, 0, st>>>(v_scales, slots);
  CFB_LAUNCH_CHECK();
  kv_encode_kernel<DT><<<grid, kThreadsKv, 0, st>>>(g, kp, vp, ko, vo, v_scales, per_head);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

bool is_pow2(uint32_t x) { return x && !(x & (x - 1)); }
uint32_t log2u(uint32_t x) { uint32_t s = 0; while ((1u << s) < x) ++s; return s; }

}  // namespace
}  // namespace cfb

using namespace cfb;

extern "C" size_t cfb200_kv_scale_count(int32_t scope, size_t num_pages, size_t num_kv_heads) {
  return scope == kScopeTensor ? 1 : scope == kScopeLayerHead ? num_kv_heads : num_pages * num_kv_heads;
}

extern "C" int32_t cfb200_kv_encode_k16v8(const void* k, const void* v, int32_t src_dtype, size_t num_pages, size_t page_tokens,
                                          size_t num_kv_heads, size_t head_dim, int32_t scope, uint16_t* k_f16_bits, int8_t* v_codes,
                                          float* v_scales, void* stream) {
  CFB_CHECK_ARG(k && v && k_f16_bits && v_codes && v_scales, "NULL buffer");
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown source dtype %d", src_dtype);
  CFB_CHECK_ARG(scope >= kScopeTensor && scope <= kScopePageHead, "scope must be 0 (tensor), 1 (layer-head) or 2 (page-head)");
  // the reference rejects an empty shape (kv_attention.rs:77-85)
  CFB_CHECK_ARG(num_pages > 0 && page_tokens > 0 && num_kv_heads > 0 && head_dim > 0, "AsymK16V8Codec::encode shape mismatch: expected 0 elems");
  const size_t ve = 16 / dtype_size(src_dtype);
  CFB_CHECK_ARG(head_dim % ve == 0, "head_dim must be a multiple of %zu for this source dtype (got %zu)", ve, head_dim);
  CFB_CHECK_ARG(num_kv_heads <= (size_t)kMaxHeads, "at most %d kv heads (got %zu)", kMaxHeads, num_kv_heads);
  const size_t page_vecs = page_tokens * num_kv_heads * (head_dim / ve);
  CFB_CHECK_ARG(page_vecs < (1ull << 31), "a page holds too many elements");
  CFB_CHECK_ALIGNED(k, 16);
  CFB_CHECK_ALIGNED(v, 16);
  CFB_CHECK_ALIGNED(k_f16_bits, 16);
  CFB_CHECK_ALIGNED(v_codes, 8);
  KvGeom g;
  g.num_pages = num_pages;
  g.page_vecs = (uint32_t)page_vecs;
  g.vecs_per_row = (uint32_t)(head_dim / ve);
  g.heads = (uint32_t)num_kv_heads;
  if (is_pow2(g.vecs_per_row) && is_pow2(g.heads)) { g.row_shift = log2u(g.vecs_per_row); g.head_mask = g.heads - 1; }
  else { g.row_shift = 0xffffffffu; g.head_mask = 0; }
  cudaStream_t st = (cudaStream_t)stream;
  switch (src_dtype) {
    case CFB200_F32: return kv_encode_dt<CFB200_F32>(g, k, v, scope, k_f16_bits, v_codes, v_scales, st);
    case CFB200_F16: return kv_encode_dt<CFB200_F16>(g, k, v, scope, k_f16_bits, v_codes, v_scales, st);
    default: return kv_encode_dt<CFB200_BF16>(g, k, v, scope, k_f16_bits, v_codes, v_scales, st);
  }
}

extern "C" int32_t cfb200_kv_decode_k16v8(const uint16_t* k_f16_bits, const int8_t* v_codes, const float* v_scales, size_t num_pages,
                                          size_t page_tokens, size_t num_kv_heads, size_t head_dim, int32_t scope, float* k_out,
                                          float* v_out, void* stream) {
  CFB_CHECK_ARG(k_f16_bits && v_codes && v_scales && k_out && v_out, "NULL buffer");
  CFB_CHECK_ARG(scope >= kScopeTensor && scope <= kScopePageHead, "scope must be 0 (tensor), 1 (layer-head) or 2 (page-head)");
  CFB_CHECK_ARG(num_pages > 0 && page_tokens > 0 && num_kv_heads > 0 && head_dim > 0 && head_dim % 4 == 0,
                "empty shape or head_dim not a multiple of 4");
  CFB_CHECK_ARG(head_dim / 4 < (1ull << 31) && num_kv_heads < (1ull << 31) && page_tokens * num_kv_heads < (1ull << 31), "dimension too large");
  CFB_CHECK_ALIGNED(k_f16_bits, 8);
  CFB_CHECK_ALIGNED(v_codes, 4);
  CFB_CHECK_ALIGNED(k_out, 16);
  CFB_CHECK_ALIGNED(v_out, 16);
  const size_t nquads = num_pages * page_tokens * num_kv_heads * (head_dim / 4);
  kv_decode_kernel<<<kv_grid((nquads + kThreadsKv - 1) / kThreadsKv), kThreadsKv, 0, (cudaStream_t)stream>>>(
      k_f16_bits, v_codes, v_scales, nquads, (uint32_t)(head_dim / 4), (uint32_t)num_kv_heads, (uint32_t)(page_tokens * num_kv_heads), scope,
      k_out, v_out);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

extern "C" int32_t cfb200_e4m3_slice_encode(const float* src, size_t n, uint8_t* codes, void* stream) {
  if (n == 0) return CFB200_OK;
  CFB_CHECK_ARG(src && codes, "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 4);
  e4m3_slice_encode_kernel<false><<<kv_grid((n / 4 + kThreadsKv) / kThreadsKv), kThreadsKv, 0, (cudaStream_t)stream>>>(src, n, codes);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// The reference codec bit for bit, its log2f binade slips included (see e4m3_fix).  The slip table is built from THIS
// host's log2f on the first call on each device -- the function the reference's f32::log2 resolves to on the same host.
extern "C" int32_t cfb200_e4m3_slice_encode_ref(const float* src, size_t n, uint8_t* codes, void* stream) {
  if (n == 0) return CFB200_OK;
  CFB_CHECK_ARG(src && codes, "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 4);
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CFB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  {
    static std::mutex m;
    static bool ready[64];
    std::lock_guard<std::mutex> lock(m);
    if (!ready[dev]) {
      uint8_t slip[16] = {0};
      for (int k = -5; k <= 8; ++k)
        for (int t = 1; t <= 8; ++t) {
          uint32_t bits = ((uint32_t)(k - 1 + 127) << 23) | (0x800000u - (uint32_t)t);
          float x;
          memcpy(&x, &bits, 4);
          volatile float lg = log2f(x);  // volatile: evaluated by the library at run time, not folded by the compiler
          if ((int)floorf(lg) == k) slip[k + 5] |= (uint8_t)(1u << (t - 1));
        }
      CFB_CUDA(cudaMemcpyToSymbol(c_e4m3_slip, slip, sizeof slip));
      ready[dev] = true;
    }
  }
  e4m3_slice_encode_kernel<true><<<kv_grid((n / 4 + kThreadsKv) / kThreadsKv), kThreadsKv, 0, (cudaStream_t)stream>>>(src, n, codes);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

extern "C" int32_t cfb200_e4m3_slice_decode(const uint8_t* codes, size_t n, float* out, void* stream) {
  if (n == 0) return CFB200_OK;
  CFB_CHECK_ARG(codes && out, "NULL buffer");
  CFB_CHECK_ALIGNED(codes, 4);
  CFB_CHECK_ALIGNED(out, 16);
  e4m3_slice_decode_kernel<<<kv_grid((n / 4 + kThreadsKv) / kThreadsKv), kThreadsKv, 0, (cudaStream_t)stream>>>(codes, n, out);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}
