// Group-/block-wise quantization kernels (HBM-bound, single pass over the weights):
//   A2  group-wise fake quantization + exact k-th |v| selection   (schemes.rs:483-570)
//   A3  FP8 "grid" fake quantization                              (schemes.rs:658-716)
//   A4  E2M1 fake quantization                                    (formats.rs:369-383, :414-479)
//   E2  asymmetric INT4 with f16 scale / u4 zero point, packed
//   E3  NF4 with 8-bit double-quantised absmax
//
// Work decomposition.  A lane owns EPL (4 or 8) consecutive elements, loaded with one or two
// 128-bit instructions; a group of G = EPL * LPG elements is owned by LPG consecutive lanes
// (LPG a power of two <= 32), so group statistics are butterfly shuffles and never touch
// shared memory.  A warp processes kItems warp-slots of 32*EPL elements per loop trip to keep
// several loads in flight; the grid is persistent (a multiple of the SM count).
// Group sizes with no such decomposition go through a one-thread-per-group fallback.
#include <math.h>

#include <mutex>
#include <vector>
#include <type_traits>

#include "common.cuh"
#include "nf4_codebook.inc"

namespace cfb {
namespace {

constexpr int kThreads = 256;
#ifndef CFB_QG_ITEMS
#define CFB_QG_ITEMS 2
#endif
constexpr int kItems = CFB_QG_ITEMS;

// -------- lane loads / stores ------------------------------------------------------------------
template <int DT, int EPL>
__device__ __forceinline__ int lane_load(const void* __restrict__ src, size_t n, size_t e0, float (&f)[EPL]) {
  constexpr int EB = Elem<DT>::kBytes;
  const char* p = reinterpret_cast<const char*>(src) + e0 * EB;
  if (e0 + EPL <= n) {
    if constexpr (EB == 4 && EPL == 4) {
      Vec16<DT>::unpack(ld_stream16(p), f);
    } else if constexpr (EB == 4 && EPL == 8) {
      uint4 a = ld_stream16(p), b = ld_stream16(p + 16);
      Vec16<DT>::unpack(a, f);
      Vec16<DT>::unpack(b, f + 4);
    } else if constexpr (EB == 2 && EPL == 8) {
      Vec16<DT>::unpack(ld_stream16(p), f);
    } else if constexpr (EB == 2 && EPL == 16) {
      uint4 a = ld_stream16(p), b = ld_stream16(p + 16);
      float t0[8], t1[8];
      Vec16<DT>::unpack(a, t0);
      Vec16<DT>::unpack(b, t1);
#pragma unroll
      for (int k = 0; k < 8; ++k) { f[k] = t0[k]; f[8 + k] = t1[k]; }
    } else {  // 16-bit, 4 elements: 8 bytes
      uint2 r = ld_stream8(p);
      float t[8];
      Vec16<DT>::unpack(make_uint4(r.x, r.y, 0, 0), t);
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = t[k];
    }
    return EPL;
  }
  int nv = e0 < n ? (int)(n - e0) : 0;
#pragma unroll
  for (int k = 0; k < EPL; ++k) f[k] = k < nv ? load_elem<DT>(src, e0 + k) : 0.0f;
  return nv;
}

template <int EPL>
__device__ __forceinline__ void lane_store_f32(float* __restrict__ out, size_t e0, int nv, const float (&o)[EPL]) {
  if (nv == EPL) {
#pragma unroll
    for (int k = 0; k < EPL; k += 4)
      st_stream16(out + e0 + k, make_uint4(__float_as_uint(o[k]), __float_as_uint(o[k + 1]),
                                           __float_as_uint(o[k + 2]), __float_as_uint(o[k + 3])));
  } else {
#pragma unroll
    for (int k = 0; k < EPL; ++k)
      if (k < nv) out[e0 + k] = o[k];
  }
}

// pack EPL 4-bit codes (low nibble first) and store EPL/2 bytes at byte offset e0/2
template <int EPL>
__device__ __forceinline__ void lane_store_nibbles(uint8_t* __restrict__ codes, size_t e0, int nv, const int (&c)[EPL]) {
  unsigned long long w = 0;
#pragma unroll
  for (int k = 0; k < EPL; ++k) w |= (unsigned long long)(k < nv ? ((uint32_t)c[k] & 0xfu) : 0u) << (4 * k);  // padding packs as 0
  if (nv == EPL) {
    if constexpr (EPL == 16) st_stream8(codes + (e0 >> 1), make_uint2((uint32_t)w, (uint32_t)(w >> 32)));
    else if constexpr (EPL == 8) st_stream4(codes + (e0 >> 1), (uint32_t)w);
    else *reinterpret_cast<uint16_t*>(codes + (e0 >> 1)) = (uint16_t)w;
  } else {
    int nbytes = (nv + 1) >> 1;
    for (int b = 0; b < nbytes; ++b) codes[(e0 >> 1) + b] = (uint8_t)(w >> (8 * b));
  }
}

struct WarpWork {
  size_t nslots_pairs, warp_id, warps_total;
  int lane;
};
template <int EPL>
__device__ __forceinline__ WarpWork warp_work(size_t n) {
  WarpWork w;
  const size_t slot = 32 * (size_t)EPL;
  const size_t nslots = (n + slot - 1) / slot;
  w.nslots_pairs = (nslots + kItems - 1) / kItems;
  w.warps_total = (size_t)gridDim.x * (kThreads / 32);
  w.warp_id = (size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  w.lane = threadIdx.x & 31;
  return w;
}

__device__ __forceinline__ float keep_nan_clamp(float q, float lo, float hi) {
  return (q != q) ? q : fminf(fmaxf(q, lo), hi);  // Rust f32::clamp keeps NaN
}

// -------- A2 -----------------------------------------------------------------------------------
__device__ __forceinline__ float a2_elem(float v, float sc, const DivRound& d1, const DivRound& d2,
                                         bool awq, float thr, float qmin, float qmax) {
  const bool sal = awq && (fabsf(v) >= thr);
  float q = sal ? d2(v) : d1(v);
  q = keep_nan_clamp(copysignf(q, v), qmin, qmax);
  return __fmul_rn(q, sal ? d2.scale : sc);
}

template <int EPL, int LPG>
__global__ void __launch_bounds__(kThreads)
fakequant_group_kernel(const float* __restrict__ src, size_t n, float qmin, float qmax, int awq,
                       const float* __restrict__ thr_p, float* __restrict__ out) {
  const WarpWork w = warp_work<EPL>(n);
  const float thr = awq ? *thr_p : 0.0f;
  // the loads of a trip are issued one trip ahead (register double buffer)
  float nf[kItems][EPL];
  int nnv[kItems];
  auto fetch = [&](size_t pr2) {
#pragma unroll
    for (int it = 0; it < kItems; ++it) nnv[it] = lane_load<CFB200_F32, EPL>(src, n, ((pr2 * kItems + it) * 32 + w.lane) * EPL, nf[it]);
  };
  if (w.warp_id < w.nslots_pairs) fetch(w.warp_id);
  for (size_t pr = w.warp_id; pr < w.nslots_pairs; pr += w.warps_total) {
    float f[kItems][EPL];
    int nv[kItems];
    size_t e0[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
      nv[it] = nnv[it];
#pragma unroll
      for (int k = 0; k < EPL; ++k) f[it][k] = nf[it][k];
    }
    if (pr + w.warps_total < w.nslots_pairs) fetch(pr + w.warps_total);
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      float m = 0.0f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) m = fmaxf(m, fabsf(f[it][k]));  // padded lanes hold 0
      m = group_max<LPG>(m);
      const float sc = (m < 1e-12f) ? 1.0f : __fdiv_rn(m, qmax);
      const DivRound d1(sc), d2(__fmul_rn(sc, 0.5f));
      float o[EPL];
#pragma unroll
      for (int k = 0; k < EPL; ++k) o[k] = a2_elem(f[it][k], sc, d1, d2, awq != 0, thr, qmin, qmax);
      lane_store_f32<EPL>(out, e0[it], nv[it], o);
    }
  }
}

// any group size: one thread per group
__global__ void fakequant_group_generic_kernel(const float* __restrict__ src, size_t n, size_t g, float qmin,
                                               float qmax, int awq, const float* __restrict__ thr_p,
                                               float* __restrict__ out) {
  const float thr = awq ? *thr_p : 0.0f;
  const size_t ngroups = (n + g - 1) / g;
  for (size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += (size_t)gridDim.x * blockDim.x) {
    size_t lo = gi * g, hi = lo + g < n ? lo + g : n;
    float m = 0.0f;
    for (size_t i = lo; i < hi; ++i) m = fmaxf(m, fabsf(src[i]));
    const float sc = (m < 1e-12f) ? 1.0f : __fdiv_rn(m, qmax);
    const DivRound d1(sc), d2(__fmul_rn(sc, 0.5f));
    for (size_t i = lo; i < hi; ++i) out[i] = a2_elem(src[i], sc, d1, d2, awq != 0, thr, qmin, qmax);
  }
}

// -------- exact k-th largest |v| (radix select, passes of 11 + 10 + 10 bits, MSB first) --------
__global__ void select_init_kernel(SelectState* s, unsigned long long k) {
  for (int i = threadIdx.x; i < kSelectBins; i += blockDim.x) s->hist[i] = 0;
  if (threadIdx.x == 0) { s->k = k; s->prefix = 0; s->mask = 0; s->ticket = 0; }
}

// One block of 256 threads: a thread owns nbins / 256 consecutive bins; suffix sums of the threads' totals (counted from
// the top) and a short walk inside the owning thread's bins locate the bin holding rank k; its bits are fixed and
// the bins are cleared.  Run by the LAST CTA of a histogram pass (ticket), so a pass is one launch.
__device__ __forceinline__ void select_scan_block(SelectState* s, int shift, int nbits, float* thr_out, int last, unsigned base = 0u) {
  __shared__ unsigned long long suf[256 + 1];
  const int t = threadIdx.x, per = (1 << nbits) / 256;  // 4 or 8 bins per thread
  unsigned long long bins[kSelectBins / 256];
  unsigned long long mine = 0;
  // written by other CTAs' atomics: read from L2 (ld.cg), all of a thread's loads in flight together
#pragma unroll
  for (int j = 0; j < kSelectBins / 256; ++j) bins[j] = j < per ? __ldcg(&s->hist[t * per + j]) : 0ull;
#pragma unroll
  for (int j = 0; j < kSelectBins / 256; ++j)
    if (j < per) {
      s->hist[t * per + j] = 0;
      mine += bins[j];
    }
  suf[t] = mine;
  if (t == 0) suf[256] = 0;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {  // suf[t] = sum of the bins of threads t .. 255
    const unsigned long long add = (t + o < 256) ? suf[t + o] : 0ull;
    __syncthreads();
    suf[t] += add;
    __syncthreads();
  }
  const unsigned long long k = __ldcg(&s->k);
  __syncthreads();
  // walking down from the top bin, the first bin whose suffix sum reaches k holds the rank; bin 0 if none does
  const bool none = suf[0] < k;
  if ((suf[t] >= k && suf[t + 1] < k) || (none && t == 0)) {
    unsigned long long above = suf[t + 1];
    int b = per - 1;
    if (none) b = 0;
    else
      for (; b > 0; --b) {
        if (above + bins[b] >= k) break;
        above += bins[b];
      }
    s->k = none ? k - (suf[0] - bins[0]) : k - above;
    s->prefix |= ((unsigned)(t * per + b)) << shift;
    s->mask |= ((1u << nbits) - 1u) << shift;
    s->bin_count = bins[b];
    if (last) {
      s->prefix += base;  // candidate passes work on offsets from the lower edge of the bracket
      *thr_out = __uint_as_float(s->prefix);
    }
  }
}

// Tail of every histogram pass: the CTA's bins go to the global histogram, and the CTA that delivers last scans it.
__device__ __forceinline__ void select_deliver_and_scan(const unsigned* sh, unsigned nbins, SelectState* s, int shift, int nbits,
                                                        float* thr_out, int last, unsigned base = 0u) {
  __shared__ int s_last;
  for (unsigned i = threadIdx.x; i < nbins; i += kThreads)
    if (sh[i]) atomicAdd(&s->hist[i], (unsigned long long)sh[i]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&s->ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    __threadfence();
    select_scan_block(s, shift, nbits, thr_out, last, base);
    __syncthreads();
    if (threadIdx.x == 0) s->ticket = 0;
  }
}

__global__ void __launch_bounds__(kThreads)
select_hist_kernel(const float* __restrict__ src, const float* __restrict__ sub, float* __restrict__ diff_out, size_t n, int shift,
                   int nbits, SelectState* __restrict__ s, float* thr_out, int last, const int* skip_if_set) {
  // sub != NULL: the values are src - sub, which this pass also writes to diff_out (the later passes read them there)
  __shared__ unsigned sh[kSelectBins];
  if (skip_if_set && __ldcg(skip_if_set)) return;  // the single-pass path already found the answer
  const unsigned nbins = 1u << nbits, bin_mask = nbins - 1u;
  for (unsigned i = threadIdx.x; i < nbins; i += kThreads) sh[i] = 0;
  __syncthreads();
  const unsigned prefix = __ldcg(&s->prefix), mask = __ldcg(&s->mask);
  auto add = [&](unsigned bits) {
    unsigned key = bits & 0x7fffffffu;  // |v| under IEEE total order; NaN above +inf
    if ((key & mask) == prefix) atomicAdd(&sh[(key >> shift) & bin_mask], 1u);
  };
  const size_t nvec = n / 4;
  const uint4* p = reinterpret_cast<const uint4*>(src);
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (size_t)gridDim.x * kThreads) {
    uint4 r = __ldg(p + i);
    if (sub) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(sub) + i);
      r.x = __float_as_uint(__fsub_rn(__uint_as_float(r.x), __uint_as_float(q.x)));
      r.y = __float_as_uint(__fsub_rn(__uint_as_float(r.y), __uint_as_float(q.y)));
      r.z = __float_as_uint(__fsub_rn(__uint_as_float(r.z), __uint_as_float(q.z)));
      r.w = __float_as_uint(__fsub_rn(__uint_as_float(r.w), __uint_as_float(q.w)));
      reinterpret_cast<uint4*>(diff_out)[i] = r;
    }
    add(r.x); add(r.y); add(r.z); add(r.w);
  }
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - nvec * 4)) {
    const size_t i = nvec * 4 + threadIdx.x;
    float v = src[i];
    if (sub) { v = __fsub_rn(v, sub[i]); diff_out[i] = v; }
    add(__float_as_uint(v));
  }
  __syncthreads();
  select_deliver_and_scan(sh, nbins, s, shift, nbits, thr_out, last);
}

// ---- single-pass path: sample -> bracket -> one full pass -> exact rank among the candidates -----------------------
constexpr int kSampleBits = 13, kSampleBins = 1 << kSampleBits, kSampleShift = 31 - kSampleBits;  // top 13 bits of |v|
constexpr int kFastStage = 2048;       // candidates a CTA of the bracket pass can hold in shared memory
constexpr unsigned kFastSpanBits = 21; // the bracket must span fewer than 2^21 keys: two radix passes (11 + 10 bits) over the offsets
constexpr size_t kSampleCount = 1u << 18;
struct SelectFast {
  unsigned lo_key, hi_key;           // candidates: lo_key <= key < hi_key
  unsigned long long cnt_above;      // keys >= hi_key
  unsigned long long cand_total;     // candidates written to the dense buffer
  int fast_ok, overflow;
  unsigned ticket, pad;
  unsigned sample_hist[kSampleBins];
};

__device__ __forceinline__ unsigned abs_key(float v) { return __float_as_uint(v) & 0x7fffffffu; }

// A spread-out sample of the tensor, binned on the top 14 magnitude bits; the last CTA turns the two sample ranks that
// bracket rank k (6 standard deviations of the sample count on either side) into a key range.
__global__ void __launch_bounds__(kThreads)
select_sample_kernel(const float* __restrict__ src, const float* __restrict__ sub, size_t n, size_t samples, unsigned long long k,
                     SelectFast* __restrict__ f, SelectState* __restrict__ s) {
  __shared__ unsigned sh[kSampleBins];  // 32 KB: the CTA's own histogram, delivered once
  for (int i = threadIdx.x; i < kSampleBins; i += kThreads) sh[i] = 0;
  __syncthreads();
  const size_t stride = n / samples;  // >= 4: the path is only taken for large tensors
  const size_t step = (size_t)gridDim.x * kThreads;
  for (size_t j0 = (size_t)blockIdx.x * kThreads + threadIdx.x; j0 < samples; j0 += 4 * step) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {  // four independent loads in flight per thread
      const size_t j = j0 + u * step;
      const size_t pos = j * stride + (size_t)((unsigned)(j * 2654435761u) % (unsigned)(stride < 0xffffffffu ? stride : 0xffffffffu));
      v[u] = j < samples ? __ldg(src + pos) : 0.0f;
      if (sub && j < samples) v[u] = __fsub_rn(v[u], __ldg(sub + pos));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u * step < samples) atomicAdd(&sh[abs_key(v[u]) >> kSampleShift], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kSampleBins; i += kThreads)
    if (sh[i]) atomicAdd(&f->sample_hist[i], sh[i]);
  __shared__ int s_last;
  __shared__ unsigned long long suf[kThreads + 1];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&f->ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  constexpr int per = kSampleBins / kThreads;  // 64 consecutive bins per thread
  const int t = threadIdx.x;
  unsigned bins[per];
  unsigned long long mine = 0;
#pragma unroll
  for (int j = 0; j < per; ++j) bins[j] = __ldcg(&f->sample_hist[t * per + j]);
#pragma unroll
  for (int j = 0; j < per; ++j) mine += bins[j];
  suf[t] = mine;
  if (t == 0) suf[kThreads] = 0;
  __syncthreads();
  for (int o = 1; o < kThreads; o <<= 1) {
    const unsigned long long add = (t + o < kThreads) ? suf[t + o] : 0ull;
    __syncthreads();
    suf[t] += add;
    __syncthreads();
  }
  const double ks = (double)k * (double)samples / (double)n;
  const double m = 6.0 * sqrt(ks > 1.0 ? ks : 1.0) + 8.0;
  const double r_hi = ks - m, r_lo = ks + m;
  if (t == 0) {
    if (r_hi < 1.0) f->hi_key = 0x80000000u;   // nothing is assumed to lie above the bracket
    if (r_lo > (double)suf[0]) f->lo_key = 0u;
    f->ticket = 0;
    s->k = k;  // the select state was cleared by the memset that precedes this launch; only the rank is not zero
  }
  // bin of sample rank r (counted from the top): suffix(bin) >= r > suffix(bin + 1)
  auto locate = [&](double r, bool upper_edge) {
    const unsigned long long rr = (unsigned long long)ceil(r);
    if (suf[t] >= rr && suf[t + 1] < rr) {
      unsigned long long above = suf[t + 1];
      int b = per - 1;
      bool found = false;
#pragma unroll
      for (int j = per - 1; j > 0; --j) {  // registers: unrolled, no dependent memory trips
        if (!found) {
          if (above + bins[j] >= rr) { b = j; found = true; }
          else above += bins[j];
        }
      }
      if (!found) b = 0;
      const unsigned bin = (unsigned)(t * per + b);
      if (upper_edge) f->hi_key = (bin + 1u) << kSampleShift;  // bin 16383 -> 0x80000000
      else f->lo_key = bin << kSampleShift;
    }
  };
  if (r_hi >= 1.0) locate(r_hi, true);
  if (r_lo <= (double)suf[0]) locate(r_lo, false);
}

// The one full pass: keys at or above the bracket are counted, keys inside it are collected in shared memory and
// appended to the dense candidate buffer with one reservation per CTA.  The last CTA checks that rank k falls among the
// candidates.
__global__ void __launch_bounds__(kThreads)
select_bracket_kernel(const float* __restrict__ src, const float* __restrict__ sub, float* __restrict__ diff_out, size_t n,
                      unsigned long long k, SelectFast* __restrict__ f, unsigned* __restrict__ cand, unsigned long long cand_cap,
                      SelectState* __restrict__ s) {
  __shared__ unsigned s_stage[kFastStage];
  __shared__ unsigned s_cnt;
  __shared__ unsigned long long s_base;
  __shared__ int s_last;
  __shared__ unsigned long long s_sum[kThreads / 32];
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  const unsigned lo = f->lo_key, hi = f->hi_key;
  unsigned above = 0;
  auto visit = [&](unsigned bits) {
    const unsigned key = bits & 0x7fffffffu;
    if (key >= hi) ++above;
    else if (key >= lo) {
      const unsigned slot = atomicAdd(&s_cnt, 1u);
      if (slot < (unsigned)kFastStage) s_stage[slot] = key - lo;  // offset from the lower edge
    }
  };
  const size_t nvec = n / 4;
  const uint4* p = reinterpret_cast<const uint4*>(src);
  const size_t gstep = (size_t)gridDim.x * kThreads;
  size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (!sub) {  // plain tensor: four loads in flight per thread
    for (; i + 3 * gstep < nvec; i += 4 * gstep) {
      const uint4 r0 = ld_stream16(p + i), r1 = ld_stream16(p + i + gstep), r2 = ld_stream16(p + i + 2 * gstep), r3 = ld_stream16(p + i + 3 * gstep);
      visit(r0.x); visit(r0.y); visit(r0.z); visit(r0.w);
      visit(r1.x); visit(r1.y); visit(r1.z); visit(r1.w);
      visit(r2.x); visit(r2.y); visit(r2.z); visit(r2.w);
      visit(r3.x); visit(r3.y); visit(r3.z); visit(r3.w);
    }
  }
  for (; i < nvec; i += gstep) {
    uint4 r = ld_stream16(p + i);
    if (sub) {
      const uint4 q = ld_stream16(reinterpret_cast<const uint4*>(sub) + i);
      r.x = __float_as_uint(__fsub_rn(__uint_as_float(r.x), __uint_as_float(q.x)));
      r.y = __float_as_uint(__fsub_rn(__uint_as_float(r.y), __uint_as_float(q.y)));
      r.z = __float_as_uint(__fsub_rn(__uint_as_float(r.z), __uint_as_float(q.z)));
      r.w = __float_as_uint(__fsub_rn(__uint_as_float(r.w), __uint_as_float(q.w)));
      reinterpret_cast<uint4*>(diff_out)[i] = r;
    }
    visit(r.x); visit(r.y); visit(r.z); visit(r.w);
  }
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)(n - nvec * 4)) {
    const size_t i = nvec * 4 + threadIdx.x;
    float v = src[i];
    if (sub) { v = __fsub_rn(v, sub[i]); diff_out[i] = v; }
    visit(__float_as_uint(v));
  }
  unsigned long long a = above;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(kFullMask, a, o);
  if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = a;
  __syncthreads();
  const unsigned cnt = s_cnt < (unsigned)kFastStage ? s_cnt : (unsigned)kFastStage;
  if (threadIdx.x == 0) {
    unsigned long long tot = 0;
    for (int w = 0; w < kThreads / 32; ++w) tot += s_sum[w];
    if (tot) atomicAdd(&f->cnt_above, tot);
    if (s_cnt > (unsigned)kFastStage) atomicExch(&f->overflow, 1);
    s_base = cnt ? atomicAdd(&f->cand_total, (unsigned long long)cnt) : 0ull;
  }
  __syncthreads();
  const unsigned long long base = s_base;
  if (base + cnt <= cand_cap) {
    for (unsigned i = threadIdx.x; i < cnt; i += kThreads) cand[base + i] = s_stage[i];
  } else if (threadIdx.x == 0) atomicExch(&f->overflow, 1);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&f->ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) {  // last CTA: does rank k fall among the candidates?
    const unsigned long long total = *reinterpret_cast<volatile unsigned long long*>(&f->cand_total);
    const unsigned long long ab = *reinterpret_cast<volatile unsigned long long*>(&f->cnt_above);
    const bool ok = !*reinterpret_cast<volatile int*>(&f->overflow) && ab < k && k <= ab + total && hi - lo <= (1u << kFastSpanBits);
    f->fast_ok = ok ? 1 : 0;
    s->k = ok ? k - ab : k;   // rank among the candidates, or the untouched rank for the three full passes
    f->ticket = 0;
  }
}

// The radix passes over the dense candidate buffer (its length is on the device).  The candidates share their top bits,
// so they are stored as offsets from the lower edge of the bracket (< 2^21) and two passes, 11 + 10 bits, resolve them.
__global__ void __launch_bounds__(kThreads)
select_hist_cand_kernel(const unsigned* __restrict__ cand, const SelectFast* __restrict__ f, int shift, int nbits,
                        SelectState* __restrict__ s, float* thr_out, int last) {
  __shared__ unsigned sh[kSelectBins];
  const int fast_ok = __ldcg(&f->fast_ok);
  const unsigned prefix = __ldcg(&s->prefix), mask = __ldcg(&s->mask), base = __ldcg(&f->lo_key);
  const size_t total = (size_t)__ldcg(&f->cand_total);
  if (!fast_ok) return;
  const unsigned nbins = 1u << nbits, bin_mask = nbins - 1u;
  for (unsigned i = threadIdx.x; i < nbins; i += kThreads) sh[i] = 0;
  __syncthreads();
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads) {
    const unsigned key = cand[i];
    if ((key & mask) == prefix) atomicAdd(&sh[(key >> shift) & bin_mask], 1u);
  }
  __syncthreads();
  select_deliver_and_scan(sh, nbins, s, shift, nbits, thr_out, last, base);
}

// -------- A3 -----------------------------------------------------------------------------------
// 2^ceil(log2f(raw)) for finite raw > 0, matching glibc's log2f-then-ceil on the host.
// raw = m * 2^e with m in [1,2).  log2f returns fl32(e + log2 m), whose ceiling is e + 1 unless
// m == 1 or log2 m is so small that the sum rounds back to e -- possible only when the top 16
// mantissa bits of raw are zero.  Only then is the logarithm evaluated (in f64, rounded to f32).
__device__ __forceinline__ float pow2_ceil_log2(float raw) {
  const unsigned bits = __float_as_uint(raw);
  int e = (int)((bits >> 23) & 0xff) - 127;
  const unsigned mant = bits & 0x7fffffu;
  if (((bits >> 23) & 0xff) == 0xff) return raw;          // inf stays inf
  if (((bits >> 23) & 0xff) == 0) {                        // subnormal (unreachable: raw >= 2.2e-15)
    return exp2f(ceilf((float)log2((double)raw)));
  }
  int E;
  if (mant == 0) E = e;
  else if (mant >= 128u) E = e + 1;
  else E = (int)ceilf((float)log2((double)raw));
  return __uint_as_float((unsigned)(E + 127) << 23);       // E in [-49, 121] here
}

// inv: 1 / sc when sc is a power of two (the mxfp8 scale; multiplying by it is the same single rounding as the
// division, subnormal results included), 0 otherwise -> IEEE division
__device__ __forceinline__ float a3_elem(float v, float sc, float inv, float fmax, float step, const DivRound& dstep) {
  float scaled = keep_nan_clamp(inv != 0.0f ? __fmul_rn(v, inv) : __fdiv_rn(v, sc), -fmax, fmax);
  float q = copysignf(dstep(scaled), scaled);
  return __fmul_rn(__fmul_rn(q, step), sc);
}

__device__ __forceinline__ float a3_scale(float a, float fmax, int mxfp8) {
  const float raw = (a < 1e-12f) ? 1.0f : __fdiv_rn(a, fmax);
  return mxfp8 ? pow2_ceil_log2(raw) : raw;
}

template <int EPL, int LPG>
__global__ void __launch_bounds__(kThreads)
fakequant_fp8grid_kernel(const float* __restrict__ src, size_t n, float fmax, float step, int mxfp8,
                         float* __restrict__ out) {
  const WarpWork w = warp_work<EPL>(n);
  const DivRound dstep(step);
  // the loads of a trip are issued one trip ahead (register double buffer)
  float nf[kItems][EPL];
  int nnv[kItems];
  auto fetch = [&](size_t pr2) {
#pragma unroll
    for (int it = 0; it < kItems; ++it) nnv[it] = lane_load<CFB200_F32, EPL>(src, n, ((pr2 * kItems + it) * 32 + w.lane) * EPL, nf[it]);
  };
  if (w.warp_id < w.nslots_pairs) fetch(w.warp_id);
  for (size_t pr = w.warp_id; pr < w.nslots_pairs; pr += w.warps_total) {
    float f[kItems][EPL];
    int nv[kItems];
    size_t e0[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
      nv[it] = nnv[it];
#pragma unroll
      for (int k = 0; k < EPL; ++k) f[it][k] = nf[it][k];
    }
    if (pr + w.warps_total < w.nslots_pairs) fetch(pr + w.warps_total);
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      float m = 0.0f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) m = fmaxf(m, fabsf(f[it][k]));
      m = group_max<LPG>(m);
      const float sc = a3_scale(m, fmax, mxfp8);
      // a power-of-two scale below infinity has an exact reciprocal (its exponent stays within [-49, 121])
      const float inv = (mxfp8 && sc < __uint_as_float(0x7f800000u)) ? __fdiv_rn(1.0f, sc) : 0.0f;
      float o[EPL];
#pragma unroll
      for (int k = 0; k < EPL; ++k) o[k] = a3_elem(f[it][k], sc, inv, fmax, step, dstep);
      lane_store_f32<EPL>(out, e0[it], nv[it], o);
    }
  }
}

__global__ void fakequant_fp8grid_generic_kernel(const float* __restrict__ src, size_t n, size_t b, float fmax,
                                                 float step, int mxfp8, float* __restrict__ out) {
  const DivRound dstep(step);
  const size_t nb = (n + b - 1) / b;
  for (size_t bi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; bi < nb; bi += (size_t)gridDim.x * blockDim.x) {
    size_t lo = bi * b, hi = lo + b < n ? lo + b : n;
    float m = 0.0f;
    for (size_t i = lo; i < hi; ++i) m = fmaxf(m, fabsf(src[i]));
    const float sc = a3_scale(m, fmax, mxfp8);
    for (size_t i = lo; i < hi; ++i) out[i] = a3_elem(src[i], sc, 0.0f, fmax, step, dstep);
  }
}

// -------- A4 -----------------------------------------------------------------------------------
// snap_e2m1: nearest of {0,.5,1,1.5,2,3,4,6}, the lower level winning a tie (strict '<' in the
// reference's scan), i.e. thresholds at the exact midpoints with '<='.  NaN -> +0.
__device__ __forceinline__ float a4_elem(float v, float scale) {
  const float x = __fdiv_rn(v, scale);
  const float a = fabsf(x);
  float best = 6.0f;
  best = a <= 5.0f ? 4.0f : best;
  best = a <= 3.5f ? 3.0f : best;
  best = a <= 2.5f ? 2.0f : best;
  best = a <= 1.75f ? 1.5f : best;
  best = a <= 1.25f ? 1.0f : best;
  best = a <= 0.75f ? 0.5f : best;
  best = a <= 0.25f ? 0.0f : best;
  best = (a != a) ? 0.0f : best;
  const float sign = (x < 0.0f) ? -1.0f : 1.0f;
  return __fmul_rn(__fmul_rn(sign, best), scale);
}

template <int EPL, int LPG>
__global__ void __launch_bounds__(kThreads)
fakequant_e2m1_kernel(const float* __restrict__ src, size_t n, float* __restrict__ out) {
  const WarpWork w = warp_work<EPL>(n);
  // the loads of a trip are issued one trip ahead (register double buffer)
  float nf[kItems][EPL];
  int nnv[kItems];
  auto fetch = [&](size_t pr2) {
#pragma unroll
    for (int it = 0; it < kItems; ++it) nnv[it] = lane_load<CFB200_F32, EPL>(src, n, ((pr2 * kItems + it) * 32 + w.lane) * EPL, nf[it]);
  };
  if (w.warp_id < w.nslots_pairs) fetch(w.warp_id);
  for (size_t pr = w.warp_id; pr < w.nslots_pairs; pr += w.warps_total) {
    float f[kItems][EPL];
    int nv[kItems];
    size_t e0[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
      nv[it] = nnv[it];
#pragma unroll
      for (int k = 0; k < EPL; ++k) f[it][k] = nf[it][k];
    }
    if (pr + w.warps_total < w.nslots_pairs) fetch(pr + w.warps_total);
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      float m = 0.0f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) m = fmaxf(m, fabsf(f[it][k]));
      m = group_max<LPG>(m);
      const float sc = (m > 1e-8f) ? __fdiv_rn(m, 6.0f) : 1.0f;
      float o[EPL];
#pragma unroll
      for (int k = 0; k < EPL; ++k) o[k] = a4_elem(f[it][k], sc);
      lane_store_f32<EPL>(out, e0[it], nv[it], o);
    }
  }
}

__global__ void fakequant_e2m1_generic_kernel(const float* __restrict__ src, size_t n, size_t b,
                                              float* __restrict__ out) {
  const size_t nb = (n + b - 1) / b;
  for (size_t bi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; bi < nb; bi += (size_t)gridDim.x * blockDim.x) {
    size_t lo = bi * b, hi = lo + b < n ? lo + b : n;
    float m = 0.0f;
    for (size_t i = lo; i < hi; ++i) m = fmaxf(m, fabsf(src[i]));
    const float sc = (m > 1e-8f) ? __fdiv_rn(m, 6.0f) : 1.0f;
    for (size_t i = lo; i < hi; ++i) out[i] = a4_elem(src[i], sc);
  }
}

// -------- E2 -----------------------------------------------------------------------------------
// truncating f32 -> f16 of the reference (tensor_store.rs:85-101), then 0/inf/NaN -> 1.0
__device__ __forceinline__ unsigned f16_trunc_scale_bits(float v) {
  const unsigned bits = __float_as_uint(v);
  const unsigned sign = (bits >> 16) & 0x8000u;
  const int exp = (int)((bits >> 23) & 0xffu);
  const unsigned mant = bits & 0x7fffffu;
  unsigned h;
  if (exp == 255) h = sign | 0x7c00u | (mant ? 0x0200u : 0u);
  else {
    const int ne = exp - 127 + 15;
    if (ne >= 31) h = sign | 0x7c00u;
    else if (ne <= 0) h = sign;
    else h = sign | ((unsigned)ne << 10) | (mant >> 13);
  }
  if ((h & 0x7fffu) == 0 || (h & 0x7c00u) == 0x7c00u) h = 0x3c00u;
  return h;
}

// WIDE: the source is 32-byte aligned, so a lane's 32 bytes come in one 256-bit load (else two 128-bit loads)
template <int DT, int EPL, int LPG, bool WIDE>
__global__ void __launch_bounds__(kThreads)
quant_int4_asym_kernel(const void* __restrict__ src, size_t n, uint8_t* __restrict__ codes,
                       uint16_t* __restrict__ scales, uint8_t* __restrict__ zps) {
  constexpr size_t G = (size_t)EPL * LPG;
  const WarpWork w = warp_work<EPL>(n);
  const size_t ngroups = (n + G - 1) / G;
  // ---- fast path: slot pairs that lie completely inside the tensor (EPL == 8 only) ----
  size_t first_generic = 0;
  if constexpr (EPL == 8 || (EPL == 16 && DT != CFB200_F32)) {
    constexpr bool kF32 = (DT == CFB200_F32);
    constexpr int NW = kF32 ? 8 : EPL / 2;  // 32-bit words per lane
    const size_t full_pairs = n / ((size_t)kItems * 32 * EPL);
    first_generic = full_pairs;
    // the loads of a trip are issued one trip ahead (register double buffer)
    uint32_t nxt[kItems][NW];
    auto prefetch = [&](size_t pr2) {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        const size_t e = ((pr2 * kItems + it) * 32 + w.lane) * EPL;
        const char* p = reinterpret_cast<const char*>(src) + e * Elem<DT>::kBytes;
        if constexpr (NW == 8) {
          const Raw32 r = WIDE ? ld_stream32(p) : ld_stream32_any(p);
#pragma unroll
          for (int k = 0; k < 8; ++k) nxt[it][k] = r.w[k];
        } else {
          const uint4 r = ld_stream16(p);
          nxt[it][0] = r.x; nxt[it][1] = r.y; nxt[it][2] = r.z; nxt[it][3] = r.w;
        }
      }
    };
    if (w.warp_id < full_pairs) prefetch(w.warp_id);
    for (size_t pr = w.warp_id; pr < full_pairs; pr += w.warps_total) {
      uint32_t raw[kItems][NW];
      size_t e0[kItems];
      int zp[kItems];
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
#pragma unroll
        for (int k = 0; k < NW; ++k) raw[it][k] = nxt[it][k];
      }
      if (pr + w.warps_total < full_pairs) prefetch(pr + w.warps_total);  // the next trip's loads fly under this trip's math
      // ---- ranges of the trip's kItems groups ----
      float glo[kItems], ghi[kItems];
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        float lo = 0.0f, hi = 0.0f;  // the range always contains 0
        if constexpr (kF32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) { lo = fminf(lo, __uint_as_float(raw[it][k])); hi = fmaxf(hi, __uint_as_float(raw[it][k])); }
        } else {
          // two elements per instruction on the packed 16-bit values (a NaN operand is ignored, as fminf / fmaxf do);
          // widening the two winners is exact
          typedef typename Vec16<DT>::Pair2 P2;
          P2 lo2 = Vec16<DT>::zero2(), hi2 = lo2;
#pragma unroll
          for (int k = 0; k < NW; ++k) {
            const P2 v2 = *reinterpret_cast<const P2*>(&raw[it][k]);
            lo2 = __hmin2(lo2, v2);
            hi2 = __hmax2(hi2, v2);
          }
          lo = fminf(Vec16<DT>::low_f32(lo2), Vec16<DT>::high_f32(lo2));
          hi = fmaxf(Vec16<DT>::low_f32(hi2), Vec16<DT>::high_f32(hi2));
        }
        glo[it] = group_min<LPG>(lo);
        ghi[it] = group_max<LPG>(hi);
      }
      // ---- scale, its reciprocal and the zero point: ONE pass of the scalar arithmetic (three IEEE divisions, the f16
      // truncation, the rounding) serves all kItems groups, lane j of a group working for item j mod kItems ----
      static_assert((kItems & (kItems - 1)) == 0 && kItems <= LPG, "items per trip: a power of two, at most the lanes of a group");
      const int mine = w.lane & (kItems - 1);
      float mlo = glo[0], mhi = ghi[0];
#pragma unroll
      for (int it = 1; it < kItems; ++it) {
        mlo = (mine == it) ? glo[it] : mlo;
        mhi = (mine == it) ? ghi[it] : mhi;
      }
      const unsigned my_sh = f16_trunc_scale_bits(__fdiv_rn(__fsub_rn(mhi, mlo), 15.0f));
      const float my_s = __half2float(__ushort_as_half((unsigned short)my_sh));
      const float my_inv = __fdiv_rn(1.0f, my_s);
      const float my_zf = keep_nan_clamp(roundf(__fdiv_rn(-mlo, my_s)), 0.0f, 15.0f);
      const int my_zp = clamp_to_int(my_zf, 0.0f, 15.0f);
      const int gbase = w.lane & ~(LPG - 1);
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        float f[EPL];
        if constexpr (kF32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(raw[it][k]);
        } else {
#pragma unroll
          for (int v = 0; v < EPL / 8; ++v) {
            float t[8];
            Vec16<DT>::unpack(make_uint4(raw[it][4 * v], raw[it][4 * v + 1], raw[it][4 * v + 2], raw[it][4 * v + 3]), t);
#pragma unroll
            for (int k = 0; k < 8; ++k) f[8 * v + k] = t[k];
          }
        }
        const float s = __shfl_sync(kFullMask, my_s, gbase + it);
        const float inv = __shfl_sync(kFullMask, my_inv, gbase + it);
        const float zf = __shfl_sync(kFullMask, my_zf, gbase + it);
        zp[it] = __shfl_sync(kFullMask, my_zp, gbase + it);
        // q = clamp(round(v/s) + zp, 0, 15) = round(clamp(v/s, -zp, 15-zp)) + zp: the bounds are
        // integers and rounding is monotone.  fmaxf first: a NaN quotient becomes -zp -> code 0,
        // which is what `NaN as u8` gives in the reference formula.
        const float dlo = -zf, dhi = 15.0f - zf;
        float dc[EPL], a[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) {
          dc[k] = fminf(fmaxf(quotient<kF32>(f[k], s, inv), dlo), dhi);
          a[k] = round_mag_fixed(dc[k]);
        }
        // signs are taken from the clamped quotient (a NaN became -zp, a clamp to 0 keeps any sign)
        const uint32_t zz = (uint32_t)zp[it] * 0x01010101u;
        uint32_t nib[EPL / 8];  // eight codes per word, low nibble first
#pragma unroll
        for (int h = 0; h < EPL / 8; ++h) {
          const int b = 8 * h;
          const uint32_t m0 = sign_mask_32(__float_as_uint(dc[b]), __float_as_uint(dc[b + 1]), __float_as_uint(dc[b + 2]), __float_as_uint(dc[b + 3]));
          const uint32_t m1 = sign_mask_32(__float_as_uint(dc[b + 4]), __float_as_uint(dc[b + 5]), __float_as_uint(dc[b + 6]), __float_as_uint(dc[b + 7]));
          const uint32_t s0 = negate_bytes(pack_mag4(a[b], a[b + 1], a[b + 2], a[b + 3]), m0);
          const uint32_t s1 = negate_bytes(pack_mag4(a[b + 4], a[b + 5], a[b + 6], a[b + 7]), m1);
          const uint32_t c0 = ((s0 & 0x7f7f7f7fu) + zz) ^ (s0 & 0x80808080u);  // per-byte add, codes 0..15
          const uint32_t c1 = ((s1 & 0x7f7f7f7fu) + zz) ^ (s1 & 0x80808080u);
          const uint32_t t0 = c0 | (c0 >> 4), t1 = c1 | (c1 >> 4);           // bytes 0 and 2 hold nibble pairs
          nib[h] = __byte_perm(t0, t1, 0x6420);
        }
        if constexpr (EPL == 16) st_stream8(codes + (e0[it] >> 1), make_uint2(nib[0], nib[1]));
        else st_stream4(codes + (e0[it] >> 1), nib[0]);
        if ((w.lane % LPG) == it) scales[e0[it] / G] = (uint16_t)my_sh;  // the lane that worked for this item holds its scale
      }
      if constexpr (LPG == 32) {
        const size_t g0 = e0[0] / G;
        if (w.lane == 0) zps[g0 >> 1] = (uint8_t)(zp[0] | (zp[1] << 4));
      } else {
#pragma unroll
        for (int it = 0; it < kItems; ++it) {
          const int partner = __shfl_down_sync(kFullMask, zp[it], LPG);
          const size_t g = e0[it] / G;
          if ((w.lane % (2 * LPG)) == 0) zps[g >> 1] = (uint8_t)(zp[it] | (partner << 4));
        }
      }
    }
  }
  // ---- generic path: the last, partially filled slot pair (or every pair when EPL != 8) ----
  for (size_t pr = first_generic + w.warp_id; pr < w.nslots_pairs; pr += w.warps_total) {
    float f[kItems][EPL];
    int nv[kItems];
    size_t e0[kItems];
    int zp[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
      nv[it] = lane_load<DT, EPL>(src, n, e0[it], f[it]);
    }
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      float lo = 0.0f, hi = 0.0f;  // the range always contains 0; padded lanes hold 0
#pragma unroll
      for (int k = 0; k < EPL; ++k) { lo = fminf(lo, f[it][k]); hi = fmaxf(hi, f[it][k]); }
      lo = group_min<LPG>(lo);
      hi = group_max<LPG>(hi);
      const unsigned sh = f16_trunc_scale_bits(__fdiv_rn(__fsub_rn(hi, lo), 15.0f));
      const float s = __half2float(__ushort_as_half((unsigned short)sh));
      const float zf = keep_nan_clamp(roundf(__fdiv_rn(-lo, s)), 0.0f, 15.0f);
      zp[it] = clamp_to_int(zf, 0.0f, 15.0f);
      const DivRound dr(s);
      int c[EPL];
#pragma unroll
      for (int k = 0; k < EPL; ++k) c[k] = clamp_to_int(__fadd_rn(dr(f[it][k]), zf), 0.0f, 15.0f);
      lane_store_nibbles<EPL>(codes, e0[it], nv[it], c);
      const size_t g = e0[it] / G;
      if ((w.lane % LPG) == 0 && g < ngroups) scales[g] = (uint16_t)sh;
    }
    // zero points: two groups per byte, even group in the low nibble
    if constexpr (LPG == 32) {
      const size_t g0 = e0[0] / G;  // even, because kItems == 2 slots start at an even slot index
      if (w.lane == 0 && g0 < ngroups) zps[g0 >> 1] = (uint8_t)(zp[0] | ((g0 + 1 < ngroups ? zp[1] : 0) << 4));
    } else {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        const int partner = __shfl_down_sync(kFullMask, zp[it], LPG);
        const size_t g = e0[it] / G;
        if ((w.lane % (2 * LPG)) == 0 && g < ngroups) zps[g >> 1] = (uint8_t)(zp[it] | ((g + 1 < ngroups ? partner : 0) << 4));
      }
    }
  }
}

// -------- E3 -----------------------------------------------------------------------------------
// Code lookup.  code(x) = #{j : x > mid_j}.  The 15 midpoints are more than 1/15.5 apart, so a
// cell index c = floor(fma(x, 15.5, 15.75)) in [0,31] contains at most one midpoint; the table
// holds for each cell the number of midpoints in lower cells and the midpoint to compare with
// (the next one at or above the cell; +inf when none is left).  fma and floor are monotone, so
// the result equals the 15-comparison count for every x in [-1-2^-20, 1+2^-20]; NaN -> cell 0,
// comparison false -> code 0.
struct Nf4Cell { float thr; int base; };
__constant__ Nf4Cell c_nf4_cells[32];

void build_nf4_cells(Nf4Cell* cells) {
  static const float mids[15] = CF_NF4_MIDPOINTS_INIT;
  int cell_of[15];
  for (int j = 0; j < 15; ++j) cell_of[j] = (int)floorf(fmaf(mids[j], 15.5f, 15.75f));
  for (int c = 0; c < 32; ++c) {
    int base = 0;
    while (base < 15 && cell_of[base] < c) ++base;
    cells[c].base = base;
    cells[c].thr = base < 15 ? mids[base] : INFINITY;
  }
}

template <int DT, int EPL, int LPG, bool WIDE>
__device__ __forceinline__ void quant_nf4_body(const void* __restrict__ src, size_t n, uint8_t* __restrict__ codes, float* __restrict__ block_absmax) {
  constexpr size_t G = (size_t)EPL * LPG;
  __shared__ Nf4Cell s_cells[32], s_rev[32];  // s_rev: the table back to front, for the fast path's index
  if (threadIdx.x < 32) {
    s_cells[threadIdx.x] = c_nf4_cells[threadIdx.x];
    s_rev[31 - threadIdx.x] = c_nf4_cells[threadIdx.x];
  }
  __syncthreads();
  const WarpWork w = warp_work<EPL>(n);
  const size_t nblocks = (n + G - 1) / G;
  // ---- fast path: slot pairs that lie completely inside the tensor (EPL == 8 only) ----
  size_t first_generic = 0;
  if constexpr (EPL == 8 || (EPL == 16 && DT != CFB200_F32)) {
    constexpr bool kF32 = (DT == CFB200_F32);
    constexpr int NW = kF32 ? 8 : EPL / 2;
    using H2 = typename std::conditional<DT == CFB200_BF16, __nv_bfloat162, __half2>::type;
    const size_t full_pairs = n / ((size_t)kItems * 32 * EPL);
    first_generic = full_pairs;
    // the loads of a trip are issued one trip ahead (register double buffer)
    uint32_t nxt[kItems][NW];
    auto prefetch = [&](size_t pr2) {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        const size_t e = ((pr2 * kItems + it) * 32 + w.lane) * EPL;
        const char* p = reinterpret_cast<const char*>(src) + e * Elem<DT>::kBytes;
        if constexpr (NW == 8) {
          const Raw32 r = WIDE ? ld_stream32(p) : ld_stream32_any(p);
#pragma unroll
          for (int k = 0; k < 8; ++k) nxt[it][k] = r.w[k];
        } else {
          const uint4 r = ld_stream16(p);
          nxt[it][0] = r.x; nxt[it][1] = r.y; nxt[it][2] = r.z; nxt[it][3] = r.w;
        }
      }
    };
    if (w.warp_id < full_pairs) prefetch(w.warp_id);
    for (size_t pr = w.warp_id; pr < full_pairs; pr += w.warps_total) {
      uint32_t raw[kItems][NW];
      size_t e0[kItems];
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
#pragma unroll
        for (int k = 0; k < NW; ++k) raw[it][k] = nxt[it][k];
      }
      if (pr + w.warps_total < full_pairs) prefetch(pr + w.warps_total);  // the next trip's loads fly under this trip's math
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        float f[EPL];
        float m = 0.0f;
        if constexpr (kF32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) { f[k] = __uint_as_float(raw[it][k]); m = fmaxf(m, fabsf(f[k])); }
        } else {
#pragma unroll
          for (int v = 0; v < EPL / 8; ++v) {
            float t[8];
            Vec16<DT>::unpack(make_uint4(raw[it][4 * v], raw[it][4 * v + 1], raw[it][4 * v + 2], raw[it][4 * v + 3]), t);
#pragma unroll
            for (int k = 0; k < 8; ++k) f[8 * v + k] = t[k];
          }
          H2 hm;
          *reinterpret_cast<uint32_t*>(&hm) = 0u;
#pragma unroll
          for (int k = 0; k < NW; ++k) hm = __hmax2(hm, __habs2(*reinterpret_cast<const H2*>(&raw[it][k])));
          const uint32_t bits = *reinterpret_cast<uint32_t*>(&hm);
          if constexpr (DT == CFB200_BF16) m = fmaxf(__uint_as_float(bits << 16), __uint_as_float(bits & 0xffff0000u));
          else { const float2 t2 = __half22float2(*reinterpret_cast<const __half2*>(&bits)); m = fmaxf(t2.x, t2.y); }
        }
        m = group_max<LPG>(m);
        const float inv = (m == 0.0f) ? 0.0f : __fdiv_rn(1.0f, m);
        uint32_t words[EPL / 8];
#pragma unroll
        for (int h = 0; h < EPL / 8; ++h) {
          uint32_t word = 0;
#pragma unroll
          for (int k = 7; k >= 0; --k) {
            const float x = __fmul_rn(f[8 * h + k], inv);
            // Cell index without a float -> int conversion: fma.ru(x, -62, 64 + 2^23) = 2^23 + ceil(4 (31 - e)) + 3 with
            // e = 15.5 x + 15.75 exact, so bits [2, 7) of the result are 31 - floor(e), the index into the reversed table
            // (checked on the host against the 15-comparison definition for every f32 in [-1 - 2^-22, 1 + 2^-22]).
            // A NaN has all of those bits set -> reversed entry 31 = cell 0, compares false -> code 0.
            const uint32_t tb = __float_as_uint(__fmaf_ru(x, -62.0f, 8388672.0f));
            const Nf4Cell e = s_rev[(tb >> 2) & 31u];
            word = word * 16u + (uint32_t)(e.base + (x > e.thr ? 1 : 0));
          }
          words[h] = word;
        }
        if constexpr (EPL == 16) st_stream8(codes + (e0[it] >> 1), make_uint2(words[0], words[1]));
        else st_stream4(codes + (e0[it] >> 1), words[0]);
        if ((w.lane % LPG) == 0) block_absmax[e0[it] / G] = m;
      }
    }
  }
  // ---- generic path: the last, partially filled slot pair (or every pair when EPL != 8) ----
  for (size_t pr = first_generic + w.warp_id; pr < w.nslots_pairs; pr += w.warps_total) {
    float f[kItems][EPL];
    int nv[kItems];
    size_t e0[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      e0[it] = ((pr * kItems + it) * 32 + w.lane) * EPL;
      nv[it] = lane_load<DT, EPL>(src, n, e0[it], f[it]);
    }
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      float m = 0.0f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) m = fmaxf(m, fabsf(f[it][k]));
      m = group_max<LPG>(m);
      const float inv = (m == 0.0f) ? 0.0f : __fdiv_rn(1.0f, m);
      int c[EPL];
#pragma unroll
      for (int k = 0; k < EPL; ++k) {
        const float x = __fmul_rn(f[it][k], inv);
        int cell = __float2int_rd(__fmaf_rn(x, 15.5f, 15.75f));
        cell = min(max(cell, 0), 31);  // only +-inf-free garbage can leave the range
        const Nf4Cell e = s_cells[cell];
        c[k] = e.base + (x > e.thr ? 1 : 0);
      }
      lane_store_nibbles<EPL>(codes, e0[it], nv[it], c);
      const size_t b = e0[it] / G;
      if ((w.lane % LPG) == 0 && b < nblocks) block_absmax[b] = m;
    }
  }
}

// second level: absmax8 = clamp(round(a / s2), 0, 255), s2 = max(a)/255 per dq_block blocks
template <int DT, int EPL, int LPG, bool WIDE>
__global__ void __launch_bounds__(kThreads)
quant_nf4_kernel(const void* __restrict__ src, size_t n, uint8_t* __restrict__ codes, float* __restrict__ block_absmax) {
  quant_nf4_body<DT, EPL, LPG, WIDE>(src, n, codes, block_absmax);
}

// One tensor of a list per blockIdx.y: the whole list in one launch, CTAs of the next tensor start as those of the
// previous one finish.
struct Nf4Seg {
  const void* src;
  size_t n;
  uint8_t* codes;
  float* block_absmax;  // inside the workspace
  uint8_t* absmax8;
  float* absmax2;
  unsigned grid_x;      // CTAs this tensor has work for
  unsigned pad;
};
template <int DT, int EPL, int LPG, bool WIDE>
__global__ void __launch_bounds__(kThreads) quant_nf4_list_kernel(const Nf4Seg* __restrict__ segs) {
  const Nf4Seg sg = segs[blockIdx.y];
  if (blockIdx.x >= sg.grid_x) return;
  quant_nf4_body<DT, EPL, LPG, WIDE>(sg.src, sg.n, sg.codes, sg.block_absmax);
}

__device__ __forceinline__ void nf4_double_quant_body(const float* __restrict__ block_absmax, size_t nblocks, size_t dq_block,
                                                      uint8_t* __restrict__ absmax8, float* __restrict__ absmax2, unsigned stride) {
  __shared__ float s_part[kThreads / 32];
  __shared__ float s_max;
  const size_t nsb = (nblocks + dq_block - 1) / dq_block;
  for (size_t sb = blockIdx.x; sb < nsb; sb += stride) {
    const size_t b0 = sb * dq_block, b1 = b0 + dq_block < nblocks ? b0 + dq_block : nblocks;
    float m = 0.0f;
    for (size_t i = b0 + threadIdx.x; i < b1; i += kThreads) m = fmaxf(m, block_absmax[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      float v = 0.0f;
      for (int i = 0; i < kThreads / 32; ++i) v = fmaxf(v, s_part[i]);
      s_max = v;
    }
    __syncthreads();
    const float mx = s_max;
    const float s2 = (mx == 0.0f || mx != mx || isinf(mx)) ? 1.0f : __fdiv_rn(mx, 255.0f);
    if (threadIdx.x == 0) absmax2[sb] = s2;
    for (size_t i = b0 + threadIdx.x; i < b1; i += kThreads) {
      const float r = keep_nan_clamp(roundf(__fdiv_rn(block_absmax[i], s2)), 0.0f, 255.0f);
      absmax8[i] = (r != r) ? 0 : (uint8_t)__float2int_rz(r);
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
nf4_double_quant_kernel(const float* __restrict__ block_absmax, size_t nblocks, size_t dq_block,
                        uint8_t* __restrict__ absmax8, float* __restrict__ absmax2) {
  nf4_double_quant_body(block_absmax, nblocks, dq_block, absmax8, absmax2, gridDim.x);
}
__global__ void __launch_bounds__(kThreads) nf4_double_quant_list_kernel(const Nf4Seg* __restrict__ segs, size_t block, size_t dq_block) {
  const Nf4Seg sg = segs[blockIdx.y];
  const size_t nblocks = (sg.n + block - 1) / block;
  if ((size_t)blockIdx.x * dq_block >= nblocks) return;  // uniform over the CTA: no super-block for it
  nf4_double_quant_body(sg.block_absmax, nblocks, dq_block, sg.absmax8, sg.absmax2, gridDim.x);
}

// -------- launch helpers -------------------------------------------------------------------------
int persistent_grid(size_t nwarp_trips) {
  size_t blocks = (nwarp_trips + (kThreads / 32) - 1) / (kThreads / 32);
  size_t cap = (size_t)sm_count() * 8;
  size_t g = blocks < cap ? blocks : cap;
  return (int)(g < 1 ? 1 : g);
}
template <int EPL>
int grid_for(size_t n) {
  size_t slot = 32 * (size_t)EPL, nslots = (n + slot - 1) / slot;
  return persistent_grid((nslots + kItems - 1) / kItems);
}
int generic_grid(size_t ngroups) {
  size_t blocks = (ngroups + 127) / 128, cap = (size_t)sm_count() * 16;
  size_t g = blocks < cap ? blocks : cap;
  return (int)(g < 1 ? 1 : g);
}

void bounds_of(int32_t bits, float* qmin, float* qmax) {
  if (bits == 4) { *qmin = -8.0f; *qmax = 7.0f; }
  else { *qmin = -128.0f; *qmax = 127.0f; }
}

// f32 sources: G -> (EPL, LPG).  Returns false when G has no lane decomposition.
#define CFB_DISPATCH_F32_GROUP(G, LAUNCH)                \
  switch (G) {                                           \
    case 4: LAUNCH(4, 1); break;                         \
    case 8: LAUNCH(4, 2); break;                         \
    case 16: LAUNCH(4, 4); break;                        \
    case 32: LAUNCH(4, 8); break;                        \
    case 64: LAUNCH(4, 16); break;                       \
    case 128: LAUNCH(4, 32); break;                      \
    case 256: LAUNCH(8, 32); break;                      \
    default: handled = false; break;                     \
  }

}  // namespace
}  // namespace cfb

using namespace cfb;

namespace cfb {
size_t select_fast_workspace_bytes(size_t n) {
  const size_t cand = n / 64 > (size_t)(1u << 18) ? n / 64 : (size_t)(1u << 18);
  return ((sizeof(SelectFast) + 255) & ~(size_t)255) + cand * sizeof(unsigned) + 256;
}

// k-th largest |v| (1 <= k <= n) into thr_out; `state` keeps the rank inside the elements equal to it and their count
int32_t select_kth_abs_rank(const float* src, size_t n, unsigned long long k, float* thr_out, SelectState* state, cudaStream_t st,
                            const float* sub, float* diff_out, void* fast_ws, size_t fast_bytes) {
  size_t blocks = (n / 4 + kThreads - 1) / kThreads, cap = (size_t)sm_count() * 8;
  int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
  // the 31 magnitude bits in three passes: 11 + 10 + 10
  static const int kShift[3] = {20, 10, 0}, kBits[3] = {11, 10, 10};
  const int* skip = nullptr;
  const float* pass_src = src;
  const float* pass_sub = sub;
  // single-pass path: large tensors, ranks in the top 5 %, enough workspace
  // (a CTA of the bracket pass stages its candidates in shared memory: about 0.5 % of its share of the tensor must fit)
  const bool fast = fast_ws && n >= ((size_t)1 << 20) && k * 20 <= n && fast_bytes >= select_fast_workspace_bytes(n) &&
                    n / (size_t)grid / 200 <= (size_t)kFastStage / 4 && (reinterpret_cast<uintptr_t>(fast_ws) & 255) == 0;
  if (fast) CFB_CUDA(cudaMemsetAsync(state, 0, sizeof(SelectState), st));
  else select_init_kernel<<<1, 256, 0, st>>>(state, k);
  if (fast) {
    SelectFast* f = reinterpret_cast<SelectFast*>(fast_ws);
    unsigned* cand = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(fast_ws) + ((sizeof(SelectFast) + 255) & ~(size_t)255));
    const size_t cand_cap = n / 64 > (size_t)(1u << 18) ? n / 64 : (size_t)(1u << 18);
    CFB_CUDA(cudaMemsetAsync(f, 0, sizeof(SelectFast), st));
    const size_t samples = kSampleCount < n / 4 ? kSampleCount : n / 4;
    select_sample_kernel<<<256, kThreads, 0, st>>>(src, sub, n, samples, k, f, state);
    select_bracket_kernel<<<grid, kThreads, 0, st>>>(src, sub, diff_out, n, k, f, cand, (unsigned long long)cand_cap, state);
    select_hist_cand_kernel<<<32, kThreads, 0, st>>>(cand, f, 10, 11, state, thr_out, 0);
    select_hist_cand_kernel<<<32, kThreads, 0, st>>>(cand, f, 0, 10, state, thr_out, 1);
    skip = &f->fast_ok;  // the full passes below only run if the bracket did not hold
    if (sub) { pass_src = diff_out; pass_sub = nullptr; }  // the bracket pass has written the differences already
  }
  for (int pass = 0; pass < 3; ++pass) {
    if (pass == 0 || pass_sub == nullptr)
      select_hist_kernel<<<grid, kThreads, 0, st>>>(pass_src, pass == 0 ? pass_sub : nullptr, diff_out, n, kShift[pass], kBits[pass], state,
                                                     thr_out, pass == 2, skip);
    else
      select_hist_kernel<<<grid, kThreads, 0, st>>>(diff_out, nullptr, nullptr, n, kShift[pass], kBits[pass], state, thr_out, pass == 2, skip);
  }
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}
}  // namespace cfb

extern "C" size_t cfb200_select_kth_workspace_bytes(void) { return sizeof(SelectState); }
extern "C" size_t cfb200_select_kth_workspace_bytes_for(size_t n) {
  return ((sizeof(SelectState) + 255) & ~(size_t)255) + select_fast_workspace_bytes(n);
}

extern "C" int32_t cfb200_select_kth_abs(const float* src, size_t n, float salient_ratio, float* thr_out,
                                         uint64_t* k_host, void* workspace, size_t workspace_bytes, void* stream) {
  CFB_CHECK_ARG(thr_out != nullptr, "thr_out is NULL");
  CFB_CHECK_ARG(n == 0 || src, "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(workspace, 8);
  if (workspace == nullptr || workspace_bytes < sizeof(SelectState))
    return set_error(CFB200_ERR_WORKSPACE, "select_kth needs %zu bytes of workspace", sizeof(SelectState));
  cudaStream_t st = (cudaStream_t)stream;
  // schemes.rs:487, :524-526: ratio clamped, k = ceil((float)n * ratio) in f32, then [1, n]
  float ratio = salient_ratio < 0.001f ? 0.001f : (salient_ratio > 0.5f ? 0.5f : salient_ratio);
  if (salient_ratio != salient_ratio) ratio = salient_ratio;
  size_t k = (size_t)ceilf((float)n * ratio);
  if (k < 1) k = 1;
  if (k > n) k = n;
  if (k_host) *k_host = k;
  if (n == 0) {
    CFB_CUDA(cudaMemsetAsync(thr_out, 0, sizeof(float), st));
    return CFB200_OK;
  }
  // a workspace of cfb200_select_kth_workspace_bytes_for(n) bytes enables the single-pass path
  const size_t head = (sizeof(SelectState) + 255) & ~(size_t)255;
  void* fast = nullptr;
  size_t fast_bytes = 0;
  if (workspace_bytes >= cfb200_select_kth_workspace_bytes_for(n) && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0) {
    fast = reinterpret_cast<char*>(workspace) + head;
    fast_bytes = workspace_bytes - head;
  }
  return select_kth_abs_rank(src, n, (unsigned long long)k, thr_out, reinterpret_cast<SelectState*>(workspace), st, nullptr, nullptr, fast,
                             fast_bytes);
}

extern "C" int32_t cfb200_fakequant_group(const float* src, size_t n, int32_t bits, size_t group_size,
                                          int32_t awq_salient, const float* thr, float* out, void* stream) {
  CFB_CHECK_ARG(n == 0 || (src && out), "NULL buffer");
  CFB_CHECK_ARG(!awq_salient || thr, "thr is NULL with awq_salient set");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(out, 16);
  if (n == 0) return CFB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  float qmin, qmax;
  bounds_of(bits, &qmin, &qmax);
  const size_t g = group_size < 2 ? 2 : group_size;  // schemes.rs:486
  bool handled = true;
#define LAUNCH(EPL, LPG) \
  fakequant_group_kernel<EPL, LPG><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, qmin, qmax, awq_salient, thr, out)
  CFB_DISPATCH_F32_GROUP(g, LAUNCH)
#undef LAUNCH
  if (!handled)
    fakequant_group_generic_kernel<<<generic_grid((n + g - 1) / g), 128, 0, st>>>(src, n, g, qmin, qmax, awq_salient, thr, out);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

extern "C" int32_t cfb200_fakequant_fp8grid(const float* src, size_t n, size_t block_size, int32_t e5m2,
                                            int32_t mxfp8, float* out, void* stream) {
  CFB_CHECK_ARG(n == 0 || (src && out), "NULL buffer");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(out, 16);
  if (n == 0) return CFB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const float fmax = e5m2 ? 57344.0f : 448.0f;
  const float grid_steps = e5m2 ? 15.0f : 31.0f;
  float step = fmax / grid_steps;  // IEEE division on the host, as in schemes.rs:711
  if (step < 1e-6f) step = 1e-6f;
  const size_t b = block_size < 4 ? 4 : block_size;  // schemes.rs:664
  bool handled = true;
#define LAUNCH(EPL, LPG) \
  fakequant_fp8grid_kernel<EPL, LPG><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, fmax, step, mxfp8, out)
  CFB_DISPATCH_F32_GROUP(b, LAUNCH)
#undef LAUNCH
  if (!handled)
    fakequant_fp8grid_generic_kernel<<<generic_grid((n + b - 1) / b), 128, 0, st>>>(src, n, b, fmax, step, mxfp8, out);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

extern "C" int32_t cfb200_fakequant_e2m1(const float* src, size_t n, size_t block, float* out, void* stream) {
  CFB_CHECK_ARG(n == 0 || (src && out), "NULL buffer");
  CFB_CHECK_ARG(block >= 1, "block must be >= 1");
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(out, 16);
  if (n == 0) return CFB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  bool handled = true;
#define LAUNCH(EPL, LPG) fakequant_e2m1_kernel<EPL, LPG><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, out)
  CFB_DISPATCH_F32_GROUP(block, LAUNCH)
#undef LAUNCH
  if (!handled) fakequant_e2m1_generic_kernel<<<generic_grid((n + block - 1) / block), 128, 0, st>>>(src, n, block, out);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

extern "C" int32_t cfb200_quant_int4_asym(const void* src, int32_t src_dtype, size_t n, size_t group,
                                          uint8_t* codes, uint16_t* scales, uint8_t* zero_points, void* stream) {
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ARG(n == 0 || (src && codes && scales && zero_points), "NULL buffer");
  CFB_CHECK_ARG(group == 32 || group == 64 || group == 128 || group == 256, "group must be 32, 64, 128 or 256 (got %zu)", group);
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 16);
  CFB_CHECK_ALIGNED(scales, 2);
  if (n == 0) return CFB200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool wide = (reinterpret_cast<uintptr_t>(src) & 31) == 0;
#define LAUNCH(DT, EPL, LPG)                                                                                              \
  do {                                                                                                                    \
    if (wide) quant_int4_asym_kernel<DT, EPL, LPG, true><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, codes, scales, zero_points);  \
    else quant_int4_asym_kernel<DT, EPL, LPG, false><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, codes, scales, zero_points);      \
  } while (0)
  if (src_dtype == CFB200_F32) {
    switch (group) {
      case 32: LAUNCH(CFB200_F32, 8, 4); break;
      case 64: LAUNCH(CFB200_F32, 8, 8); break;
      case 128: LAUNCH(CFB200_F32, 8, 16); break;
      default: LAUNCH(CFB200_F32, 8, 32); break;
    }
  } else if (src_dtype == CFB200_BF16) {
    switch (group) {
      case 32: LAUNCH(CFB200_BF16, 8, 4); break;
      case 64: LAUNCH(CFB200_BF16, 16, 4); break;   // 16 elements (32 bytes) per lane: the per-group arithmetic is paid by half as many lanes
      case 128: LAUNCH(CFB200_BF16, 16, 8); break;
      default: LAUNCH(CFB200_BF16, 16, 16); break;
    }
  } else {
    switch (group) {
      case 32: LAUNCH(CFB200_F16, 8, 4); break;
      case 64: LAUNCH(CFB200_F16, 16, 4); break;   // 16 elements (32 bytes) per lane: the per-group arithmetic is paid by half as many lanes
      case 128: LAUNCH(CFB200_F16, 16, 8); break;
      default: LAUNCH(CFB200_F16, 16, 16); break;
    }
  }
#undef LAUNCH
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// The NF4 code table goes to constant memory once per device (not per host thread), on the first NF4 call there.
static int32_t nf4_upload_cells(int dev, cudaStream_t st) {
  static std::mutex cells_mutex;
  static bool cells_ready[64];
  std::lock_guard<std::mutex> lock(cells_mutex);
  if (!cells_ready[dev]) {
    Nf4Cell cells[32];
    build_nf4_cells(cells);
    CFB_CUDA(cudaMemcpyToSymbolAsync(c_nf4_cells, cells, sizeof cells, 0, cudaMemcpyHostToDevice, st));
    CFB_CUDA(cudaStreamSynchronize(st));  // `cells` lives on this stack frame
    cells_ready[dev] = true;
  }
  return CFB200_OK;
}

extern "C" size_t cfb200_quant_nf4_workspace_bytes(size_t n, size_t block) {
  if (block == 0) return 0;
  return ((n + block - 1) / block) * sizeof(float);
}

extern "C" int32_t cfb200_quant_nf4(const void* src, int32_t src_dtype, size_t n, size_t block, size_t dq_block,
                                    uint8_t* codes, uint8_t* absmax8, float* absmax2, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ARG(n == 0 || (src && codes && absmax8 && absmax2), "NULL buffer");
  CFB_CHECK_ARG(block == 32 || block == 64 || block == 128 || block == 256, "block must be 32, 64, 128 or 256 (got %zu)", block);
  CFB_CHECK_ARG(dq_block >= 1 && dq_block <= 1024, "dq_block must be in [1, 1024] (got %zu)", dq_block);
  CFB_CHECK_ALIGNED(src, 16);
  CFB_CHECK_ALIGNED(codes, 16);
  CFB_CHECK_ALIGNED(workspace, 4);
  if (n == 0) return CFB200_OK;
  if (workspace == nullptr || workspace_bytes < cfb200_quant_nf4_workspace_bytes(n, block))
    return set_error(CFB200_ERR_WORKSPACE, "quant_nf4 needs %zu bytes of workspace, got %zu",
                     cfb200_quant_nf4_workspace_bytes(n, block), workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CFB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  {
    const int32_t rc_cells = nf4_upload_cells(dev, st);
    if (rc_cells) return rc_cells;
  }
  float* am = reinterpret_cast<float*>(workspace);
  const bool wide = (reinterpret_cast<uintptr_t>(src) & 31) == 0;
#define LAUNCH(DT, EPL, LPG)                                                                             \
  do {                                                                                                   \
    if (wide) quant_nf4_kernel<DT, EPL, LPG, true><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, codes, am);  \
    else quant_nf4_kernel<DT, EPL, LPG, false><<<grid_for<EPL>(n), kThreads, 0, st>>>(src, n, codes, am);      \
  } while (0)
  if (src_dtype == CFB200_F32) {
    switch (block) {
      case 32: LAUNCH(CFB200_F32, 8, 4); break;
      case 64: LAUNCH(CFB200_F32, 8, 8); break;
      case 128: LAUNCH(CFB200_F32, 8, 16); break;
      default: LAUNCH(CFB200_F32, 8, 32); break;
    }
  } else if (src_dtype == CFB200_BF16) {
    switch (block) {
      case 32: LAUNCH(CFB200_BF16, 8, 4); break;
      case 64: LAUNCH(CFB200_BF16, 16, 4); break;   // 16 elements (32 bytes) per lane: twice the bytes in flight per warp
      case 128: LAUNCH(CFB200_BF16, 16, 8); break;
      default: LAUNCH(CFB200_BF16, 16, 16); break;
    }
  } else {
    switch (block) {
      case 32: LAUNCH(CFB200_F16, 8, 4); break;
      case 64: LAUNCH(CFB200_F16, 16, 4); break;   // 16 elements (32 bytes) per lane: twice the bytes in flight per warp
      case 128: LAUNCH(CFB200_F16, 16, 8); break;
      default: LAUNCH(CFB200_F16, 16, 16); break;
    }
  }
#undef LAUNCH
  CFB_LAUNCH_CHECK();
  const size_t nblocks = (n + block - 1) / block, nsb = (nblocks + dq_block - 1) / dq_block;
  size_t cap = (size_t)sm_count() * 8;
  nf4_double_quant_kernel<<<(int)(nsb < cap ? nsb : cap), kThreads, 0, st>>>(am, nblocks, dq_block, absmax8, absmax2);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// A whole list of tensors in two launches (codes + block maxima, then the double quantisation): blockIdx.y picks
// the tensor.  workspace = descriptor table (count entries, 256-byte aligned) + the f32 block maxima of every tensor.
namespace {
inline size_t nf4_align256(size_t x) { return (x + 255) & ~(size_t)255; }
}
extern "C" size_t cfb200_quant_nf4_tensors_workspace_bytes(int32_t count, const size_t* ns, size_t block) {
  if (count <= 0 || !ns || block == 0) return 0;
  size_t total = nf4_align256((size_t)count * sizeof(Nf4Seg));
  for (int i = 0; i < count; ++i) total += nf4_align256(((ns[i] + block - 1) / block) * sizeof(float));
  return total;
}

extern "C" int32_t cfb200_quant_nf4_tensors(int32_t count, const void* const* srcs, int32_t src_dtype, const size_t* ns, size_t block,
                                            size_t dq_block, uint8_t* const* codes, uint8_t* const* absmax8, float* const* absmax2,
                                            void* workspace, size_t workspace_bytes, void* stream) {
  CFB_CHECK_ARG(count >= 0, "negative count");
  if (count == 0) return CFB200_OK;
  CFB_CHECK_ARG(count <= 65535, "at most 65535 tensors per call (got %d)", count);
  CFB_CHECK_ARG(srcs && ns && codes && absmax8 && absmax2, "NULL argument");
  CFB_CHECK_ARG(dtype_ok(src_dtype), "unknown src_dtype %d", src_dtype);
  CFB_CHECK_ARG(block == 32 || block == 64 || block == 128 || block == 256, "block must be 32, 64, 128 or 256 (got %zu)", block);
  CFB_CHECK_ARG(dq_block >= 1 && dq_block <= 1024, "dq_block must be in [1, 1024] (got %zu)", dq_block);
  CFB_CHECK_ALIGNED(workspace, 256);
  const size_t need = cfb200_quant_nf4_tensors_workspace_bytes(count, ns, block);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(CFB200_ERR_WORKSPACE, "quant_nf4_tensors needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CFB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::vector<Nf4Seg> table((size_t)count);
  char* ws = reinterpret_cast<char*>(workspace);
  size_t off = nf4_align256((size_t)count * sizeof(Nf4Seg));
  bool wide = true;
  size_t max_n = 0, max_nsb = 0;
  for (int i = 0; i < count; ++i) {
    CFB_CHECK_ARG(ns[i] == 0 || (srcs[i] && codes[i] && absmax8[i] && absmax2[i]), "tensor %d: NULL buffer", i);
    CFB_CHECK_ALIGNED(srcs[i], 16);
    CFB_CHECK_ALIGNED(codes[i], 16);
    wide = wide && (reinterpret_cast<uintptr_t>(srcs[i]) & 31) == 0;
    const size_t nb = (ns[i] + block - 1) / block;
    table[i] = Nf4Seg{srcs[i], ns[i], codes[i], reinterpret_cast<float*>(ws + off), absmax8[i], absmax2[i], 0u, 0u};
    off += nf4_align256(nb * sizeof(float));
    max_n = ns[i] > max_n ? ns[i] : max_n;
    const size_t nsb = (nb + dq_block - 1) / dq_block;
    max_nsb = nsb > max_nsb ? nsb : max_nsb;
  }
  if (max_n == 0) return CFB200_OK;
  int32_t rc = nf4_upload_cells(dev, st);
  if (rc) return rc;
  unsigned gx = 1;
#define LAUNCH(DT, EPL, LPG)                                                                                    \
  do {                                                                                                          \
    gx = (unsigned)grid_for<EPL>(max_n);                                                                        \
    for (int i = 0; i < count; ++i) table[i].grid_x = ns[i] ? (unsigned)grid_for<EPL>(ns[i]) : 0u;              \
    CFB_CUDA(cudaMemcpyAsync(ws, table.data(), (size_t)count * sizeof(Nf4Seg), cudaMemcpyHostToDevice, st));    \
    const dim3 grid(gx, (unsigned)count);                                                                       \
    if (wide) quant_nf4_list_kernel<DT, EPL, LPG, true><<<grid, kThreads, 0, st>>>(reinterpret_cast<const Nf4Seg*>(ws));  \
    else quant_nf4_list_kernel<DT, EPL, LPG, false><<<grid, kThreads, 0, st>>>(reinterpret_cast<const Nf4Seg*>(ws));     \
  } while (0)
  if (src_dtype == CFB200_F32) {
    switch (block) {
      case 32: LAUNCH(CFB200_F32, 8, 4); break;
      case 64: LAUNCH(CFB200_F32, 8, 8); break;
      case 128: LAUNCH(CFB200_F32, 8, 16); break;
      default: LAUNCH(CFB200_F32, 8, 32); break;
    }
  } else if (src_dtype == CFB200_BF16) {
    switch (block) {
      case 32: LAUNCH(CFB200_BF16, 8, 4); break;
      case 64: LAUNCH(CFB200_BF16, 16, 4); break;
      case 128: LAUNCH(CFB200_BF16, 16, 8); break;
      default: LAUNCH(CFB200_BF16, 16, 16); break;
    }
  } else {
    switch (block) {
      case 32: LAUNCH(CFB200_F16, 8, 4); break;
      case 64: LAUNCH(CFB200_F16, 16, 4); break;
      case 128: LAUNCH(CFB200_F16, 16, 8); break;
      default: LAUNCH(CFB200_F16, 16, 16); break;
    }
  }
#undef LAUNCH
  CFB_LAUNCH_CHECK();
  const size_t cap = (size_t)sm_count() * 8;
  const dim3 g2((unsigned)(max_nsb < cap ? max_nsb : cap), (unsigned)count);
  nf4_double_quant_list_kernel<<<g2, kThreads, 0, st>>>(reinterpret_cast<const Nf4Seg*>(ws), block, dq_block);
  CFB_LAUNCH_CHECK();
  return CFB200_OK;
}

// ---------------------------------------------------------------------------------------------
// NF4 without any allocation by anybody: the block-absmax scratch lives in a file-scope device
// array that every device loading this library carries until the process exits.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kNf4StaticMaxBlocks = (size_t)1 << 20;  // 4 MiB of f32 block maxima
static __device__ __align__(256) float g_nf4_static_scratch[kNf4StaticMaxBlocks];
// In host code the array's name is only a handle for the runtime, not a device address; the
// address each device gives it is looked up once per device and kept here.
float* g_nf4_static_ptr[64];
std::mutex g_nf4_static_mutex;
}  // namespace

extern "C" size_t cfb200_quant_nf4_static_max_elements(size_t block) { return kNf4StaticMaxBlocks * block; }

extern "C" int32_t cfb200_quant_nf4_static(const void* src, int32_t src_dtype, size_t n, size_t block, size_t dq_block,
                                           uint8_t* codes, uint8_t* absmax8, float* absmax2, void* stream) {
  CFB_CHECK_ARG(block == 32 || block == 64 || block == 128 || block == 256, "block must be 32, 64, 128 or 256 (got %zu)", block);
  const size_t nblocks = n / block + (n % block != 0);  // no wrap-around for n near SIZE_MAX
  if (nblocks > kNf4StaticMaxBlocks)
    return set_error(CFB200_ERR_INVALID,
                     "cfb200_quant_nf4_static handles at most %zu elements at block %zu (%zu blocks of built-in scratch); got %zu "
                     "elements -- split the tensor or use cfb200_quant_nf4 with a caller workspace",
                     kNf4StaticMaxBlocks * block, block, kNf4StaticMaxBlocks, n);
  int dev = 0;
  CFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CFB200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  float* scratch;
  {
    std::lock_guard<std::mutex> lock(g_nf4_static_mutex);
    if (g_nf4_static_ptr[dev] == nullptr) {  // first call on this device, with this device current
      float* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_nf4_static_scratch);
      if (e != cudaSuccess || p == nullptr)
        return set_error(CFB200_ERR_CUDA, "cudaGetSymbolAddress(nf4 static scratch) failed: %s", cudaGetErrorString(e));
      g_nf4_static_ptr[dev] = p;
    }
    scratch = g_nf4_static_ptr[dev];
  }
  // Every block slot in [0, nblocks) is overwritten before it is read, so nothing needs clearing.
  return cfb200_quant_nf4(src, src_dtype, n, block, dq_block, codes, absmax8, absmax2, scratch,
                          kNf4StaticMaxBlocks * sizeof(float), stream);
}
