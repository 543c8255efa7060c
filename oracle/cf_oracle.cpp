// CPU oracle for the CastForge quantize-and-execute hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, loop for loop, the arithmetic of the
// reference's CPU passes and interpreter so that the CUDA path can be checked bit for bit.
// Only the test-suite, the smoke check and the benchmark's CPU-baseline legs may load it; the
// product library never links or calls it.
//
// Parity status.  The reference is Rust and cannot be compiled in this environment, and its own
// tests hold no golden codes or scales for this path, so rows A1-A10 are pinned by code reading
// plus the small fixtures the reference's tests use (re-derived by hand in tests/golden).
// The extension schemes (per-channel INT8, asymmetric INT4 packing, NF4, true E4M3 casts, GPTQ)
// have no reference arithmetic at all: for those this file *is* the specification and their
// parity is "unpinned".
//
// Every function cites the reference file:line it follows (paths relative to the reference
// project root).  All arithmetic is IEEE binary32 unless stated.  Compile WITHOUT -ffast-math and
// with -ffp-contract=off so that no multiply-add is fused (Rust never contracts).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "nf4_codebook.inc"

namespace {

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// Rust `f32::max` / `f32::min` (LLVM maxnum/minnum as lowered on x86): a NaN operand, quiet OR
// signalling, is dropped.  glibc's fmaxf returns NaN for a signalling NaN, so it is not used.
inline float rmax(float a, float b) { return (b != b) ? a : ((a != a) ? b : (a > b ? a : b)); }
inline float rmin(float a, float b) { return (b != b) ? a : ((a != a) ? b : (a < b ? a : b)); }

// Rust `f32::clamp(lo, hi)`: NaN stays NaN.
inline float rclamp(float x, float lo, float hi) {
  if (x < lo) return lo;
  if (x > hi) return hi;
  return x;
}

// Rust `as i8` from f32: saturating, NaN -> 0.
inline int8_t f32_as_i8(float x) {
  if (x != x) return 0;
  if (x <= -128.0f) return -128;
  if (x >= 127.0f) return 127;
  return (int8_t)x;  // truncation toward zero
}

inline int set_threads(int threads) {
#ifdef _OPENMP
  int t = threads <= 0 ? omp_get_max_threads() : threads;
  return t < 1 ? 1 : t;
#else
  (void)threads;
  return 1;
#endif
}

// `fold(0.0, |acc, v| acc.max(v.abs()))` -- formats.rs:672, schemes.rs:533.
// max is associative and commutative on non-NaN values and NaN operands are dropped, so a
// parallel reduction yields the same bits as the sequential fold.
float amax(const float* v, size_t n, int threads) {
  float m = 0.0f;
  if (threads > 1 && n > (1u << 16)) {
#ifdef _OPENMP
#pragma omp parallel for reduction(max : m) num_threads(threads) schedule(static)
#endif
    for (long long i = 0; i < (long long)n; ++i) {
      float a = std::fabs(v[i]);
      if (a > m) m = a;  // NaN compares false: ignored, as in Rust
    }
    return m;
  }
  for (size_t i = 0; i < n; ++i) m = rmax(m, std::fabs(v[i]));
  return m;
}

// symmetric_int_quant_bounds -- formats.rs:654-660.  Any bit count other than 4 means 8.
inline void bounds(int bits, int* eff, float* qmin, float* qmax) {
  if (bits == 4) { *eff = 4; *qmin = -8.0f; *qmax = 7.0f; }
  else { *eff = 8; *qmin = -128.0f; *qmax = 127.0f; }
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------------
// A10: dtype conversions -- src/ir/tensor_store.rs:58-111
// ---------------------------------------------------------------------------------------------

float cfo_f16_bits_to_f32(uint16_t bits) {  // tensor_store.rs:58-82
  uint32_t sign = (bits >> 15) & 1u, exp = (bits >> 10) & 0x1fu, mant = bits & 0x03ffu, out;
  if (exp == 0) {
    if (mant == 0) out = sign << 31;
    else {
      uint32_t m = mant, e = 127 - 14;
      while ((m & 0x0400u) == 0) { m <<= 1; e -= 1; }
      m &= 0x03ffu;
      out = (sign << 31) | (e << 23) | (m << 13);
    }
  } else if (exp == 0x1f) out = (sign << 31) | 0x7f800000u | (mant << 13);
  else out = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
  return u2f(out);
}

uint16_t cfo_f32_to_f16_bits(float val) {  // tensor_store.rs:85-101 (truncating, FTZ)
  uint32_t bits = f2u(val);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  int32_t exp = (int32_t)((bits >> 23) & 0xffu);
  uint32_t mant = bits & 0x007fffffu;
  if (exp == 255) return sign | 0x7c00u | (mant != 0 ? 0x0200u : 0u);
  int32_t ne = exp - 127 + 15;
  if (ne >= 31) return sign | 0x7c00u;
  if (ne <= 0) return sign;
  return sign | (uint16_t)(ne << 10) | (uint16_t)(mant >> 13);
}

float cfo_bf16_bits_to_f32(uint16_t bits) { return u2f((uint32_t)bits << 16); }  // :104-106
uint16_t cfo_f32_to_bf16_bits(float v) { return (uint16_t)(f2u(v) >> 16); }      // :109-111

// resolve_f32_attr's widening of F16/BF16 backings -- tensor_store.rs:314-348.
// dtype: 0 = f32, 1 = f16, 2 = bf16.
void cfo_to_f32(const void* src, int dtype, size_t n, float* out, int threads) {
  int t = set_threads(threads);
  (void)t;
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long i = 0; i < (long long)n; ++i) {
    if (dtype == 0) out[i] = ((const float*)src)[i];
    else if (dtype == 1) out[i] = cfo_f16_bits_to_f32(((const uint16_t*)src)[i]);
    else out[i] = cfo_bf16_bits_to_f32(((const uint16_t*)src)[i]);
  }
}

// ---------------------------------------------------------------------------------------------
// A1: per-tensor symmetric quantization -- src/passes/quantize/formats.rs:664-698
// ---------------------------------------------------------------------------------------------

// The `{:.6}` scale string with trailing zeros (then a trailing '.') trimmed and ".0" appended
// when no '.' is left -- formats.rs:680-688.  `out` needs >= 64 bytes.
void cfo_format_scale(float scale, char* out) {
  char buf[96];
  std::snprintf(buf, sizeof buf, "%.6f", (double)scale);
  std::string s(buf);
  while (!s.empty() && s.back() == '0') s.pop_back();
  while (!s.empty() && s.back() == '.') s.pop_back();
  if (s.find('.') == std::string::npos) s += ".0";
  std::snprintf(out, 64, "%s", s.c_str());
}

// `scale.parse::<f32>().unwrap_or(1.0)` -- src/codegen/eval.rs:312, :331-334.
float cfo_parse_scale(const char* s) {
  char* end = nullptr;
  float v = std::strtof(s, &end);
  if (end == s || *end != '\0') return 1.0f;
  return v;
}

// quantize_symmetric_f32.  One code per int8 byte for 4 bits too; zero point is always 0.
void cfo_quant_sym(const float* v, size_t n, int bits, int8_t* q, float* scale_out,
                   char* scale_str /* >= 64 bytes, may be NULL */, int threads) {
  int eff; float qmin, qmax;
  bounds(bits, &eff, &qmin, &qmax);
  int t = set_threads(threads);
  float m = amax(v, n, t);
  float scale = (m < 1e-12f) ? 1.0f : m / qmax;
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long i = 0; i < (long long)n; ++i)
    q[i] = f32_as_i8(rclamp(std::round(v[i] / scale), qmin, qmax));
  *scale_out = scale;
  if (scale_str) cfo_format_scale(scale, scale_str);
}

// run_qat_ste's per-tensor fake quantization -- formats.rs:764-769 (f32 tensors only).
void cfo_fakequant_tensor(const float* v, size_t n, int bits, float* out, float* scale_out,
                          int threads) {
  int eff; float qmin, qmax;
  bounds(bits, &eff, &qmin, &qmax);
  int t = set_threads(threads);
  float m = amax(v, n, t);
  float scale = (m < 1e-12f) ? 1.0f : m / qmax;
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long i = 0; i < (long long)n; ++i)
    out[i] = rclamp(std::round(v[i] / scale), qmin, qmax) * scale;
  *scale_out = scale;
}

// run_smoothquant's per-constant arithmetic -- schemes.rs:229-243.  For a constant the
// "activation range" is the constant's own absmax folded in f64 from 1e-5
// (formats.rs:136-153), cast to f32.  Returns smooth_scale and eff_qscale through `params`.
void cfo_smoothquant(const float* v, size_t n, int bits, float alpha, float* out,
                     float* params /* [2] */, int threads) {
  int eff; float qmin, qmax;
  bounds(bits, &eff, &qmin, &qmax);
  int t = set_threads(threads);
  alpha = rclamp(alpha, 0.05f, 0.95f);
  double peak = 1e-5;
  for (size_t i = 0; i < n; ++i) { double a = std::fabs((double)v[i]); if (a > peak) peak = a; }
  float act_max = (float)peak;
  float w_max = rmax(amax(v, n, t), 1e-5f);
  float smooth = rmax(std::pow(rmax(act_max, 1e-4f), alpha) / std::pow(w_max, 1.0f - alpha), 1e-4f);
  float effq = rmax(w_max * smooth / qmax, 1e-6f);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long i = 0; i < (long long)n; ++i) {
    float migrated = v[i] * smooth;
    float qq = rclamp(std::round(migrated / effq), qmin, qmax);
    out[i] = (qq * effq) / smooth;
  }
  params[0] = smooth;
  params[1] = effq;
}

// ---------------------------------------------------------------------------------------------
// A2: group-wise fake quantization with the AWQ salient threshold -- schemes.rs:483-570
// ---------------------------------------------------------------------------------------------

// IEEE total order on |v| (non-negative sign bit): plain unsigned compare of the bit pattern;
// NaN sorts above +inf, as `total_cmp` does (schemes.rs:523).
static inline uint32_t abs_key(float v) { return f2u(v) & 0x7fffffffu; }

// faithful != 0: full descending sort as the reference does (used when timing the baseline);
// faithful == 0: nth_element, same k-th value.
void cfo_salient_threshold(const float* v, size_t n, float salient_ratio, int faithful,
                           float* thr_out, uint64_t* k_out) {
  float ratio = rclamp(salient_ratio, 0.001f, 0.5f);
  size_t k = (size_t)std::ceil((float)n * ratio);  // schemes.rs:524-526
  k = std::min(std::max(k, (size_t)1), n);
  std::vector<uint32_t> keys(n);
  for (size_t i = 0; i < n; ++i) keys[i] = abs_key(v[i]);
  if (faithful) std::sort(keys.begin(), keys.end(), std::greater<uint32_t>());
  else std::nth_element(keys.begin(), keys.begin() + (k - 1), keys.end(), std::greater<uint32_t>());
  *thr_out = n ? u2f(keys[k - 1]) : 0.0f;
  *k_out = k;
}

void cfo_fakequant_group(const float* v, size_t n, int bits, size_t group_size,
                         float salient_ratio, int awq_salient, int faithful, float* out,
                         float* thr_out, uint64_t* k_out, int threads) {
  int eff; float qmin, qmax;
  bounds(bits, &eff, &qmin, &qmax);
  size_t g = std::max(group_size, (size_t)2);
  float thr; uint64_t k;
  cfo_salient_threshold(v, n, salient_ratio, faithful, &thr, &k);
  int t = set_threads(threads);
  long long ngroups = (long long)((n + g - 1) / g);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long gi = 0; gi < ngroups; ++gi) {
    size_t lo = (size_t)gi * g, hi = std::min(n, lo + g);
    float gm = 0.0f;
    for (size_t i = lo; i < hi; ++i) gm = rmax(gm, std::fabs(v[i]));
    float scale = (gm < 1e-12f) ? 1.0f : gm / qmax;
    for (size_t i = lo; i < hi; ++i) {
      float e = (awq_salient && std::fabs(v[i]) >= thr) ? scale * 0.5f : scale;
      float qq = rclamp(std::round(v[i] / e), qmin, qmax);
      out[i] = qq * e;
    }
  }
  if (thr_out) *thr_out = thr;
  if (k_out) *k_out = k;
}

// ---------------------------------------------------------------------------------------------
// A3: FP8 "grid" fake quantization -- schemes.rs:658-716
// ---------------------------------------------------------------------------------------------
void cfo_fakequant_fp8grid(const float* v, size_t n, size_t block_size, int e5m2, int mxfp8,
                           float* out, int threads) {
  float fp8_max = e5m2 ? 57344.0f : 448.0f;
  float grid = e5m2 ? 15.0f : 31.0f;
  size_t b = std::max(block_size, (size_t)4);
  float step = rmax(fp8_max / grid, 1e-6f);
  int t = set_threads(threads);
  long long nb = (long long)((n + b - 1) / b);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long bi = 0; bi < nb; ++bi) {
    size_t lo = (size_t)bi * b, hi = std::min(n, lo + b);
    float a = 0.0f;
    for (size_t i = lo; i < hi; ++i) a = rmax(a, std::fabs(v[i]));
    float raw = (a < 1e-12f) ? 1.0f : a / fp8_max;
    float sc = mxfp8 ? std::pow(2.0f, std::ceil(std::log2(raw))) : raw;  // powf / log2f
    for (size_t i = lo; i < hi; ++i) {
      float scaled = rclamp(v[i] / sc, -fp8_max, fp8_max);
      float qq = std::round(scaled / step) * step;
      out[i] = qq * sc;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// A4: E2M1 (FP4) fake quantization -- formats.rs:369-383, :414-479
// ---------------------------------------------------------------------------------------------
static inline float snap_e2m1(float val) {
  static const float L[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float sign = (val < 0.0f) ? -1.0f : 1.0f;
  float a = std::fabs(val), best = 0.0f, best_err = std::numeric_limits<float>::max();
  for (float lvl : L) {
    float err = std::fabs(a - lvl);
    if (err < best_err) { best_err = err; best = lvl; }  // strict <: lower level wins ties
  }
  return sign * best;
}

// `blk` is the already-resolved block length (nvfp4 with 32 requested -> 16; else max(b,4)).
void cfo_fakequant_e2m1(const float* v, size_t n, size_t blk, float* out, int threads) {
  int t = set_threads(threads);
  long long nb = (long long)((n + blk - 1) / blk);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long bi = 0; bi < nb; ++bi) {
    size_t lo = (size_t)bi * blk, hi = std::min(n, lo + blk);
    float a = 0.0f;
    for (size_t i = lo; i < hi; ++i) a = rmax(a, std::fabs(v[i]));
    float scale = (a > 1e-8f) ? a / 6.0f : 1.0f;
    for (size_t i = lo; i < hi; ++i) out[i] = snap_e2m1(v[i] / scale) * scale;
  }
}

// ---------------------------------------------------------------------------------------------
// A5: blocked Hadamard rotation down the columns of a [K, N] matrix -- formats.rs:303-327
// ---------------------------------------------------------------------------------------------
// Returns the block length actually used, or 0 when K % b != 0 (data left untouched).
uint64_t cfo_fwht_cols(float* w, size_t K, size_t N, size_t block_size, int threads) {
  size_t b = 1;
  while (b < block_size) b <<= 1;  // next_power_of_two (0 and 1 -> 1)
  b = std::max(std::min(b, K), (size_t)2);
  if (K % b != 0) return 0;
  float norm = 1.0f / std::sqrt((float)b);
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long col = 0; col < (long long)N; ++col) {
    std::vector<float> buf(b);
    for (size_t kb = 0; kb < K; kb += b) {
      for (size_t i = 0; i < b; ++i) buf[i] = w[(kb + i) * N + col];
      for (size_t h = 1; h < b; h *= 2)
        for (size_t i = 0; i < b; i += h * 2)
          for (size_t j = i; j < i + h; ++j) {
            float x = buf[j], y = buf[j + h];
            buf[j] = x + y;
            buf[j + h] = x - y;
          }
      for (size_t i = 0; i < b; ++i) w[(kb + i) * N + col] = buf[i] * norm;
    }
  }
  return b;
}

// ---------------------------------------------------------------------------------------------
// A8: interpreter dequantize + GEMM -- src/codegen/eval.rs:296-347, :1145-1179, :1465-1507
// ---------------------------------------------------------------------------------------------

// `(q as i32 - zp as i32) as f32 * sc` -- eval.rs:314-317.  `sc` is the PARSED 6-decimal string.
void cfo_dequant_i8(const int8_t* q, size_t n, float sc, int64_t zp, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = (float)((int32_t)q[i] - (int32_t)zp) * sc;
}

static inline float gelu_tanh(float x) {  // eval_gelu_scalar (tanh form)
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.0f + std::tanh(c * (x + 0.044715f * x * x * x)));
}

// eval_matmul_2d: C[m,n] = sum_k A[m,k] * B, k ascending, separate multiply and add.
// B is [K,N] row-major, or [N,K] when packed_rhs.  Optional fused_qmatmul epilogue
// (eval.rs:1151-1176): 0 none, 1 bias, 2 bias_relu, 3 bias_tanh, 4 bias_silu, 5 bias_gelu,
// 6 bias_scale; `bias` and `z` are indexed modulo their lengths.
void cfo_matmul_2d(const float* A, const float* B, size_t M, size_t N, size_t K, int packed_rhs,
                   int epilogue, const float* bias, size_t bias_len, const float* z,
                   size_t z_len, float* C, int threads) {
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) collapse(2) if (t > 1)
#endif
  for (long long row = 0; row < (long long)M; ++row)
    for (long long col = 0; col < (long long)N; ++col) {
      float acc = 0.0f;
      for (size_t kk = 0; kk < K; ++kk) {
        float bv = packed_rhs ? B[(size_t)col * K + kk] : B[kk * N + (size_t)col];
        acc += A[(size_t)row * K + kk] * bv;
      }
      if (epilogue != 0) {
        size_t i = (size_t)row * N + (size_t)col;
        float val = acc + bias[i % (bias_len ? bias_len : 1)];
        float zz = z ? z[i % (z_len ? z_len : 1)] : 0.0f;
        switch (epilogue) {
          case 2: val = rmax(val, zz); break;
          case 3: val = std::tanh(val); break;
          case 4: val = val / (1.0f + std::exp(-val)); break;
          case 5: val = gelu_tanh(val); break;
          case 6: val = val * zz; break;
          default: break;
        }
        acc = val;
      }
      C[(size_t)row * N + (size_t)col] = acc;
    }
}

// castforge.static_quantize prologue -- eval.rs:1369-1382.
void cfo_static_quantize(const float* x, size_t n, float scale_attr, int bits, float* out) {
  float qmax = (bits == 4) ? 7.0f : 127.0f;
  float sc = scale_attr > 0.0f ? scale_attr : 1.0f / 127.0f;
  for (size_t i = 0; i < n; ++i) out[i] = rclamp(std::round(x[i] / sc), -qmax, qmax) * sc;
}

// ---------------------------------------------------------------------------------------------
// A9: block ops around the GEMMs -- src/codegen/eval.rs:1058-1137, :1180-1213, :1607-1668
// ---------------------------------------------------------------------------------------------

// fused_rmsnorm (res == NULL) / fused_residual_rmsnorm.  Weight indexed by flat position when it
// is long enough, else by column, else 1 (eval.rs:1081-1084).
void cfo_rmsnorm(const float* x, const float* res, const float* w, size_t w_len, size_t rows, size_t cols,
                 float eps, float* out) {
  for (size_t r = 0; r < rows; ++r) {
    float sq = 0.0f;
    for (size_t c = 0; c < cols; ++c) {
      float h = x[r * cols + c];
      if (res) h = h + res[r * cols + c];
      sq += h * h;
    }
    float inv_rms = 1.0f / std::sqrt(sq / (float)cols + eps);
    for (size_t c = 0; c < cols; ++c) {
      size_t idx = r * cols + c;
      float h = x[idx];
      if (res) h = h + res[idx];
      float wv = w ? (idx < w_len ? w[idx] : (c < w_len ? w[c] : 1.0f)) : 1.0f;
      out[idx] = h * inv_rms * wv;
    }
  }
}

void cfo_rope(const float* x, const float* cs, const float* sn, size_t rows, size_t cols, float* out) {  // :1096-1118
  size_t half = cols / 2;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      size_t idx = r * cols + c;
      float rot = c < half ? -x[r * cols + c + half] : x[r * cols + c - half];
      out[idx] = x[idx] * cs[idx] + rot * sn[idx];
    }
}

void cfo_swiglu(const float* g, const float* u, size_t n, float* out) {  // :1090-1095
  for (size_t i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + std::exp(-g[i]))) * u[i];
}

// eval_fused_attention_2d per head (k given row-major [seq_kv, d_k], i.e. k_transposed/packed),
// heads addressed by strides so a head can be a column slice of a [seq, heads*d] activation.
void cfo_attention(const float* q, const float* k, const float* v, const float* mask, int batch, int seq_q, int seq_kv,
                   int d_k, int d_v, size_t ld_q, size_t ld_k, size_t ld_v, size_t ld_o, size_t hs_q, size_t hs_k,
                   size_t hs_v, size_t hs_o, float scale, float* out) {
  std::vector<float> qk((size_t)seq_kv), probs((size_t)seq_kv);
  for (int b = 0; b < batch; ++b)
    for (int r = 0; r < seq_q; ++r) {
      for (int c = 0; c < seq_kv; ++c) {
        float acc = 0.0f;
        for (int d = 0; d < d_k; ++d) acc += q[b * hs_q + (size_t)r * ld_q + d] * k[b * hs_k + (size_t)c * ld_k + d];
        qk[c] = acc;
      }
      float mx = -std::numeric_limits<float>::infinity();
      for (int c = 0; c < seq_kv; ++c) mx = rmax(mx, qk[c] * scale + (mask ? mask[(size_t)r * seq_kv + c] : 0.0f));
      float sum = 0.0f;
      for (int c = 0; c < seq_kv; ++c) {
        float e = std::exp(qk[c] * scale + (mask ? mask[(size_t)r * seq_kv + c] : 0.0f) - mx);
        probs[c] = e;
        sum += e;
      }
      for (int d = 0; d < d_v; ++d) out[b * hs_o + (size_t)r * ld_o + d] = 0.0f;
      for (int c = 0; c < seq_kv; ++c) {
        float p = probs[c] / sum;
        for (int d = 0; d < d_v; ++d) out[b * hs_o + (size_t)r * ld_o + d] += p * v[b * hs_v + (size_t)c * ld_v + d];
      }
    }
}

// ---------------------------------------------------------------------------------------------
// E4 codec: float8_e4m3fn -- src/passes/serving/mutable_loads.rs:367-429 (the reference codec)
// ---------------------------------------------------------------------------------------------
uint8_t cfo_e4m3_encode_ref(float v) {
  if (v != v) return 0x7F;
  uint8_t sign = std::signbit(v) ? 0x80 : 0x00;
  float a = std::fabs(v);
  if (a == 0.0f) return sign;
  if (a >= 448.0f) return sign | 0x7E;
  const float min_normal = 1.0f / 64.0f;
  auto as_u8 = [](float f) -> uint8_t {  // Rust saturating `as u8`
    if (f != f || f <= 0.0f) return 0;
    if (f >= 255.0f) return 255;
    return (uint8_t)f;
  };
  if (a < min_normal) {
    float scaled = a * 512.0f, fl = std::floor(scaled), diff = scaled - fl;
    uint8_t mant = as_u8(fl);
    if (diff > 0.5f || (diff == 0.5f && (mant & 1) == 1)) mant += 1;
    return sign | mant;
  }
  int e_unb = (int)std::floor(std::log2(a));  // log2f
  uint8_t e_b = (uint8_t)(e_unb + 7);
  float norm = a / std::ldexp(1.0f, e_unb) - 1.0f;  // powi(2, e) is exact
  float sm = norm * 8.0f, fm = std::floor(sm), dm = sm - fm;
  uint8_t mant = as_u8(fm);
  if (dm > 0.5f || (dm == 0.5f && (mant & 1) == 1)) mant += 1;
  uint8_t e = e_b, m = mant;
  if (m == 8) { m = 0; e += 1; }
  if (e > 15 || (e == 15 && m >= 7)) return sign | 0x7E;
  return sign | (uint8_t)(e << 3) | m;
}

float cfo_e4m3_decode(uint8_t b) {  // mutable_loads.rs:413-429
  float sign = (b & 0x80) ? -1.0f : 1.0f;
  uint8_t exp = (b >> 3) & 0x0F, mant = b & 0x07;
  if (exp == 0x0F && mant == 0x07) return std::numeric_limits<float>::quiet_NaN();
  if (exp == 0) {
    if (mant == 0) return sign < 0.0f ? -0.0f : 0.0f;
    return sign * ((float)mant / 512.0f);
  }
  return sign * (1.0f + (float)mant / 8.0f) * std::ldexp(1.0f, (int)exp - 7);
}

// The codec's *intent* stated without libm: round-to-nearest-even onto the E4M3FN grid,
// saturating to +-448, NaN -> 0x7F.  It differs from cfo_e4m3_encode_ref only where the
// reference's `log2().floor()` lands on the wrong binade (inputs a few ulp below a power of
// two); tests enumerate that set.  This is the behaviour of the hardware conversion
// `cvt.rn.satfinite.e4m3x2.f32`, and the specification the CUDA cast kernels are held to.
uint8_t cfo_e4m3_encode_rne(float v) {
  if (v != v) return 0x7F;
  uint8_t sign = std::signbit(v) ? 0x80 : 0x00;
  float a = std::fabs(v);
  if (a >= 448.0f) return sign | 0x7E;  // satfinite (also +-inf)
  if (a == 0.0f) return sign;
  int e;
  (void)std::frexp(a, &e);  // a = f * 2^e, f in [0.5,1)
  int e_unb = e - 1;
  if (e_unb < -6) e_unb = -6;  // subnormal binade shares the step of the lowest normal binade
  float step = std::ldexp(1.0f, e_unb - 3);
  float qv = std::nearbyint(a / step);  // RNE in the default rounding mode; a/step is exact
  float r = qv * step;
  if (r > 448.0f) return sign | 0x7E;
  if (r == 0.0f) return sign;
  int e2;
  (void)std::frexp(r, &e2);
  int eu = e2 - 1;
  if (eu < -6) return sign | (uint8_t)(r * 512.0f);
  uint8_t m = (uint8_t)((r / std::ldexp(1.0f, eu) - 1.0f) * 8.0f);
  return sign | (uint8_t)((eu + 7) << 3) | m;
}

// ---------------------------------------------------------------------------------------------
// Extension schemes.  No reference arithmetic exists for these; the conventions are inherited
// from the reference where it has one (A1's absmax/round/clamp formula, the truncating f16
// conversion of tensor_store.rs:85-101, low-nibble-first packing of gguf.rs:520-531).
// ---------------------------------------------------------------------------------------------

// E1: per-output-channel symmetric INT8/INT4.  A1's formula applied to each row of a
// [rows, cols] row-major matrix.
void cfo_quant_per_channel(const float* v, size_t rows, size_t cols, int bits, int8_t* q,
                           float* scales, int threads) {
  int eff; float qmin, qmax;
  bounds(bits, &eff, &qmin, &qmax);
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long r = 0; r < (long long)rows; ++r) {
    const float* row = v + (size_t)r * cols;
    float m = 0.0f;
    for (size_t c = 0; c < cols; ++c) m = rmax(m, std::fabs(row[c]));
    float scale = (m < 1e-12f) ? 1.0f : m / qmax;
    for (size_t c = 0; c < cols; ++c)
      q[(size_t)r * cols + c] = f32_as_i8(rclamp(std::round(row[c] / scale), qmin, qmax));
    scales[r] = scale;
  }
}

// E2: asymmetric INT4 over flat groups of `group` elements (group even).
//   lo = min(0, min v), hi = max(0, max v)            (NaN ignored)
//   s32 = (hi - lo) / 15;  sh = truncating f16 of s32;  if sh encodes 0 -> sh = f16(1.0)
//   s = f32(sh);  zp = clamp(round(-lo / s), 0, 15);  q = clamp(round(v / s) + zp, 0, 15)
// codes: two per byte, element 2j in the low nibble; zero points: two groups per byte, group
// 2j in the low nibble; scales: one f16 bit pattern per group.
void cfo_quant_int4_asym(const float* v, size_t n, size_t group, uint8_t* codes,
                         uint16_t* scales, uint8_t* zps, int threads) {
  int t = set_threads(threads);
  long long ng = (long long)((n + group - 1) / group);
  std::vector<uint8_t> zp_full((size_t)ng);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long gi = 0; gi < ng; ++gi) {
    size_t b0 = (size_t)gi * group, b1 = std::min(n, b0 + group);
    float lo = 0.0f, hi = 0.0f;
    for (size_t i = b0; i < b1; ++i) { lo = rmin(lo, v[i]); hi = rmax(hi, v[i]); }
    float s32 = (hi - lo) / 15.0f;
    uint16_t sh = cfo_f32_to_f16_bits(s32);
    if ((sh & 0x7fffu) == 0 || (sh & 0x7c00u) == 0x7c00u) sh = 0x3c00u;  // zero/inf/NaN -> 1.0
    float s = cfo_f16_bits_to_f32(sh);
    float zf = rclamp(std::round(-lo / s), 0.0f, 15.0f);
    uint8_t zp = (uint8_t)f32_as_i8(zf);
    scales[gi] = sh;
    zp_full[(size_t)gi] = zp;
    for (size_t i = b0; i < b1; ++i) {
      float qf = rclamp(std::round(v[i] / s) + zf, 0.0f, 15.0f);
      uint8_t c = (uint8_t)f32_as_i8(qf);
      // group is even, so a byte never straddles two groups (no write race)
      if ((i & 1) == 0) codes[i >> 1] = (uint8_t)((codes[i >> 1] & 0xF0) | c);
      else codes[i >> 1] = (uint8_t)((codes[i >> 1] & 0x0F) | (c << 4));
    }
  }
  for (long long gi = 0; gi < ng; gi += 2) {
    uint8_t b = zp_full[(size_t)gi];
    if (gi + 1 < ng) b |= (uint8_t)(zp_full[(size_t)gi + 1] << 4);
    zps[gi >> 1] = b;
  }
}

// Dequantize E2 output: w = (q - zp) * s  (f32).
void cfo_dequant_int4_asym(const uint8_t* codes, const uint16_t* scales, const uint8_t* zps,
                           size_t n, size_t group, float* out) {
  for (size_t i = 0; i < n; ++i) {
    size_t g = i / group;
    int q = (codes[i >> 1] >> ((i & 1) * 4)) & 0xF;
    int zp = (zps[g >> 1] >> ((g & 1) * 4)) & 0xF;
    out[i] = (float)(q - zp) * cfo_f16_bits_to_f32(scales[g]);
  }
}

static const float kNf4Levels[16] = CF_NF4_LEVELS_INIT;
static const float kNf4Mid[15] = CF_NF4_MIDPOINTS_INIT;

// E3: NF4 over flat blocks of `block` elements (block even) with the block absmax values
// double-quantized to 8 bits in super-blocks of `dq_block` absmax values.
//   a = amax(block); inv = (a == 0) ? 0 : 1.0f / a; x = v * inv
//   code = number of midpoints m_j with x > m_j   (the lower level wins an exact tie)
//   absmax8[b] = clamp(round(a / s2), 0, 255) with s2 = max(a over the super-block) / 255
//   (s2 == 0 -> s2 = 1).  absmax2[sb] = s2 (f32).
// A NaN input compares false against every midpoint and gets code 0.
void cfo_quant_nf4(const float* v, size_t n, size_t block, size_t dq_block, uint8_t* codes,
                   uint8_t* absmax8, float* absmax2, int threads) {
  int t = set_threads(threads);
  long long nb = (long long)((n + block - 1) / block);
  std::vector<float> am((size_t)nb);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long bi = 0; bi < nb; ++bi) {
    size_t b0 = (size_t)bi * block, b1 = std::min(n, b0 + block);
    float a = 0.0f;
    for (size_t i = b0; i < b1; ++i) a = rmax(a, std::fabs(v[i]));
    am[(size_t)bi] = a;
    float inv = (a == 0.0f) ? 0.0f : 1.0f / a;
    for (size_t i = b0; i < b1; ++i) {
      float x = v[i] * inv;
      uint8_t c = 0;
      for (int j = 0; j < 15; ++j) c += (x > kNf4Mid[j]) ? 1 : 0;
      if ((i & 1) == 0) codes[i >> 1] = (uint8_t)((codes[i >> 1] & 0xF0) | c);
      else codes[i >> 1] = (uint8_t)((codes[i >> 1] & 0x0F) | (c << 4));
    }
  }
  long long nsb = (nb + (long long)dq_block - 1) / (long long)dq_block;
  for (long long sb = 0; sb < nsb; ++sb) {
    size_t b0 = (size_t)sb * dq_block, b1 = std::min((size_t)nb, b0 + dq_block);
    float mx = 0.0f;
    for (size_t i = b0; i < b1; ++i) mx = rmax(mx, am[i]);
    float s2 = (mx == 0.0f || mx != mx || std::isinf(mx)) ? 1.0f : mx / 255.0f;
    absmax2[sb] = s2;
    for (size_t i = b0; i < b1; ++i) {
      float r = rclamp(std::round(am[i] / s2), 0.0f, 255.0f);
      absmax8[i] = (r != r) ? 0 : (uint8_t)r;
    }
  }
}

void cfo_dequant_nf4(const uint8_t* codes, const uint8_t* absmax8, const float* absmax2,
                     size_t n, size_t block, size_t dq_block, float* out) {
  for (size_t i = 0; i < n; ++i) {
    size_t b = i / block;
    float a = (float)absmax8[b] * absmax2[b / dq_block];
    int c = (codes[i >> 1] >> ((i & 1) * 4)) & 0xF;
    out[i] = kNf4Levels[c] * a;
  }
}

void cfo_nf4_levels(float* out16) { std::memcpy(out16, kNf4Levels, sizeof kNf4Levels); }

// E4 casts.  Per-tensor weight scale: s = amax/448 (amax < 1e-12 -> 1), code = e4m3_rne(v * (1/s)).
// Per-token (row) activation scale: the same formula per row of [rows, cols].
void cfo_cast_e4m3_rows(const float* v, size_t rows, size_t cols, uint8_t* codes, float* scales,
                        int threads) {
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long r = 0; r < (long long)rows; ++r) {
    const float* row = v + (size_t)r * cols;
    float a = 0.0f;
    for (size_t c = 0; c < cols; ++c) a = rmax(a, std::fabs(row[c]));
    float s = (a < 1e-12f) ? 1.0f : a / 448.0f;
    scales[r] = s;
    float inv = 1.0f / s;
    for (size_t c = 0; c < cols; ++c) codes[(size_t)r * cols + c] = cfo_e4m3_encode_rne(row[c] * inv);
  }
}

// FP8 x FP8 -> f32 GEMM used to check the tensor-core kernel: C[m,n] = sa[m]*sw * sum_k a*w
// accumulated in f64 (order-independent reference), A [M,K] codes, W [N,K] codes.
void cfo_gemm_e4m3(const uint8_t* A, const float* sa, const uint8_t* W, float sw, size_t M,
                   size_t N, size_t K, float* C, int threads) {
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = cfo_e4m3_decode((uint8_t)i);
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) collapse(2) if (t > 1)
#endif
  for (long long m = 0; m < (long long)M; ++m)
    for (long long nn = 0; nn < (long long)N; ++nn) {
      double acc = 0.0;
      for (size_t k = 0; k < K; ++k)
        acc += (double)lut[A[(size_t)m * K + k]] * (double)lut[W[(size_t)nn * K + k]];
      C[(size_t)m * N + (size_t)nn] = (float)(acc * (double)sa[m] * (double)sw);
    }
}

// W4A16 reference GEMM: C[m,n] = sum_k A[m,k] * dequant(W)[n,k], f64 accumulate, A given as f32
// (already widened from bf16), W in E2 layout with groups along K.
void cfo_gemm_w4a16(const float* A, const uint8_t* codes, const uint16_t* scales,
                    const uint8_t* zps, size_t M, size_t N, size_t K, size_t group, float* C,
                    int threads) {
  std::vector<float> W(N * K);
  cfo_dequant_int4_asym(codes, scales, zps, N * K, group, W.data());
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) collapse(2) if (t > 1)
#endif
  for (long long m = 0; m < (long long)M; ++m)
    for (long long nn = 0; nn < (long long)N; ++nn) {
      double acc = 0.0;
      for (size_t k = 0; k < K; ++k) acc += (double)A[(size_t)m * K + k] * (double)W[(size_t)nn * K + k];
      C[(size_t)m * N + (size_t)nn] = (float)acc;
    }
}

// E5: GPTQ (4 bits, group `group` along K, natural column order), after the published algorithm
// (Frantar et al. 2022): H = X^T X / T; H += damp * mean(diag H) * I; U = upper Cholesky factor of
// H^-1 obtained the textbook way (invert, then factor); columns left to right, each column's error
// e = (w - q) / U[j,j] pushed into the later columns: w[l] -= e * U[j,l].  All state is f64; the
// group parameters use the f32 arithmetic of cfo_quant_int4_asym on the current values.
// Outputs in the layout of cfo_quant_int4_asym over the row-major [N,K] matrix; Wdq = (q - zp) * s.
// Returns 0, or 1 when H is not positive definite after damping.
int cfo_gptq(const float* W, const float* X, size_t N, size_t K, size_t T, size_t group, double damp,
             uint8_t* codes, uint16_t* scales, uint8_t* zps, float* Wdq, int threads) {
  std::vector<double> H(K * K, 0.0);
  int t = set_threads(threads);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long i = 0; i < (long long)K; ++i)
    for (size_t j = (size_t)i; j < K; ++j) {
      double s = 0.0;
      for (size_t r = 0; r < T; ++r) s += (double)X[r * K + (size_t)i] * (double)X[r * K + j];
      H[(size_t)i * K + j] = H[j * K + (size_t)i] = s / (double)T;
    }
  double mean = 0.0;
  for (size_t i = 0; i < K; ++i) mean += H[i * K + i];
  mean /= (double)K;
  for (size_t i = 0; i < K; ++i) {
    H[i * K + i] += damp * mean;
    if (!(H[i * K + i] > 0.0)) H[i * K + i] = 1.0;
  }
  // lower Cholesky H = L L^T (in place, lower part)
  auto chol_lower = [&](std::vector<double>& A) -> bool {
    for (size_t j = 0; j < K; ++j) {
      double d = A[j * K + j];
      for (size_t k = 0; k < j; ++k) d -= A[j * K + k] * A[j * K + k];
      if (!(d > 0.0)) return false;
      d = std::sqrt(d);
      A[j * K + j] = d;
      for (size_t i = j + 1; i < K; ++i) {
        double s = A[i * K + j];
        for (size_t k = 0; k < j; ++k) s -= A[i * K + k] * A[j * K + k];
        A[i * K + j] = s / d;
      }
    }
    for (size_t i = 0; i < K; ++i)
      for (size_t j = i + 1; j < K; ++j) A[i * K + j] = 0.0;
    return true;
  };
  if (!chol_lower(H)) return 1;
  // Linv by forward substitution, then Hinv = Linv^T Linv
  std::vector<double> Li(K * K, 0.0);
  for (size_t c = 0; c < K; ++c)
    for (size_t i = c; i < K; ++i) {
      double s = (i == c) ? 1.0 : 0.0;
      for (size_t j = c; j < i; ++j) s -= H[i * K + j] * Li[j * K + c];
      Li[i * K + c] = s / H[i * K + i];
    }
  std::vector<double> Hinv(K * K, 0.0);
  for (size_t i = 0; i < K; ++i)
    for (size_t j = i; j < K; ++j) {
      double s = 0.0;
      for (size_t k = j; k < K; ++k) s += Li[k * K + i] * Li[k * K + j];
      Hinv[i * K + j] = Hinv[j * K + i] = s;
    }
  if (!chol_lower(Hinv)) return 1;  // Hinv = Lh Lh^T, so U = Lh^T
  auto U = [&](size_t r, size_t c) { return Hinv[c * K + r]; };

  size_t groups = K / group;
  std::vector<uint8_t> zp_full(N * groups);
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
  for (long long n = 0; n < (long long)N; ++n) {
    std::vector<double> w(K);
    for (size_t k = 0; k < K; ++k) w[k] = (double)W[(size_t)n * K + k];
    float s = 1.0f, zf = 0.0f;
    for (size_t j = 0; j < K; ++j) {
      if (j % group == 0) {
        float lo = 0.0f, hi = 0.0f;
        for (size_t i = j; i < j + group; ++i) { lo = rmin(lo, (float)w[i]); hi = rmax(hi, (float)w[i]); }
        uint16_t sh = cfo_f32_to_f16_bits((hi - lo) / 15.0f);
        if ((sh & 0x7fffu) == 0 || (sh & 0x7c00u) == 0x7c00u) sh = 0x3c00u;
        s = cfo_f16_bits_to_f32(sh);
        zf = rclamp(std::round(-lo / s), 0.0f, 15.0f);
        scales[(size_t)n * groups + j / group] = sh;
        zp_full[(size_t)n * groups + j / group] = (uint8_t)f32_as_i8(zf);
      }
      float wj = (float)w[j];
      float qf = rclamp(std::round(wj / s) + zf, 0.0f, 15.0f);
      uint8_t c = (uint8_t)f32_as_i8(qf);
      size_t idx = (size_t)n * K + j;
      if ((idx & 1) == 0) codes[idx >> 1] = (uint8_t)((codes[idx >> 1] & 0xF0) | c);
      else codes[idx >> 1] = (uint8_t)((codes[idx >> 1] & 0x0F) | (c << 4));
      float wq = (qf - zf) * s;
      if (Wdq) Wdq[idx] = wq;
      double e = (w[j] - (double)wq) / U(j, j);
      for (size_t l = j + 1; l < K; ++l) w[l] -= e * U(j, l);
    }
  }
  size_t ng = N * groups;
  for (size_t gi = 0; gi < ng; gi += 2) {
    uint8_t b = zp_full[gi];
    if (gi + 1 < ng) b |= (uint8_t)(zp_full[gi + 1] << 4);
    zps[gi >> 1] = b;
  }
  return 0;
}

// The GPTQ column walk in the device kernels' own arithmetic: f32 state, every operation in the order
// castforge_b200/csrc/gptq.cu performs it, so that codes, scales and zero points can be compared with `==` (cfo_gptq
// above keeps f64 state and differs from any f32 walk on near-ties).  No reference counterpart (GPTQ is absent from
// the reference, src/passes/quantize/schemes.rs:115-121); this restates the product's specification:
//   per block of 128 columns (= one group): lo / hi over the row's CURRENT values, scale = truncating f16 of
//   (hi - lo) / 15 (0 / inf / NaN -> 1.0), zp = clamp(round(-lo / s), 0, 15);
//   per column j of the block: q = clamp(round(w / s) + zp), wq = (q - zp) * s, e = (w - wq) / U[j][j],
//     then w[c] = fma(-e, U[j][c], w[c]) for the block's later columns c (j ascending);
//   after the block: for every later column n, acc = 0; acc = fma(e[k], U[b + k][n], acc) for k = 0..127; w[n] -= acc.
// W: `rows` rows of K f32 values (already widened); U: K x K f32, row-major (the factor the device computed).
// zps_unpacked: one byte per group.  Wdq: NULL or rows x K.
void cfo_gptq_walk_f32(const float* W, size_t rows, size_t K, const float* U, uint8_t* codes, uint16_t* scales,
                       uint8_t* zps_unpacked, float* Wdq, int threads) {
  const size_t groups = K / 128;
  int t = set_threads(threads);
  std::vector<float> state(W, W + rows * K);  // every row's current values
  // block-major: all rows walk block b before any row walks block b + 1 (rows are independent, so the order across
  // rows changes nothing); the 128 rows of U a block needs then stay in cache for every row
  for (size_t b = 0; b < K; b += 128) {
    const size_t rest = K - b - 128;
#ifdef _OPENMP
#pragma omp parallel for num_threads(t) schedule(static) if (t > 1)
#endif
    for (long long r = 0; r < (long long)rows; ++r) {
      float* w = state.data() + (size_t)r * K;
      float e[128];
      float lo = 0.0f, hi = 0.0f;
      for (size_t i = b; i < b + 128; ++i) { lo = std::fmin(lo, w[i]); hi = std::fmax(hi, w[i]); }
      uint16_t sh = cfo_f32_to_f16_bits((hi - lo) / 15.0f);
      if ((sh & 0x7fffu) == 0 || (sh & 0x7c00u) == 0x7c00u) sh = 0x3c00u;
      const float sc = cfo_f16_bits_to_f32(sh);
      float zf = std::round(-lo / sc);
      zf = (zf != zf) ? 0.0f : std::fmin(std::fmax(zf, 0.0f), 15.0f);
      scales[(size_t)r * groups + b / 128] = sh;
      zps_unpacked[(size_t)r * groups + b / 128] = (uint8_t)zf;
      for (size_t j = 0; j < 128; ++j) {
        const float wj = w[b + j];
        float qf = std::round(wj / sc) + zf;
        qf = (qf != qf) ? 0.0f : std::fmin(std::fmax(qf, 0.0f), 15.0f);
        const float wq = (qf - zf) * sc;
        const float ej = (wj - wq) / U[(b + j) * K + b + j];
        e[j] = ej;
        w[b + j] = wq;
        const size_t idx = (size_t)r * K + b + j;
        const uint8_t c = (uint8_t)qf;
        if ((idx & 1) == 0) codes[idx >> 1] = (uint8_t)((codes[idx >> 1] & 0xF0) | c);
        else codes[idx >> 1] = (uint8_t)((codes[idx >> 1] & 0x0F) | (c << 4));
        const float* urow = U + (b + j) * K + b;
        for (size_t c2 = j + 1; c2 < 128; ++c2) w[b + c2] = std::fma(-ej, urow[c2], w[b + c2]);
      }
      // the block's errors into every later column: k outermost so that U is read along its rows; each column's sum
      // still adds k = 0..127 in ascending order into its own accumulator, which starts at zero
      if (rest) {
        std::vector<float> acc(rest, 0.0f);
        float* ap = acc.data();
        for (size_t k = 0; k < 128; ++k) {
          const float ek = e[k];
          const float* urow = U + (b + k) * K + b + 128;
#pragma omp simd
          for (size_t n = 0; n < rest; ++n) ap[n] = std::fma(ek, urow[n], ap[n]);
        }
        float* wr = w + b + 128;
        for (size_t n = 0; n < rest; ++n) wr[n] = wr[n] - ap[n];
      }
    }
  }
  if (Wdq) std::memcpy(Wdq, state.data(), rows * K * sizeof(float));
}

// GGUF Q8_0 export of a per-tensor INT8 tensor (gguf.rs:283-296) and the Q8_0 / Q4_0 decoders (:513-552).
size_t cfo_gguf_pack_q8_0(const int8_t* codes, size_t n, float scale, uint8_t* out) {
  size_t blocks = ((n > 0 ? n : 1) + 31) / 32;
  uint16_t sc = cfo_f32_to_f16_bits(scale);
  for (size_t b = 0; b < blocks; ++b) {
    out[b * 34] = (uint8_t)(sc & 0xff);
    out[b * 34 + 1] = (uint8_t)(sc >> 8);
    for (size_t i = 0; i < 32; ++i) out[b * 34 + 2 + i] = (b * 32 + i < n) ? (uint8_t)codes[b * 32 + i] : 0;
  }
  return blocks * 34;
}
void cfo_gguf_unpack_q8_0(const uint8_t* blocks, size_t n, float* out) {
  for (size_t e = 0; e < n; ++e) {
    const uint8_t* blk = blocks + (e / 32) * 34;
    float d = cfo_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    out[e] = (float)(int8_t)blk[2 + e % 32] * d;
  }
}
void cfo_gguf_unpack_q4_0(const uint8_t* blocks, size_t n, float* out) {
  for (size_t e = 0; e < n; ++e) {
    const uint8_t* blk = blocks + (e / 32) * 18;
    float d = cfo_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    size_t i = e % 32;
    int q = (int)((blk[2 + i / 2] >> ((i & 1) * 4)) & 0xF) - 8;
    out[e] = (float)q * d;
  }
}

// ---------------------------------------------------------------------------------------------
// KV-cache codecs.  K16/V8: AsymK16V8Codec, src/passes/serving/kv_attention.rs:52-222.
// Layout [num_pages, page_tokens, num_kv_heads, head_dim]; scope 0 = PerTensor, 1 = PerLayerHead, 2 = PerPageHead.
// ---------------------------------------------------------------------------------------------
static inline size_t kv_slot(int scope, size_t p, size_t h, size_t H) { return scope == 0 ? 0 : scope == 1 ? h : p * H + h; }

// compute_v_scales (kv_attention.rs:125-183): absmax / 127, 1.0 (KV_ZERO_SCALE_SENTINEL, :10) when the absmax is 0
void cfo_kv_v_scales(const float* v, size_t P, size_t T, size_t H, size_t D, int scope, float* scales) {
  size_t slots = scope == 0 ? 1 : scope == 1 ? H : P * H;
  std::vector<float> amax(slots, 0.0f);
  for (size_t p = 0; p < P; ++p)
    for (size_t t = 0; t < T; ++t)
      for (size_t h = 0; h < H; ++h) {
        float& m = amax[kv_slot(scope, p, h, H)];
        const float* row = v + ((p * T + t) * H + h) * D;
        for (size_t d = 0; d < D; ++d) m = rmax(m, std::fabs(row[d]));
      }
  for (size_t i = 0; i < slots; ++i) scales[i] = amax[i] > 0.0f ? amax[i] / 127.0f : 1.0f;
}

// encode (:69-121).  Returns 1 for the shape the reference rejects (:77-85), else 0.
int cfo_kv_encode_k16v8(const float* k, const float* v, size_t P, size_t T, size_t H, size_t D, int scope, uint16_t* k_bits,
                        int8_t* v_codes, float* v_scales) {
  if (P * T * H * D == 0) return 1;
  size_t n = P * T * H * D;
  for (size_t i = 0; i < n; ++i) k_bits[i] = cfo_f32_to_f16_bits(k[i]);
  cfo_kv_v_scales(v, P, T, H, D, scope, v_scales);
  for (size_t p = 0; p < P; ++p)
    for (size_t t = 0; t < T; ++t)
      for (size_t h = 0; h < H; ++h) {
        float scale = v_scales[kv_slot(scope, p, h, H)];
        size_t base = ((p * T + t) * H + h) * D;
        for (size_t d = 0; d < D; ++d) v_codes[base + d] = f32_as_i8(rclamp(std::round(v[base + d] / scale), -127.0f, 127.0f));
      }
  return 0;
}

// decode (:186-221)
void cfo_kv_decode_k16v8(const uint16_t* k_bits, const int8_t* v_codes, const float* v_scales, size_t P, size_t T, size_t H, size_t D,
                         int scope, float* k_out, float* v_out) {
  size_t n = P * T * H * D;
  for (size_t i = 0; i < n; ++i) k_out[i] = cfo_f16_bits_to_f32(k_bits[i]);
  for (size_t p = 0; p < P; ++p)
    for (size_t t = 0; t < T; ++t)
      for (size_t h = 0; h < H; ++h) {
        float scale = v_scales[kv_slot(scope, p, h, H)];
        size_t base = ((p * T + t) * H + h) * D;
        for (size_t d = 0; d < D; ++d) v_out[base + d] = (float)v_codes[base + d] * scale;
      }
}

// E4M3FN slice codec (src/passes/serving/mutable_loads.rs:431-441).  which = 0: the reference's encoder as written
// (cfo_e4m3_encode_ref); 1: round-to-nearest-even onto the grid (cfo_e4m3_encode_rne), which the device follows.
void cfo_e4m3_slice_encode(const float* src, size_t n, int which, uint8_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = which == 0 ? cfo_e4m3_encode_ref(src[i]) : cfo_e4m3_encode_rne(src[i]);
}
void cfo_e4m3_slice_decode(const uint8_t* codes, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = cfo_e4m3_decode(codes[i]);
}

// ---------------------------------------------------------------------------------------------
// Weight surgery upstream of quantize: merge_f32_tensors (src/passes/weights/merge.rs:396-440),
// apply_dare_pruning (:357-384) and the task-vector arithmetic of MergeTaskVectorsPass::run (:271-290).
// ---------------------------------------------------------------------------------------------
static inline float rust_signum(float x) { return x != x ? x : std::copysign(1.0f, x); }

static void merge_linear(const float* a, const float* b, size_t n, float t, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = (1.0f - t) * a[i] + t * b[i];
}

// method: 0 linear, 1 slerp, 2 ties.  coef_out (nullable): the two coefficients the slerp used (or 1-t, t).
void cfo_merge_f32(const float* a, const float* b, size_t n, int method, float t, float* out, float* coef_out) {
  if (coef_out) { coef_out[0] = 1.0f - t; coef_out[1] = t; }
  if (method == 1) {
    float sa = 0.0f, sb = 0.0f;
    for (size_t i = 0; i < n; ++i) sa += a[i] * a[i];
    for (size_t i = 0; i < n; ++i) sb += b[i] * b[i];
    float norm_a = std::sqrt(sa), norm_b = std::sqrt(sb);
    if (norm_a < 1e-8f || norm_b < 1e-8f) return merge_linear(a, b, n, t, out);
    float dot = 0.0f;
    for (size_t i = 0; i < n; ++i) dot += (a[i] / norm_a) * (b[i] / norm_b);
    float dc = rclamp(dot, -0.9995f, 0.9995f);
    float omega = std::acos(dc), sin_omega = std::sin(omega);
    if (std::fabs(sin_omega) < 1e-6f) return merge_linear(a, b, n, t, out);
    float ca = std::sin((1.0f - t) * omega) / sin_omega, cb = std::sin(t * omega) / sin_omega;
    if (coef_out) { coef_out[0] = ca; coef_out[1] = cb; }
    for (size_t i = 0; i < n; ++i) out[i] = ca * a[i] + cb * b[i];
    return;
  }
  if (method == 2) {
    for (size_t i = 0; i < n; ++i) {
      float va = a[i], vb = b[i];
      float elected = rust_signum((1.0f - t) * va + t * vb);
      float sum = 0.0f, wsum = 0.0f;
      if (rust_signum(va) == elected || va == 0.0f) { sum += (1.0f - t) * va; wsum += 1.0f - t; }
      if (rust_signum(vb) == elected || vb == 0.0f) { sum += t * vb; wsum += t; }
      out[i] = wsum > 0.0f ? sum / wsum : (1.0f - t) * va + t * vb;
    }
    return;
  }
  merge_linear(a, b, n, t, out);
}

// The `drop_count` entries of smallest |delta| (ties: lowest index first -- the sort is stable) become 0, the rest are
// scaled by 1 / (1 - p).  NaN deltas have no defined place in the reference's ordering and are not supported.
void cfo_dare_prune(const float* delta, size_t n, float drop_rate, float* out) {
  float p = rclamp(drop_rate, 0.0f, 0.99f);
  std::memcpy(out, delta, n * sizeof(float));
  if (p <= 1e-6f || n == 0) return;
  size_t drop_count = (size_t)std::floor((float)n * p);
  if (drop_count == 0) return;
  std::vector<size_t> idx(n);
  for (size_t i = 0; i < n; ++i) idx[i] = i;
  std::stable_sort(idx.begin(), idx.end(), [&](size_t x, size_t y) { return std::fabs(delta[x]) < std::fabs(delta[y]); });
  float rescale = 1.0f / (1.0f - p);
  for (size_t r = 0; r < n; ++r) {
    if (r < drop_count) out[idx[r]] = 0.0f;
    else out[idx[r]] *= rescale;
  }
}

void cfo_task_vector_merge(const float* base, const float* const* finetuned, int count, size_t n, float lambda, float drop_rate,
                           float* out) {
  std::vector<std::vector<float>> tvs;
  std::vector<float> delta(n), pruned(n);
  for (int c = 0; c < count; ++c) {
    for (size_t i = 0; i < n; ++i) delta[i] = finetuned[c][i] - base[i];
    cfo_dare_prune(delta.data(), n, drop_rate, pruned.data());
    tvs.push_back(pruned);
  }
  std::memcpy(out, base, n * sizeof(float));
  for (auto& tv : tvs)
    for (size_t i = 0; i < n; ++i) out[i] += lambda * tv[i];
}

// apply_2to4_mask (src/passes/weights/prune.rs:548-565): stable ascending sort of the four magnitudes, first two -> 0.0
void cfo_apply_2to4_mask(float* vals, size_t n) {
  for (size_t g = 0; g + 4 <= n; g += 4) {
    int idx[4] = {0, 1, 2, 3};
    float* c = vals + g;
    std::stable_sort(idx, idx + 4, [&](int x, int y) { return std::fabs(c[x]) < std::fabs(c[y]); });
    c[idx[0]] = 0.0f;
    c[idx[1]] = 0.0f;
  }
}

// keep_cols of PruneStructuredPass::run (prune.rs:339-341)
size_t cfo_prune_keep_cols(size_t cols, float sparsity) {
  float kf = std::round((float)cols * (1.0f - rclamp(sparsity, 0.0f, 0.9f)));
  size_t k = (kf != kf || kf <= 0.0f) ? 0 : (size_t)kf;
  if (cols == 0) return 0;
  return k < 1 ? 1 : (k > cols ? cols : k);
}

// prune_2d_columns_by_l1 (prune.rs:568-603).  out: rows x keep (keep = clamp(keep_cols, 1, cols)), kept: keep indices.
// Returns keep (cols when the reference returns its input unchanged: an empty matrix).
size_t cfo_prune_columns_l1(const float* values, size_t rows, size_t cols, size_t keep_cols, float* out, int32_t* kept) {
  if (rows == 0 || cols == 0) {
    for (size_t c = 0; c < cols; ++c) kept[c] = (int32_t)c;
    return cols;
  }
  size_t keep = keep_cols < 1 ? 1 : (keep_cols > cols ? cols : keep_cols);
  std::vector<std::pair<size_t, float>> sc(cols);
  for (size_t c = 0; c < cols; ++c) {
    float l1 = 0.0f;
    for (size_t r = 0; r < rows; ++r) l1 += std::fabs(values[r * cols + c]);
    sc[c] = {c, l1};
  }
  std::stable_sort(sc.begin(), sc.end(), [](const std::pair<size_t, float>& a, const std::pair<size_t, float>& b) { return a.second > b.second; });
  std::vector<size_t> ki;
  for (size_t i = 0; i < keep; ++i) ki.push_back(sc[i].first);
  std::sort(ki.begin(), ki.end());
  for (size_t i = 0; i < keep; ++i) kept[i] = (int32_t)ki[i];
  for (size_t r = 0; r < rows; ++r)
    for (size_t i = 0; i < keep; ++i) out[r * keep + i] = values[r * cols + ki[i]];
  return keep;
}

// pack-weights (src/passes/weights/fold.rs:549-554): [K, N] -> [N, K]
void cfo_transpose_f32(const float* w, size_t K, size_t N, float* out) {
  for (size_t k = 0; k < K; ++k)
    for (size_t n = 0; n < N; ++n) out[n * K + k] = w[k * N + n];
}

// LoRA / DoRA baking: BakeLoraPass::run (src/passes/weights/lora.rs:79-88), run_bake_dora (:277-380)
void cfo_lora_bake(float* W, const float* A, const float* B, size_t k, size_t n, size_t r, float alpha) {
  for (size_t row = 0; row < k; ++row)
    for (size_t col = 0; col < n; ++col) {
      float delta = 0.0f;
      for (size_t p = 0; p < r; ++p) delta += A[row * r + p] * B[p * n + col];
      W[row * n + col] += alpha * delta;
    }
}
void cfo_column_norms(const float* W, size_t k, size_t n, float* mags) {
  for (size_t col = 0; col < n; ++col) {
    float sq = 0.0f;
    for (size_t row = 0; row < k; ++row) {
      float v = W[row * n + col];
      sq += v * v;
    }
    mags[col] = rmax(std::sqrt(sq), 1e-8f);
  }
}
// orig_mags nullable: the column then keeps its own norm.  norms_out (nullable): the norms of the columns before renormalising.
void cfo_dora_renorm(float* W, size_t k, size_t n, const float* orig_mags, float* norms_out) {
  std::vector<float> norm(n);
  cfo_column_norms(W, k, n, norm.data());
  for (size_t col = 0; col < n; ++col) {
    float mag = orig_mags ? orig_mags[col] : norm[col];
    for (size_t row = 0; row < k; ++row) {
      float dir = W[row * n + col] / norm[col];
      W[row * n + col] = mag * dir;
    }
  }
  if (norms_out) std::memcpy(norms_out, norm.data(), n * sizeof(float));
}

int cfo_max_threads(void) { return set_threads(0); }

}  // extern "C"
