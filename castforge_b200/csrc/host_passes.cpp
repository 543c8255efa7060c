// Pipeline-spec grammar, the `quantize` pass family's option handling, and the driver that runs a
// quantize pass over a host TensorStore through the device entry points.
//   split_pipeline_spec / parse_pass_spec_item     src/passes/registry/manager.rs:410-459
//   option validation + alias list                  manager.rs:512-540, :548-727, config/passes.toml:49-71
//   quantize option defaults and scheme inference   src/passes/registry/families.rs:89-185, leaf.rs:98-257
//   dispatch on the scheme string                   src/passes/quantize/schemes.rs:84-154
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <set>

#include "../../include/cfb200.h"
#include "host.h"

namespace cfb {
namespace host {

const std::string* opt_get(const PassOptions& o, const std::string& k) {
  for (auto& kv : o)
    if (kv.first == k) return &kv.second;
  return nullptr;
}

static std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && isspace((unsigned char)s[a])) ++a;
  while (b > a && isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}

std::vector<std::string> split_pipeline_spec(const std::string& spec) {
  std::vector<std::string> out;
  size_t start = 0, depth = 0;
  for (size_t i = 0; i < spec.size(); ++i) {
    const char c = spec[i];
    if (c == '(') ++depth;
    else if (c == ')') depth = depth ? depth - 1 : 0;
    else if ((c == ',' || c == '|') && depth == 0) {
      out.push_back(spec.substr(start, i - start));
      start = i + 1;
    }
  }
  out.push_back(spec.substr(start));
  return out;
}

bool parse_pass_spec_item(const std::string& raw, std::string* name, PassOptions* opts, std::string* err) {
  const std::string item = trim(raw);
  opts->clear();
  const size_t open = item.find('(');
  if (open == std::string::npos) { *name = item; return true; }
  const size_t close = item.rfind(')');
  if (close == std::string::npos) { *err = "Unclosed `(` in pass specification `" + item + "`"; return false; }
  if (!trim(item.substr(close + 1)).empty()) { *err = "Unexpected trailing characters after `)` in pass specification `" + item + "`"; return false; }
  *name = trim(item.substr(0, open));
  const std::string inner = item.substr(open + 1, close > open ? close - open - 1 : 0);
  size_t s = 0;
  while (s <= inner.size()) {
    size_t e = inner.find(',', s);
    if (e == std::string::npos) e = inner.size();
    const std::string kv = trim(inner.substr(s, e - s));
    s = e + 1;
    if (kv.empty()) continue;
    const size_t eq = kv.find('=');
    if (eq == std::string::npos) { *err = "Expected `key=value` option in `" + item + "`"; return false; }
    std::string v = trim(kv.substr(eq + 1));
    while (!v.empty() && v.front() == '"') v.erase(0, 1);
    while (!v.empty() && v.back() == '"') v.pop_back();
    while (!v.empty() && v.front() == '\'') v.erase(0, 1);
    while (!v.empty() && v.back() == '\'') v.pop_back();
    const std::string k = trim(kv.substr(0, eq));
    bool replaced = false;
    for (auto& o : *opts)
      if (o.first == k) { o.second = v; replaced = true; }
    if (!replaced) opts->emplace_back(k, v);
  }
  return true;
}

static std::string jstr(const std::string& s) {
  std::string o = "\"";
  for (char c : s) {
    if (c == '"' || c == '\\') o.push_back('\\');
    o.push_back(c);
  }
  return o + "\"";
}
// serde_json::to_string_pretty of Vec<PassTelemetry> (field order of manager.rs:112-124)
std::string telemetry_json(const std::vector<PassTelemetry>& t) {
  if (t.empty()) return "[]";
  std::string o = "[\n";
  for (size_t i = 0; i < t.size(); ++i) {
    const PassTelemetry& p = t[i];
    o += "  {\n";
    o += "    \"iteration\": " + std::to_string(p.iteration) + ",\n";
    o += "    \"pass_name\": " + jstr(p.pass_name) + ",\n";
    o += std::string("    \"changed\": ") + (p.changed ? "true" : "false") + ",\n";
    o += "    \"elapsed_us\": " + std::to_string(p.elapsed_us) + ",\n";
    o += "    \"live_ops_before\": " + std::to_string(p.live_ops_before) + ",\n";
    o += "    \"live_ops_after\": " + std::to_string(p.live_ops_after) + ",\n";
    o += "    \"ops_created\": " + std::to_string(p.ops_created) + ",\n";
    o += "    \"ops_modified\": " + std::to_string(p.ops_modified) + ",\n";
    o += "    \"ops_removed\": " + std::to_string(p.ops_removed) + "\n";
    o += i + 1 < t.size() ? "  },\n" : "  }\n";
  }
  return o + "]";
}

// ---- names and options ----------------------------------------------------------------------------
static const char* const kPassNames[] = {"quantize", "quantize-weights", "quantize-groupwise", "quantize-fp8", "quantize-fp4",
                                         "calibrate-quantize", "smooth-quantize", "insert-qat-ste", "rotate-hadamard",
                                         "lower-mixed-precision", "fuse-gemm", "fuse-dequant-matmul"};
bool is_known_pass(const std::string& name) {
  for (const char* n : kPassNames)
    if (name == n) return true;
  return false;
}

// keys the reference accepts on any pass besides the catalogued ones (manager.rs:548-727); only the
// ones that can matter for the passes kept here are listed
static bool is_alias_key(const std::string& k) {
  static const std::set<std::string> keys = {
      "mode", "kind", "target", "targets", "dtype", "group", "mxfp8", "size", "samples", "num_samples", "block_size",
      "salient_ratio", "awq_salient", "alpha", "bits", "group_size", "hadamard", "scheme", "format", "min_elements", "method",
      "ratio", "value", "name", "count", "filter", "prefix", "all", "eps", "tol", "tolerance"};
  return keys.count(k) != 0;
}
static bool catalog_has(const std::string& pass, const std::string& k) {
  // config/passes.toml: documented options per pass
  static const std::map<std::string, std::set<std::string>> cat = {
      {"quantize", {"scheme", "bits", "group_size", "salient_ratio", "format", "block_size", "alpha"}},
      {"quantize-weights", {"bits", "min_elements"}},
      {"quantize-groupwise", {"bits", "group_size", "awq_salient", "salient_ratio"}},
      {"quantize-fp8", {"format", "mxfp8", "block_size"}},
      {"quantize-fp4", {"scheme", "block_size"}},
      {"calibrate-quantize", {"bits", "samples"}},
      {"smooth-quantize", {"bits", "alpha", "samples"}},
      {"insert-qat-ste", {"bits"}},
      {"rotate-hadamard", {"block_size"}},
      {"lower-mixed-precision", {"dtype"}},
      {"fuse-gemm", {"kind"}},
      {"fuse-dequant-matmul", {}}};
  auto it = cat.find(pass);
  return it != cat.end() && it->second.count(k) != 0;
}

template <typename T>
static bool parse_num(const std::string* s, T* out) {
  if (!s) return false;
  char* e = nullptr;
  if (std::is_floating_point<T>::value) {
    const double v = strtod(s->c_str(), &e);
    if (e == s->c_str() || *e) return false;
    *out = (T)v;
  } else {
    if (s->empty() || (*s)[0] == '-' || (*s)[0] == '+') return false;  // Rust's unsigned parse rejects signs... '+' is accepted, keep strict
    const unsigned long long v = strtoull(s->c_str(), &e, 10);
    if (e == s->c_str() || *e) return false;
    *out = (T)v;
  }
  return true;
}

bool resolve_quantize(const std::string& pass, const PassOptions& opts, QuantizeConfig* c, std::string* err) {
  if (!is_known_pass(pass)) { *err = "Unknown pass `" + pass + "`. Run `castforge list-passes` to see available passes."; return false; }
  for (auto& kv : opts)
    if (!catalog_has(pass, kv.first) && !is_alias_key(kv.first)) {
      *err = "Pass `" + pass + "`: unrecognized option `" + kv.first + "`";
      return false;
    }
  auto has = [&](const char* k) { return opt_get(opts, k) != nullptr; };
  QuantizeConfig q;
  if (pass == "quantize") {
    const std::string* s = opt_get(opts, "scheme");
    if (!s) s = opt_get(opts, "mode");
    if (!s) s = opt_get(opts, "dtype");
    if (s) q.scheme = *s;
    else if (has("alpha")) q.scheme = "smoothquant";
    else if (has("salient_ratio")) q.scheme = "awq";
    else if (has("group_size") || has("awq_salient")) q.scheme = "groupwise";  // NB: the alias `group` does not select it
    else if (has("format") || has("mxfp8")) q.scheme = "fp8";
    else if (has("samples") || has("num_samples")) q.scheme = "w8a8";
    else if (has("block_size") && !has("bits")) q.scheme = "hadamard";
    else q.scheme = "weight";
  } else if (pass == "quantize-weights") q.scheme = "weight";
  else if (pass == "quantize-groupwise") q.scheme = "groupwise";
  else if (pass == "quantize-fp8") q.scheme = "fp8";
  else if (pass == "quantize-fp4") {
    const std::string* s = opt_get(opts, "scheme");
    if (!s) s = opt_get(opts, "format");
    q.scheme = s ? *s : "nvfp4";
  } else if (pass == "calibrate-quantize") q.scheme = "w8a8";
  else if (pass == "smooth-quantize") q.scheme = "smoothquant";
  else if (pass == "insert-qat-ste") q.scheme = "qat_ste";
  else if (pass == "rotate-hadamard") q.scheme = "hadamard";
  else if (pass == "lower-mixed-precision") {
    const std::string* s = opt_get(opts, "dtype");
    q.scheme = s ? *s : "f16";
  } else q.scheme = pass;  // fuse-gemm / fuse-dequant-matmul: graph-only
  std::string sl = q.scheme;
  std::transform(sl.begin(), sl.end(), sl.begin(), ::tolower);
  const bool four = sl == "groupwise" || sl == "awq" || sl == "gptq" || sl == "fp4" || sl == "mxfp4" || sl == "nvfp4" ||
                    sl == "int4_asym" || sl == "nf4" || pass == "quantize-groupwise";
  q.bits = four ? 4 : 8;
  unsigned b;
  if (parse_num(opt_get(opts, "bits"), &b) && b <= 255) q.bits = (int)b;
  parse_num(opt_get(opts, "min_elements"), &q.min_elements);
  if (!parse_num(opt_get(opts, "group_size"), &q.group_size)) parse_num(opt_get(opts, "group"), &q.group_size);
  if (const std::string* s = opt_get(opts, "awq_salient")) q.awq_salient = *s != "false";
  parse_num(opt_get(opts, "salient_ratio"), &q.salient_ratio);
  if (const std::string* s = opt_get(opts, "format")) q.format = *s;
  else if (const std::string* d = opt_get(opts, "dtype")) q.format = *d;
  if (const std::string* s = opt_get(opts, "mxfp8")) q.mxfp8 = *s != "false";
  q.block_size = pass == "quantize-fp4" ? 16 : 32;
  if (!parse_num(opt_get(opts, "block_size"), &q.block_size) && pass == "quantize") parse_num(opt_get(opts, "size"), &q.block_size);
  if (!parse_num(opt_get(opts, "samples"), &q.samples)) parse_num(opt_get(opts, "num_samples"), &q.samples);
  parse_num(opt_get(opts, "alpha"), &q.alpha);
  if (const std::string* s = opt_get(opts, "hadamard")) q.hadamard = (*s == "true" || *s == "1");
  *c = q;
  return true;
}

// ---- device streaming engine ------------------------------------------------------------------------
namespace {

struct OutPiece { std::string suffix; DType dtype; std::vector<int64_t> shape; size_t offset, bytes; };
struct Plan {
  size_t in_bytes = 0, out_bytes = 0, scratch_bytes = 0;
  std::vector<OutPiece> pieces;  // piece 0 replaces the entry itself
};

struct Slot { void *in = nullptr, *out = nullptr, *scratch = nullptr; size_t in_cap = 0, out_cap = 0, scratch_cap = 0; cudaEvent_t free_ev = nullptr; bool used = false; };
struct Engine {
  std::mutex busy;  // one pipeline at a time per device: the slots and streams below are shared by every caller
  int dev = -1;
  cudaStream_t s_h2d = nullptr, s_cmp = nullptr, s_d2h = nullptr;
  Slot slots[3];
  float* small = nullptr;  // per-tensor scalars {scale, absmax, thr, spare} x kMaxTensors
  size_t small_cap = 0;
};
Engine g_engine[16];

bool ck(cudaError_t e, std::string* err, const char* what) {
  if (e == cudaSuccess) return true;
  *err = std::string(what) + ": " + cudaGetErrorString(e);
  return false;
}
bool grow(void** p, size_t* cap, size_t need, std::string* err) {
  if (need <= *cap) return true;
  if (*p) cudaFree(*p);
  *p = nullptr;
  *cap = 0;
  const size_t want = need + need / 8 + 256;
  if (!ck(cudaMalloc(p, want), err, "cudaMalloc (staging)")) return false;
  *cap = want;
  return true;
}
Engine* engine(std::string* err) {
  static std::mutex init_mutex;
  std::lock_guard<std::mutex> lock(init_mutex);
  int dev = 0;
  if (!ck(cudaGetDevice(&dev), err, "cudaGetDevice")) return nullptr;
  if (dev < 0 || dev >= 16) { *err = "device ordinal out of range"; return nullptr; }
  Engine& e = g_engine[dev];
  if (e.dev != dev) {
    if (!ck(cudaStreamCreateWithFlags(&e.s_h2d, cudaStreamNonBlocking), err, "cudaStreamCreate")) return nullptr;
    if (!ck(cudaStreamCreateWithFlags(&e.s_cmp, cudaStreamNonBlocking), err, "cudaStreamCreate")) return nullptr;
    if (!ck(cudaStreamCreateWithFlags(&e.s_d2h, cudaStreamNonBlocking), err, "cudaStreamCreate")) return nullptr;
    for (auto& s : e.slots)
      if (!ck(cudaEventCreateWithFlags(&s.free_ev, cudaEventDisableTiming), err, "cudaEventCreate")) return nullptr;
    e.dev = dev;
  }
  return &e;
}

int dev_dtype(DType d) { return d == DType::F32 ? CFB200_F32 : d == DType::F16 ? CFB200_F16 : CFB200_BF16; }
bool is_float(DType d) { return d == DType::F32 || d == DType::F16 || d == DType::BF16; }

// widen f16 / bf16 host data to f32 exactly as tensor_store.rs:58-111 does
void widen_to_f32(const TensorEntry& e, float* out) {
  const size_t n = e.num_elements();
  if (e.dtype == DType::F32) { memcpy(out, e.data.data(), n * 4); return; }
  const uint16_t* src = reinterpret_cast<const uint16_t*>(e.data.data());
  for (size_t i = 0; i < n; ++i) {
    uint32_t o;
    const uint16_t b = src[i];
    if (e.dtype == DType::BF16) o = (uint32_t)b << 16;
    else {
      const uint32_t s = (b >> 15) & 1, ex = (b >> 10) & 0x1f, m = b & 0x3ff;
      if (ex == 0) {
        if (!m) o = s << 31;
        else { uint32_t mm = m, ee = 127 - 14; while (!(mm & 0x400)) { mm <<= 1; --ee; } mm &= 0x3ff; o = (s << 31) | (ee << 23) | (mm << 13); }
      } else if (ex == 31) o = (s << 31) | 0x7f800000u | (m << 13);
      else o = (s << 31) | ((ex + 112) << 23) | (m << 13);
    }
    memcpy(out + i, &o, 4);
  }
}

}  // namespace

bool run_quantize_on_store(TensorStore& store, const QuantizeConfig& cfg, PassResult* res, std::string* err) {
  res->pass_name = "quantize";
  std::string s = cfg.scheme;
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  enum Kind { kWeight, kGroup, kFp8, kFp4, kQat, kSmooth, kHadamard, kPerChannel, kInt4, kNf4, kE4m3, kGraphOnly } kind;
  if (s == "f16" || s == "bf16" || s == "mixed_precision" || s == "amp" || s == "w8a8" || s == "calibrate" || s == "static" ||
      s == "fuse-gemm" || s == "fuse-dequant-matmul")
    kind = kGraphOnly;  // graph rewrites: no tensor data is touched (formats.rs:38-112, :541-611)
  else if (s == "hadamard" || s == "quarot" || s == "spinquant") kind = kHadamard;
  else if (s == "groupwise" || s == "awq" || s == "gptq") kind = kGroup;
  else if (s == "fp8" || s == "mxfp8" || s == "e4m3" || s == "e5m2") kind = kFp8;
  else if (s == "fp4" || s == "mxfp4" || s == "nvfp4" || s == "e2m1") kind = kFp4;
  else if (s == "smoothquant" || s == "smooth") kind = kSmooth;
  else if (s == "qat" || s == "qat_ste" || s == "ste") kind = kQat;
  else if (s == "per_channel") kind = kPerChannel;   // explicit extension schemes: must be spelt exactly
  else if (s == "int4_asym") kind = kInt4;
  else if (s == "nf4") kind = kNf4;
  else if (s == "fp8_e4m3") kind = kE4m3;
  else if (s.rfind("ext:", 0) == 0) { *err = "unknown extension scheme `" + cfg.scheme + "`"; return false; }
  else kind = kWeight;  // any other string silently means per-tensor weights (schemes.rs:114-150)
  if (kind == kGraphOnly) return true;
  if (cfg.hadamard && kind != kHadamard) {  // optional rotation before the main scheme (schemes.rs:103-111)
    QuantizeConfig h = cfg;
    h.scheme = "hadamard";
    h.hadamard = false;
    PassResult hr;
    if (!run_quantize_on_store(store, h, &hr, err)) return false;
    res->ops_modified += hr.ops_modified;
  }

  Engine* eng = engine(err);
  if (!eng) return false;
  // Calls from several host threads are allowed (the reference's C ABI is re-entrant); on one device they take turns.
  std::lock_guard<std::mutex> engine_lock(eng->busy);
  const int bits = cfg.bits;
  const bool awq = cfg.awq_salient || s == "awq";

  // ---- eligibility and per-tensor plans ----
  std::vector<size_t> todo;
  std::vector<Plan> plans;
  for (size_t i = 0; i < store.size(); ++i) {
    TensorEntry& e = store.at(i);
    if (e.quantized || !is_float(e.dtype)) continue;
    const size_t n = e.num_elements();
    const size_t rank = e.shape.size();
    Plan p;
    bool ok = true;
    const bool needs_f32 = kind == kGroup || kind == kFp8 || kind == kFp4 || kind == kQat || kind == kSmooth || kind == kHadamard;
    p.in_bytes = needs_f32 ? n * 4 : n * dtype_bytes(e.dtype);
    switch (kind) {
      case kWeight: ok = n >= cfg.min_elements; p.out_bytes = n; p.pieces.push_back({"", bits == 4 ? DType::I4 : DType::I8, e.shape, 0, n}); break;
      case kGroup: ok = rank >= 2 && n >= 2; break;
      case kFp8: ok = n >= 2; break;
      case kFp4: ok = n >= 2 && e.dtype == DType::F32; break;
      case kQat: ok = n >= 2 && e.dtype == DType::F32; break;
      case kSmooth: ok = n >= 2; break;
      case kHadamard: ok = rank == 2 && e.shape[0] >= 2 && e.shape[1] > 0; break;
      case kPerChannel: {
        ok = rank == 2 && n >= 2;
        if (!ok) break;
        const size_t rows = (size_t)e.shape[0];
        p.out_bytes = ((n + 255) & ~(size_t)255) + rows * 4;
        p.pieces.push_back({"", bits == 4 ? DType::I4 : DType::I8, e.shape, 0, n});
        p.pieces.push_back({".scales", DType::F32, {(int64_t)rows}, (n + 255) & ~(size_t)255, rows * 4});
        break;
      }
      case kInt4: {
        const size_t g = cfg.group_size;
        ok = n >= 2 && (g == 32 || g == 64 || g == 128 || g == 256);
        if (!ok) break;
        const size_t ng = (n + g - 1) / g, cb = (n + 1) / 2, o1 = (cb + 255) & ~(size_t)255, o2 = (o1 + ng * 2 + 255) & ~(size_t)255;
        p.out_bytes = o2 + (ng + 1) / 2;
        p.pieces.push_back({"", DType::U8, {(int64_t)cb}, 0, cb});
        p.pieces.push_back({".scales", DType::F16, {(int64_t)ng}, o1, ng * 2});
        p.pieces.push_back({".zeros", DType::U8, {(int64_t)((ng + 1) / 2)}, o2, (ng + 1) / 2});
        break;
      }
      case kNf4: {
        const size_t blk = cfg.block_size == 32 ? 64 : cfg.block_size;  // default block 64 for NF4
        ok = n >= 2 && (blk == 32 || blk == 64 || blk == 128 || blk == 256);
        if (!ok) break;
        const size_t nb = (n + blk - 1) / blk, nsb = (nb + 255) / 256, cb = (n + 1) / 2;
        const size_t o1 = (cb + 255) & ~(size_t)255, o2 = (o1 + nb + 255) & ~(size_t)255;
        p.out_bytes = o2 + nsb * 4;
        p.scratch_bytes = nb * 4;
        p.pieces.push_back({"", DType::U8, {(int64_t)cb}, 0, cb});
        p.pieces.push_back({".absmax8", DType::U8, {(int64_t)nb}, o1, nb});
        p.pieces.push_back({".absmax2", DType::F32, {(int64_t)nsb}, o2, nsb * 4});
        break;
      }
      case kE4m3: ok = n >= 2; p.out_bytes = n; p.pieces.push_back({"", DType::U8, e.shape, 0, n}); break;
      default: break;
    }
    if (!ok) continue;
    if (needs_f32) { p.out_bytes = n * 4; p.pieces.push_back({"", DType::F32, e.shape, 0, n * 4}); }
    if (kind == kGroup) p.scratch_bytes = cfb200_select_kth_workspace_bytes_for(n);
    todo.push_back(i);
    plans.push_back(std::move(p));
  }
  if (todo.empty()) return true;

  size_t max_in = 0, max_out = 0, max_scr = 0;
  for (auto& p : plans) { max_in = std::max(max_in, p.in_bytes); max_out = std::max(max_out, p.out_bytes); max_scr = std::max(max_scr, p.scratch_bytes); }
  for (auto& sl : eng->slots) {
    if (!grow(&sl.in, &sl.in_cap, max_in, err) || !grow(&sl.out, &sl.out_cap, max_out, err) || !grow(&sl.scratch, &sl.scratch_cap, max_scr, err)) return false;
    sl.used = false;
  }
  {
    void* p = eng->small;
    size_t cap = eng->small_cap;
    if (!grow(&p, &cap, todo.size() * 16, err)) return false;
    eng->small = (float*)p;
    eng->small_cap = cap;
  }
  HostBuffer small_host = HostBuffer::owned(todo.size() * 16);
  std::vector<std::vector<HostBuffer>> outs(todo.size());
  std::vector<HostBuffer> widened(todo.size());
  std::vector<uint64_t> aux(todo.size(), 0);
  std::vector<cudaEvent_t> evs;
  auto new_event = [&]() { cudaEvent_t e; cudaEventCreateWithFlags(&e, cudaEventDisableTiming); evs.push_back(e); return e; };
  bool ok_all = true;
  // Entries that are still slices of a file (lazy SafeTensors load) are read, several threads per slice, into a ring
  // of three pinned staging buffers: while tensor t is being read, the copies and kernels of t-1 and t-2 are in flight.
  HostBuffer staging[3];
  cudaEvent_t staging_free[3] = {nullptr, nullptr, nullptr};
  size_t n_staged = 0;

  for (size_t t = 0; t < todo.size() && ok_all; ++t) {
    TensorEntry& e = store.at(todo[t]);
    const Plan& p = plans[t];
    Slot& sl = eng->slots[t % 3];
    const size_t n = e.num_elements();
    const bool needs_f32 = p.in_bytes == n * 4 && e.dtype != DType::F32;
    if (e.external() && needs_f32) ok_all = e.resolve(err);  // widened on the host below: read it whole first
    if (!ok_all) break;
    const void* hsrc = e.data.data();
    int staged = -1;
    if (e.external()) {
      staged = (int)(n_staged++ % 3);
      if (staging[staged].size() < p.in_bytes) staging[staged] = HostBuffer::owned(max_in);
      if (staging_free[staged]) cudaEventSynchronize(staging_free[staged]);  // the copy that last used this buffer is done
      ok_all = read_file_slice_parallel(e.ext_path, e.ext_offset, e.ext_length, staging[staged].data(), err);
      if (!ok_all) break;
      hsrc = staging[staged].data();
    }
    if (needs_f32) {  // fake-quant passes work on f32 values (resolve_f32_attr)
      widened[t] = HostBuffer::owned(n * 4);
      widen_to_f32(e, reinterpret_cast<float*>(widened[t].data()));
      hsrc = widened[t].data();
    }
    if (sl.used) cudaStreamWaitEvent(eng->s_h2d, sl.free_ev, 0);
    ok_all = ck(cudaMemcpyAsync(sl.in, hsrc, p.in_bytes, cudaMemcpyHostToDevice, eng->s_h2d), err, "H2D copy");
    if (!ok_all) break;
    cudaEvent_t e_in = new_event();
    cudaEventRecord(e_in, eng->s_h2d);
    if (staged >= 0) staging_free[staged] = e_in;
    cudaStreamWaitEvent(eng->s_cmp, e_in, 0);
    float* sm = eng->small + 4 * t;
    uint8_t* out = static_cast<uint8_t*>(sl.out);
    int32_t rc = 0;
    const int dd = needs_f32 ? CFB200_F32 : dev_dtype(e.dtype);
    switch (kind) {
      case kWeight: rc = cfb200_quant_sym_tensor(sl.in, dd, n, bits, (int8_t*)out, sm, eng->s_cmp); break;
      case kQat: rc = cfb200_fakequant_tensor((const float*)sl.in, n, bits, (float*)out, sm, eng->s_cmp); break;
      case kGroup:
        if (awq) rc = cfb200_select_kth_abs((const float*)sl.in, n, cfg.salient_ratio, sm + 2, &aux[t], sl.scratch, sl.scratch_cap, eng->s_cmp);
        if (!rc) rc = cfb200_fakequant_group((const float*)sl.in, n, bits, cfg.group_size, awq, sm + 2, (float*)out, eng->s_cmp);
        break;
      case kFp8: {
        std::string f = cfg.format;
        std::transform(f.begin(), f.end(), f.begin(), ::tolower);
        rc = cfb200_fakequant_fp8grid((const float*)sl.in, n, cfg.block_size, f == "e5m2", cfg.mxfp8, (float*)out, eng->s_cmp);
        break;
      }
      case kFp4: {
        const size_t blk = (s == "nvfp4" && cfg.block_size == 32) ? 16 : std::max<size_t>(cfg.block_size, 4);  // formats.rs:419-423
        rc = cfb200_fakequant_e2m1((const float*)sl.in, n, blk, (float*)out, eng->s_cmp);
        aux[t] = (n + blk - 1) / blk;
        break;
      }
      case kSmooth: {
        // the two scalars need powf on the host (schemes.rs:229-238): absmax -> sync -> scalars -> apply
        rc = cfb200_absmax(sl.in, CFB200_F32, n, sm + 1, eng->s_cmp);
        float am = 0.0f;
        if (!rc) {
          cudaMemcpyAsync(small_host.data() + 16 * t + 4, sm + 1, 4, cudaMemcpyDeviceToHost, eng->s_cmp);
          cudaStreamSynchronize(eng->s_cmp);
          memcpy(&am, small_host.data() + 16 * t + 4, 4);
          const float alpha = std::min(std::max(cfg.alpha, 0.05f), 0.95f);
          float qmax = bits == 4 ? 7.0f : 127.0f;
          const float act = (float)std::max((double)am, 1e-5);
          const float wmax = fmaxf(am, 1e-5f);
          const float smooth = fmaxf(powf(fmaxf(act, 1e-4f), alpha) / powf(wmax, 1.0f - alpha), 1e-4f);
          const float effq = fmaxf(wmax * smooth / qmax, 1e-6f);
          rc = cfb200_smoothquant_apply((const float*)sl.in, n, bits, smooth, effq, (float*)out, eng->s_cmp);
        }
        break;
      }
      case kHadamard: {
        cudaMemcpyAsync(out, sl.in, n * 4, cudaMemcpyDeviceToDevice, eng->s_cmp);
        rc = cfb200_fwht_cols((float*)out, (size_t)e.shape[0], (size_t)e.shape[1], std::max<size_t>(cfg.block_size, 2), &aux[t], eng->s_cmp);
        break;
      }
      case kPerChannel: rc = cfb200_quant_per_channel(sl.in, dd, (size_t)e.shape[0], n / (size_t)e.shape[0], bits, (int8_t*)out, (float*)(out + p.pieces[1].offset), eng->s_cmp); break;
      case kInt4: rc = cfb200_quant_int4_asym(sl.in, dd, n, cfg.group_size, out, (uint16_t*)(out + p.pieces[1].offset), out + p.pieces[2].offset, eng->s_cmp); break;
      case kNf4: {
        const size_t blk = cfg.block_size == 32 ? 64 : cfg.block_size;
        rc = cfb200_quant_nf4(sl.in, dd, n, blk, 256, out, out + p.pieces[1].offset, (float*)(out + p.pieces[2].offset), sl.scratch, sl.scratch_cap, eng->s_cmp);
        break;
      }
      case kE4m3: rc = cfb200_cast_e4m3_tensor(sl.in, dd, n, out, sm, eng->s_cmp); break;
      default: break;
    }
    if (rc) { *err = std::string("device pass failed on `") + e.name + "`: " + cfb200_last_error(); ok_all = false; break; }
    cudaEvent_t e_c = new_event();
    cudaEventRecord(e_c, eng->s_cmp);
    cudaStreamWaitEvent(eng->s_d2h, e_c, 0);
    for (const OutPiece& pc : p.pieces) {
      outs[t].push_back(HostBuffer::owned(pc.bytes));
      if (pc.bytes) ok_all = ok_all && ck(cudaMemcpyAsync(outs[t].back().data(), out + pc.offset, pc.bytes, cudaMemcpyDeviceToHost, eng->s_d2h), err, "D2H copy");
    }
    cudaEventRecord(sl.free_ev, eng->s_d2h);
    sl.used = true;
  }
  if (ok_all) {
    cudaStreamWaitEvent(eng->s_d2h, evs.empty() ? nullptr : evs.back(), 0);
    ok_all = ck(cudaMemcpyAsync(small_host.data(), eng->small, todo.size() * 16, cudaMemcpyDeviceToHost, eng->s_d2h), err, "D2H copy (scalars)");
  }
  cudaStreamSynchronize(eng->s_h2d);
  cudaStreamSynchronize(eng->s_cmp);
  const cudaError_t fin = cudaStreamSynchronize(eng->s_d2h);
  for (cudaEvent_t ev : evs) cudaEventDestroy(ev);
  if (!ok_all) return false;
  if (!ck(fin, err, "device pipeline")) return false;
  if (kind == kWeight) {  // the cooperative A1 launch reports an expired wait through a device flag, not a return code
    int32_t flag = 0;
    if (cfb200_quant_sym_status(&flag) != 0) { *err = std::string("device status: ") + cfb200_last_error(); return false; }
    if (flag != 0) { *err = "the quantize kernel gave up a bounded wait on this device: results are incomplete"; return false; }
  }

  // ---- publish results into the store ----
  for (size_t t = 0; t < todo.size(); ++t) {
    TensorEntry& e = store.at(todo[t]);
    const Plan& p = plans[t];
    float sm[4];
    memcpy(sm, small_host.data() + 16 * t, 16);
    const std::string base = e.name;
    const DType orig = e.dtype;
    for (size_t k = 1; k < p.pieces.size(); ++k) {
      TensorEntry x;
      x.name = base + p.pieces[k].suffix;
      x.dtype = p.pieces[k].dtype;
      x.shape = p.pieces[k].shape;
      x.data = std::move(outs[t][k]);
      store.insert(std::move(x));
    }
    TensorEntry& ee = *store.get(base);
    ee.data = std::move(outs[t][0]);
    ee.ext_path.clear();  // the result replaces the file slice
    ee.ext_offset = ee.ext_length = 0;
    ee.dtype = p.pieces[0].dtype;
    switch (kind) {
      case kWeight: case kE4m3:
        ee.quantized = true; ee.scale = sm[0]; ee.zero_point = 0; ee.expressed = orig;
        if (kind == kE4m3) ee.attrs["castforge.fp8_format"] = "fp8_e4m3fn";
        break;
      case kGroup:
        ee.attrs["castforge.quant_scheme"] = awq ? "awq_groupwise" : "gptq_groupwise";
        ee.attrs["castforge.quant_bits"] = std::to_string(bits == 4 ? 4 : 8);
        ee.attrs["castforge.group_size"] = std::to_string(std::max<size_t>(cfg.group_size, 2));
        ee.attrs["castforge.num_groups"] = std::to_string((ee.num_elements() + std::max<size_t>(cfg.group_size, 2) - 1) / std::max<size_t>(cfg.group_size, 2));
        if (awq) ee.attrs["castforge.awq_salient_channels"] = std::to_string(aux[t]);
        break;
      case kFp8: {
        std::string f = cfg.format;
        std::transform(f.begin(), f.end(), f.begin(), ::tolower);
        ee.attrs["castforge.fp8_format"] = f == "e5m2" ? "fp8_e5m2" : "fp8_e4m3";
        ee.attrs["castforge.mxfp8"] = cfg.mxfp8 ? "true" : "false";
        break;
      }
      case kFp4: ee.attrs["castforge.quant_scheme"] = s == "nvfp4" ? "nvfp4" : "mxfp4"; ee.attrs["castforge.num_blocks"] = std::to_string(aux[t]); break;
      case kQat: ee.attrs["castforge.qat_ste"] = "true"; ee.attrs["castforge.qat_bits"] = std::to_string(bits == 4 ? 4 : 8); ee.attrs["castforge.qat_scale"] = format_f32_shortest(sm[0]); break;
      case kSmooth: ee.attrs["castforge.quant_scheme"] = "smoothquant"; ee.attrs["castforge.quant_bits"] = std::to_string(bits == 4 ? 4 : 8); break;
      case kHadamard: ee.attrs["castforge.hadamard_rotated"] = "true"; ee.attrs["castforge.hadamard_block"] = std::to_string(aux[t]); break;
      case kPerChannel: ee.attrs["castforge.quant_scheme"] = "per_channel"; ee.expressed = orig; break;
      case kInt4: ee.attrs["castforge.quant_scheme"] = "int4_asym"; ee.attrs["castforge.group_size"] = std::to_string(cfg.group_size); ee.expressed = orig; break;
      case kNf4: ee.attrs["castforge.quant_scheme"] = "nf4"; ee.expressed = orig; break;
      default: break;
    }
    res->ops_modified += 1;
    if (kind == kWeight) res->ops_created += 1;  // the uniform_dequantize the reference adds (schemes.rs:406-440)
  }
  res->changed = res->ops_modified > 0;
  return true;
}

}  // namespace host
}  // namespace cfb
