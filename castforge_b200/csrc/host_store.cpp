// TensorStore, its SafeTensors layout and the pinned host-buffer pool.
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <mutex>
#include <thread>

#include "host.h"

namespace cfb {
namespace host {

const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "F32";
    case DType::F16: return "F16";
    case DType::BF16: return "BF16";
    case DType::I8: return "I8";
    case DType::I4: return "I8";  // 4-bit codes are stored one per byte (formats.rs:664-698)
    default: return "U8";
  }
}
size_t dtype_bytes(DType d) { return d == DType::F32 ? 4 : (d == DType::F16 || d == DType::BF16) ? 2 : 1; }

// ---- pinned buffer pool -----------------------------------------------------------------------
// cudaHostAlloc costs milliseconds per hundred MB, so released buffers are kept (by capacity) and
// handed out again; a pass that runs repeatedly allocates nothing after its first run.
namespace {
struct PoolItem { uint8_t* p; size_t cap; bool pinned; };
std::mutex g_pool_mu;
std::vector<PoolItem> g_pool;
size_t g_pool_bytes = 0;
constexpr size_t kPoolLimit = (size_t)48 << 30;

bool have_device() {
  static int state = -1;
  if (state < 0) {
    int n = 0;
    state = (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? 1 : 0;
    cudaGetLastError();
  }
  return state == 1;
}
}  // namespace

HostBuffer HostBuffer::owned(size_t bytes) {
  HostBuffer b;
  b.bytes_ = bytes;
  b.owned_ = true;
  if (bytes == 0) return b;
  {
    std::lock_guard<std::mutex> lk(g_pool_mu);
    int best = -1;
    for (size_t i = 0; i < g_pool.size(); ++i)
      if (g_pool[i].cap >= bytes && g_pool[i].cap <= bytes + bytes / 4 + 4096 && (best < 0 || g_pool[i].cap < g_pool[best].cap)) best = (int)i;
    if (best >= 0) {
      b.ptr_ = g_pool[best].p;
      b.cap_ = g_pool[best].cap;
      b.pinned_ = g_pool[best].pinned;
      g_pool_bytes -= b.cap_;
      g_pool.erase(g_pool.begin() + best);
      return b;
    }
  }
  b.cap_ = bytes;
  void* p = nullptr;
  if (have_device() && cudaHostAlloc(&p, bytes, cudaHostAllocDefault) == cudaSuccess) {
    b.pinned_ = true;
  } else {
    cudaGetLastError();
    p = malloc(bytes);
  }
  b.ptr_ = static_cast<uint8_t*>(p);
  return b;
}
HostBuffer HostBuffer::borrowed(void* p, size_t bytes) {
  HostBuffer b;
  b.ptr_ = static_cast<uint8_t*>(p);
  b.bytes_ = b.cap_ = bytes;
  return b;
}
void HostBuffer::release() {
  if (owned_ && ptr_) {
    std::lock_guard<std::mutex> lk(g_pool_mu);
    if (g_pool_bytes + cap_ <= kPoolLimit) {
      g_pool.push_back({ptr_, cap_, pinned_});
      g_pool_bytes += cap_;
    } else if (pinned_) {
      cudaFreeHost(ptr_);
    } else {
      free(ptr_);
    }
  }
  ptr_ = nullptr;
  bytes_ = cap_ = 0;
  owned_ = pinned_ = false;
}
HostBuffer::~HostBuffer() { release(); }
HostBuffer::HostBuffer(HostBuffer&& o) noexcept { *this = std::move(o); }
HostBuffer& HostBuffer::operator=(HostBuffer&& o) noexcept {
  if (this != &o) {
    release();
    ptr_ = o.ptr_; bytes_ = o.bytes_; cap_ = o.cap_; owned_ = o.owned_; pinned_ = o.pinned_;
    o.ptr_ = nullptr; o.bytes_ = o.cap_ = 0; o.owned_ = o.pinned_ = false;
  }
  return *this;
}

size_t TensorEntry::num_elements() const {
  size_t n = 1;
  for (int64_t d : shape) n *= (size_t)(d > 0 ? d : 1);
  return n;
}

bool read_file_slice_parallel(const std::string& path, uint64_t offset, uint64_t length, uint8_t* dst, std::string* err) {
  if (length == 0) return true;
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) { if (err) *err = "cannot open `" + path + "`"; return false; }
  const uint64_t kMinChunk = (uint64_t)2 << 20;
  unsigned hw = std::thread::hardware_concurrency();
  uint64_t parts = std::min<uint64_t>(std::max<uint64_t>(length / kMinChunk, 1), std::min<unsigned>(hw ? hw : 4, 16));
  const uint64_t per = (length + parts - 1) / parts;
  std::vector<int> ok(parts, 1);
  auto work = [&](uint64_t pi) {
    uint64_t lo = pi * per, hi = std::min(length, lo + per);
    while (lo < hi) {
      const ssize_t r = ::pread(fd, dst + lo, (size_t)(hi - lo), (off_t)(offset + lo));
      if (r <= 0) { ok[pi] = 0; return; }
      lo += (uint64_t)r;
    }
  };
  std::vector<std::thread> th;
  for (uint64_t pi = 1; pi < parts; ++pi) {
    try { th.emplace_back(work, pi); } catch (...) { work(pi); }  // no thread to be had: read that part here
  }
  work(0);
  for (auto& t : th) t.join();
  ::close(fd);
  for (int o : ok)
    if (!o) { if (err) *err = "short read from `" + path + "`"; return false; }
  return true;
}

bool TensorEntry::resolve(std::string* err) {
  if (!external()) return true;
  HostBuffer buf = HostBuffer::owned((size_t)ext_length);
  if (!read_file_slice_parallel(ext_path, ext_offset, ext_length, buf.data(), err)) return false;
  data = std::move(buf);
  ext_path.clear();
  ext_offset = ext_length = 0;
  return true;
}

TensorEntry* TensorStore::get(const std::string& name) {
  auto it = entries_.find(name);
  return it == entries_.end() ? nullptr : it->second.get();
}
TensorEntry& TensorStore::insert(TensorEntry e) {
  const std::string key = e.name;
  auto it = entries_.find(key);
  if (it == entries_.end()) {
    order_.push_back(key);
    it = entries_.emplace(key, std::unique_ptr<TensorEntry>(new TensorEntry())).first;
  }
  *it->second = std::move(e);
  return *it->second;
}

// ---- number formatting --------------------------------------------------------------------------
std::string format_f32_shortest(float v) {
  if (v != v || isinf(v)) return "null";  // serde_json prints non-finite floats as null
  if (v == 0.0f) return signbit(v) ? "-0.0" : "0.0";
  char buf[64];
  int prec = 1;
  for (; prec <= 9; ++prec) {
    snprintf(buf, sizeof buf, "%.*e", prec - 1, (double)v);
    if (strtof(buf, nullptr) == v) break;
  }
  // buf = d.ddde[+-]XX ; re-layout the way ryu does
  std::string s(buf);
  const size_t epos = s.find('e');
  std::string mant = s.substr(0, epos);
  const int exp10 = atoi(s.c_str() + epos + 1);
  bool neg = mant[0] == '-';
  if (neg) mant.erase(0, 1);
  std::string digits;
  for (char c : mant)
    if (c != '.') digits.push_back(c);
  while (digits.size() > 1 && digits.back() == '0') digits.pop_back();
  const int nd = (int)digits.size();
  const int kk = exp10 + 1;  // position of the decimal point relative to the first digit
  std::string out;
  if (nd <= kk && kk <= 16) {          // integer: digits, zeros, ".0"
    out = digits + std::string((size_t)(kk - nd), '0') + ".0";
  } else if (0 < kk && kk <= 16) {     // dd.ddd
    out = digits.substr(0, (size_t)kk) + "." + digits.substr((size_t)kk);
  } else if (-5 < kk && kk <= 0) {     // 0.00ddd
    out = "0." + std::string((size_t)(-kk), '0') + digits;
  } else {                             // d.ddde-7
    out = digits.substr(0, 1);
    if (nd > 1) out += "." + digits.substr(1);
    out += "e" + std::to_string(kk - 1);
  }
  return neg ? "-" + out : out;
}

std::string format_scale_string(float scale) {
  char buf[96];
  snprintf(buf, sizeof buf, "%.6f", (double)scale);
  std::string s(buf);
  while (!s.empty() && s.back() == '0') s.pop_back();
  while (!s.empty() && s.back() == '.') s.pop_back();
  if (s.find('.') == std::string::npos) s += ".0";
  return s;
}

static std::string json_escape(const std::string& s) {
  std::string o;
  for (unsigned char c : s) {
    if (c == '"') o += "\\\"";
    else if (c == '\\') o += "\\\\";
    else if (c == '\n') o += "\\n";
    else if (c == '\t') o += "\\t";
    else if (c == '\r') o += "\\r";
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
    else o.push_back((char)c);
  }
  return o;
}

// ---- SafeTensors writer (tensor_store.rs:427-554) -----------------------------------------------
std::string TensorStore::to_safetensors(std::string* err) const {
  std::string header = "{";
  size_t off = 0;
  bool first = true;
  for (const std::string& name : order_) {
    const TensorEntry& e = *entries_.at(name);
    const size_t nbytes = e.byte_size();
    if (!first) header += ",";
    first = false;
    header += "\"" + json_escape(name) + "\":{\"dtype\":\"" + dtype_name(e.dtype) + "\",\"shape\":[";
    for (size_t i = 0; i < e.shape.size(); ++i) {
      if (i) header += ",";
      header += std::to_string(e.shape[i] > 0 ? e.shape[i] : 1);
    }
    header += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + nbytes) + "]";
    if (e.quantized) header += ",\"scale\":" + format_f32_shortest(e.scale) + ",\"zero_point\":" + std::to_string(e.zero_point);
    header += "}";
    off += nbytes;
  }
  header += "}";
  while (header.size() % 8 != 0) header.push_back(' ');  // :542-546
  std::string out;
  out.reserve(8 + header.size() + off);
  const uint64_t hl = header.size();
  out.append(reinterpret_cast<const char*>(&hl), 8);  // little-endian host
  out += header;
  for (const std::string& name : order_) {
    const TensorEntry& e = *entries_.at(name);
    if (e.external()) {  // still on disk: copy the slice through
      const size_t at = out.size();
      out.resize(at + (size_t)e.ext_length);
      if (!read_file_slice_parallel(e.ext_path, e.ext_offset, e.ext_length, reinterpret_cast<uint8_t*>(&out[at]), err)) return std::string();
    } else {
      out.append(reinterpret_cast<const char*>(e.data.data()), e.data.size());
    }
  }
  return out;
}

// ---- minimal JSON reader for the header -----------------------------------------------------------
namespace {
struct JVal {
  enum Kind { Null, Num, Str, Arr, Obj, Bool } kind = Null;
  double num = 0;
  std::string str;
  std::vector<JVal> arr;
  std::vector<std::pair<std::string, JVal>> obj;
  const JVal* find(const char* k) const {
    for (auto& kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
};
struct JParser {
  const char* p;
  const char* end;
  std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool fail(const char* m) { if (err.empty()) err = m; return false; }
  bool str(std::string* out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'u': {
            if (p + 4 >= end) return fail("bad \\u escape");
            unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
            if (cp < 0x80) out->push_back((char)cp);
            else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
            else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
            p += 4;
            break;
          }
          default: out->push_back(*p);
        }
        ++p;
      } else {
        out->push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  bool value(JVal* v, int depth) {
    if (depth > 64) return fail("JSON nested too deeply");
    ws();
    if (p >= end) return fail("unexpected end of JSON");
    if (*p == '{') {
      v->kind = JVal::Obj;
      ++p; ws();
      if (p < end && *p == '}') { ++p; return true; }
      for (;;) {
        ws();
        std::string k;
        if (!str(&k)) return false;
        ws();
        if (p >= end || *p != ':') return fail("expected ':'");
        ++p;
        JVal c;
        if (!value(&c, depth + 1)) return false;
        v->obj.emplace_back(std::move(k), std::move(c));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (*p == '[') {
      v->kind = JVal::Arr;
      ++p; ws();
      if (p < end && *p == ']') { ++p; return true; }
      for (;;) {
        JVal c;
        if (!value(&c, depth + 1)) return false;
        v->arr.push_back(std::move(c));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (*p == '"') { v->kind = JVal::Str; return str(&v->str); }
    if (!strncmp(p, "null", std::min<size_t>(4, end - p))) { p += 4; v->kind = JVal::Null; return true; }
    if (!strncmp(p, "true", std::min<size_t>(4, end - p))) { p += 4; v->kind = JVal::Bool; v->num = 1; return true; }
    if (!strncmp(p, "false", std::min<size_t>(5, end - p))) { p += 5; v->kind = JVal::Bool; v->num = 0; return true; }
    char* e = nullptr;
    std::string tmp(p, std::min<size_t>(end - p, 64));
    v->num = strtod(tmp.c_str(), &e);
    if (e == tmp.c_str()) return fail("bad JSON value");
    p += (e - tmp.c_str());
    v->kind = JVal::Num;
    return true;
  }
};
}  // namespace

// ---- SafeTensors reader (tensor_store.rs:564-757), with its hardening: header <= 100 MiB, offsets
// inside the body, no overlapping ranges, element count matching the byte length -------------------
// Header walk shared by the eager and the lazy loader: validates every entry against `body_len` bytes of payload and
// hands (entry without data, start, stop) to `sink`.
template <class Sink>
static bool walk_safetensors_header(const char* hdr, size_t hl, uint64_t body_len, std::string* err, Sink sink) {
  auto bad = [&](const std::string& m) { if (err) *err = m; return false; };
  JParser jp{hdr, hdr + hl, ""};
  JVal root;
  if (!jp.value(&root, 0) || root.kind != JVal::Obj) return bad("Invalid safetensors JSON header: " + jp.err);
  std::vector<std::pair<size_t, size_t>> seen;
  for (auto& kv : root.obj) {
    if (kv.first == "__metadata__") continue;
    const JVal& h = kv.second;
    const JVal *jd = h.find("dtype"), *js = h.find("shape"), *jo = h.find("data_offsets");
    if (h.kind != JVal::Obj || !jd || jd->kind != JVal::Str || !js || js->kind != JVal::Arr || !jo || jo->kind != JVal::Arr || jo->arr.size() != 2)
      return bad("Malformed header entry for tensor `" + kv.first + "`");
    // data_offsets are `usize` in the reference's header struct: anything but a non-negative integer is a parse error there
    for (int k = 0; k < 2; ++k) {
      const JVal& o = jo->arr[k];
      if (o.kind != JVal::Num || !(o.num >= 0.0) || o.num > 9007199254740992.0 || o.num != (double)(uint64_t)o.num)
        return bad("Invalid data_offsets entry for tensor `" + kv.first + "`: expected a non-negative integer");
    }
    const size_t start = (size_t)jo->arr[0].num, stop = (size_t)jo->arr[1].num;
    if (stop > body_len || start > stop) return bad("Invalid data_offsets [" + std::to_string(start) + ", " + std::to_string(stop) + "] for tensor `" + kv.first + "`");
    if (start < stop)
      for (auto& r : seen)
        if (start < r.second && r.first < stop) return bad("Overlapping data_offsets [" + std::to_string(start) + ", " + std::to_string(stop) + "] for tensor `" + kv.first + "`");
    if (start < stop) seen.emplace_back(start, stop);
    TensorEntry e;
    e.name = kv.first;
    size_t elems = 1;
    for (auto& d : js->arr) {
      if (d.kind != JVal::Num || d.num < 0 || d.num > 9e15) return bad("Bad dimension for tensor `" + kv.first + "`");
      const int64_t di = (int64_t)d.num;
      e.shape.push_back(di);
      const size_t f = (size_t)(di > 0 ? di : 1);
      if (elems > ((size_t)1 << 40) / f) return bad("Tensor `" + kv.first + "` exceeds max element limit");
      elems *= f;
    }
    const std::string& dt = jd->str;
    if (dt == "F32") e.dtype = DType::F32;
    else if (dt == "F16") e.dtype = DType::F16;
    else if (dt == "BF16") e.dtype = DType::BF16;
    else if (dt == "I8") e.dtype = DType::I8;
    else e.dtype = DType::U8;  // I64, I32, F64, BOOL, ...: kept as the raw bytes of the slice (tensor_store.rs:742-750)
    const size_t nbytes = stop - start;
    // Stricter than the reference on purpose: it only asks for a multiple of the element size, but the passes here
    // copy num_elements() * size bytes of a float / I8 entry to the device, so the two must agree.
    if (e.dtype != DType::U8 && nbytes != elems * dtype_bytes(e.dtype))
      return bad("Byte length " + std::to_string(nbytes) + " does not match shape of tensor `" + kv.first + "`");
    if (const JVal* sc = h.find("scale")) {
      if (sc->kind == JVal::Num) { e.quantized = true; e.scale = (float)sc->num; }
    }
    if (const JVal* zp = h.find("zero_point")) {
      if (zp->kind == JVal::Num) { e.quantized = true; e.zero_point = (int64_t)zp->num; }
    }
    sink(std::move(e), start, stop);
  }
  return true;
}

bool TensorStore::load_safetensors(const uint8_t* bytes, size_t n, std::string* err) {
  auto bad = [&](const std::string& m) { if (err) *err = m; return false; };
  if (n < 8) return bad("Safetensors buffer shorter than 8-byte header length");
  uint64_t hl;
  memcpy(&hl, bytes, 8);
  if (hl > (uint64_t)100 * 1024 * 1024) return bad("Safetensors header length " + std::to_string(hl) + " exceeds 100 MiB limit");
  if (n < 8 + hl) return bad("Safetensors buffer truncated inside JSON header");
  const uint8_t* body = bytes + 8 + hl;
  return walk_safetensors_header(reinterpret_cast<const char*>(bytes + 8), (size_t)hl, n - 8 - hl, err, [&](TensorEntry e, size_t start, size_t stop) {
    const size_t nbytes = stop - start;
    e.data = HostBuffer::owned(nbytes);
    if (nbytes) memcpy(e.data.data(), body + start, nbytes);
    insert(std::move(e));
  });
}

long TensorStore::load_safetensors_lazy_file(const std::string& path, std::string* err) {
  auto bad = [&](const std::string& m) { if (err) *err = m; return -1L; };
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return bad("cannot open `" + path + "`");
  struct stat stt;
  if (fstat(fileno(f), &stt) != 0) { fclose(f); return bad("cannot stat `" + path + "`"); }
  const uint64_t file_len = (uint64_t)stt.st_size;
  uint64_t hl = 0;
  if (file_len < 8 || fread(&hl, 1, 8, f) != 8) { fclose(f); return bad("Safetensors file shorter than 8-byte header"); }
  if (hl > (uint64_t)100 * 1024 * 1024 || 8 + hl > file_len) { fclose(f); return bad("Invalid or truncated Safetensors header length"); }
  std::string hdr((size_t)hl, '\0');
  const bool got = fread(&hdr[0], 1, (size_t)hl, f) == (size_t)hl;
  fclose(f);
  if (!got) return bad("Invalid or truncated Safetensors header length");
  const uint64_t data_base = 8 + hl;
  long count = 0;
  if (!walk_safetensors_header(hdr.data(), hdr.size(), file_len - data_base, err, [&](TensorEntry e, size_t start, size_t stop) {
        if (stop > start) {
          e.ext_path = path;
          e.ext_offset = data_base + start;
          e.ext_length = stop - start;
        }
        insert(std::move(e));
        ++count;
      }))
    return -1;
  return count;
}

}  // namespace host
}  // namespace cfb
