// GGUF v2 / v3 reader (see gguf.hpp).  Layout per the public GGUF specification:
//   "GGUF" u32 version u64 n_tensors u64 n_kv, then n_kv (string key, u32 type, value),
//   then n_tensors (string name, u32 n_dims, u64 ne[n_dims], u32 ggml type, u64 offset),
//   then padding to general.alignment (default 32) and the tensor data.
// Limits and messages follow tools/llama-ash/src/gguf.rs (strings <= 2^24 bytes, counts
// <= 2^20, 1..4 dims, only F32 / F16 payloads).
#include "gguf.hpp"

#include <cstring>

#include "ta_core.hpp"

namespace ta {

namespace {

struct Cursor {
  FILE *fp;
  const std::string &path;
  void read(void *dst, size_t n) {
    if (n && fread(dst, 1, n, fp) != n) fail("unexpected end of GGUF file %s", path.c_str());
  }
  template <typename T>
  T scalar() {
    T v;
    read(&v, sizeof(T));   // GGUF is little-endian, as is every host this library builds for
    return v;
  }
  std::string str() {
    const uint64_t len = scalar<uint64_t>();
    if (len > (1ull << 24)) fail("GGUF string length %llu is implausible", (unsigned long long)len);
    std::string s(len, '\0');
    read(s.data(), len);
    return s;
  }
  void skip(uint64_t n) {
    if (n > (1ull << 62) || fseeko(fp, (off_t)n, SEEK_CUR) != 0) fail("GGUF seek past %llu bytes failed", (unsigned long long)n);
  }
  uint64_t tell() { return (uint64_t)ftello(fp); }
};

// byte width of a fixed-size metadata type, 0 for strings / arrays / unknown
uint64_t scalar_width(uint32_t ty) {
  switch (ty) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}

GgufValue read_value(Cursor &c, uint32_t ty) {
  GgufValue v;
  switch (ty) {
    case 0: v.kind = GgufValue::U64; v.u = c.scalar<uint8_t>(); break;
    case 1: v.kind = GgufValue::I64; v.i = c.scalar<int8_t>(); break;
    case 2: v.kind = GgufValue::U64; v.u = c.scalar<uint16_t>(); break;
    case 3: v.kind = GgufValue::I64; v.i = c.scalar<int16_t>(); break;
    case 4: v.kind = GgufValue::U64; v.u = c.scalar<uint32_t>(); break;
    case 5: v.kind = GgufValue::I64; v.i = c.scalar<int32_t>(); break;
    case 6: v.kind = GgufValue::F64; v.f = (double)c.scalar<float>(); break;
    case 7: v.kind = GgufValue::Bool; v.b = c.scalar<uint8_t>() != 0; break;
    case 8: v.kind = GgufValue::Str; v.s = c.str(); break;
    case 9: {   // array: element type, count, payload -- walked, not kept
      const uint32_t elem = c.scalar<uint32_t>();
      const uint64_t count = c.scalar<uint64_t>();
      if (const uint64_t w = scalar_width(elem)) {
        uint64_t bytes;
        if (__builtin_mul_overflow(w, count, &bytes)) fail("GGUF array size overflow");
        c.skip(bytes);
      } else if (elem == 8) {
        for (uint64_t i = 0; i < count; ++i) c.skip(c.scalar<uint64_t>());
      } else {
        fail("GGUF nested/unknown array element type %u", elem);
      }
      v.kind = GgufValue::Skipped;
      break;
    }
    case 10: v.kind = GgufValue::U64; v.u = c.scalar<uint64_t>(); break;
    case 11: v.kind = GgufValue::I64; v.i = c.scalar<int64_t>(); break;
    case 12: v.kind = GgufValue::F64; v.f = c.scalar<double>(); break;
    default: fail("unknown GGUF metadata type %u", ty);
  }
  return v;
}

}  // namespace

GgufFile::GgufFile(const std::string &path) : path_(path) {
  fp_ = fopen(path.c_str(), "rb");
  if (!fp_) fail("opening %s: %s", path.c_str(), strerror(errno));
  try {
    fseeko(fp_, 0, SEEK_END);
    file_size_ = (uint64_t)ftello(fp_);
    fseeko(fp_, 0, SEEK_SET);
    Cursor c{fp_, path_};
    char magic[4];
    c.read(magic, 4);
    if (memcmp(magic, "GGUF", 4) != 0) fail("not a GGUF file (bad magic) : %s", path.c_str());
    version_ = c.scalar<uint32_t>();
    if (version_ != 2 && version_ != 3) fail("unsupported GGUF version %u (want 2 or 3)", version_);
    const uint64_t n_tensors = c.scalar<uint64_t>(), n_kv = c.scalar<uint64_t>();
    if (n_tensors > (1ull << 20) || n_kv > (1ull << 20))
      fail("implausible GGUF header (tensors %llu, kvs %llu)", (unsigned long long)n_tensors, (unsigned long long)n_kv);
    for (uint64_t i = 0; i < n_kv; ++i) {
      std::string key = c.str();
      const uint32_t ty = c.scalar<uint32_t>();
      meta_[key] = read_value(c, ty);
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
      std::string name = c.str();
      const uint32_t n_dims = c.scalar<uint32_t>();
      if (n_dims == 0 || n_dims > 4) fail("tensor %s: bad n_dims %u", name.c_str(), n_dims);
      GgufTensorInfo info;
      for (uint32_t d = 0; d < n_dims; ++d) info.ne.push_back(c.scalar<uint64_t>());
      info.ggml_type = c.scalar<uint32_t>();
      info.offset = c.scalar<uint64_t>();
      tensors_[name] = std::move(info);
    }
    uint64_t alignment = 32;
    get_u64("general.alignment", &alignment);
    if (alignment == 0 || (alignment & (alignment - 1))) fail("bad general.alignment %llu", (unsigned long long)alignment);
    const uint64_t here = c.tell();
    data_start_ = (here + alignment - 1) / alignment * alignment;
  } catch (...) {
    fclose(fp_);
    fp_ = nullptr;
    throw;
  }
}

GgufFile::~GgufFile() {
  if (fp_) fclose(fp_);
}

const GgufValue *GgufFile::find(const std::string &key) const {
  auto it = meta_.find(key);
  return it == meta_.end() ? nullptr : &it->second;
}

bool GgufFile::get_u64(const std::string &key, uint64_t *out) const {
  const GgufValue *v = find(key);
  if (!v) return false;
  if (v->kind == GgufValue::U64) { *out = v->u; return true; }
  if (v->kind == GgufValue::I64 && v->i >= 0) { *out = (uint64_t)v->i; return true; }
  return false;
}

uint64_t GgufFile::require_u64(const std::string &key) const {
  uint64_t v = 0;
  if (!get_u64(key, &v)) fail("GGUF metadata missing integer key %s", key.c_str());
  return v;
}

double GgufFile::f64_or(const std::string &key, double fallback) const {
  const GgufValue *v = find(key);
  if (!v) return fallback;
  switch (v->kind) {
    case GgufValue::F64: return v->f;
    case GgufValue::U64: return (double)v->u;
    case GgufValue::I64: return (double)v->i;
    default: return fallback;
  }
}

const GgufTensorInfo &GgufFile::info(const std::string &name) const {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) fail("GGUF tensor %s not found", name.c_str());
  return it->second;
}

void GgufFile::read_raw(const GgufTensorInfo &info, const std::string &name, std::vector<uint8_t> *bytes) {
  if (info.ggml_type != GGML_TYPE_F32 && info.ggml_type != GGML_TYPE_F16)
    fail("tensor %s has ggml type %u; only F32/F16 are supported -- use an f16 GGUF (e.g. *.f16.gguf), not a quantized one",
         name.c_str(), info.ggml_type);
  const uint64_t elem = info.ggml_type == GGML_TYPE_F32 ? 4 : 2;
  uint64_t n = info.element_count(), total;
  if (__builtin_mul_overflow(n, elem, &total) || data_start_ + info.offset + total > file_size_)
    fail("tensor %s: payload of %llu elements runs past the end of the file", name.c_str(), (unsigned long long)n);
  bytes->resize(total);
  if (fseeko(fp_, (off_t)(data_start_ + info.offset), SEEK_SET) != 0) fail("tensor %s: seek failed", name.c_str());
  Cursor c{fp_, path_};
  c.read(bytes->data(), total);
}

std::vector<float> GgufFile::read_f32(const std::string &name) {
  const GgufTensorInfo &ti = info(name);
  std::vector<uint8_t> raw;
  read_raw(ti, name, &raw);
  const size_t n = (size_t)ti.element_count();
  std::vector<float> out(n);
  if (ti.ggml_type == GGML_TYPE_F32) {
    memcpy(out.data(), raw.data(), n * 4);
  } else {
    const uint16_t *h = reinterpret_cast<const uint16_t *>(raw.data());
    for (size_t i = 0; i < n; ++i) out[i] = f16_bits_to_f32(h[i]);
  }
  return out;
}

std::vector<uint16_t> GgufFile::read_f16_bits(const std::string &name) {
  const GgufTensorInfo &ti = info(name);
  std::vector<uint8_t> raw;
  read_raw(ti, name, &raw);
  const size_t n = (size_t)ti.element_count();
  std::vector<uint16_t> out(n);
  if (ti.ggml_type == GGML_TYPE_F16) {
    memcpy(out.data(), raw.data(), n * 2);
  } else {
    const float *f = reinterpret_cast<const float *>(raw.data());
    for (size_t i = 0; i < n; ++i) out[i] = f32_to_f16_bits(f[i]);
  }
  return out;
}

}  // namespace ta
