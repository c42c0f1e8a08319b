// GGUF v2 / v3 reader for F32 and F16 tensors: the model-file format on the input side of the
// llama runner (reference: tools/llama-ash/src/gguf.rs:1-285).  The header is indexed once --
// scalar and string metadata kept, arrays (tokenizer tables) walked and dropped -- and tensor
// payloads are read on demand.  Host-only; no CUDA.
#pragma once
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

namespace ta {

constexpr uint32_t GGML_TYPE_F32 = 0, GGML_TYPE_F16 = 1;

struct GgufValue {
  enum Kind : uint8_t { U64, I64, F64, Bool, Str, Skipped } kind = Skipped;
  uint64_t u = 0;
  int64_t i = 0;
  double f = 0.0;
  bool b = false;
  std::string s;
};

struct GgufTensorInfo {
  std::vector<uint64_t> ne;   // dimensions as stored: ne[0] varies fastest
  uint32_t ggml_type = 0;
  uint64_t offset = 0;        // bytes from the start of the data section
  uint64_t element_count() const {
    uint64_t n = 1;
    for (uint64_t d : ne) n *= d;
    return n;
  }
};

class GgufFile {
 public:
  explicit GgufFile(const std::string &path);   // fails (ta::fail) on a malformed file
  ~GgufFile();
  GgufFile(const GgufFile &) = delete;
  GgufFile &operator=(const GgufFile &) = delete;

  const GgufValue *find(const std::string &key) const;
  uint64_t require_u64(const std::string &key) const;          // unsigned, or a non-negative signed value
  bool get_u64(const std::string &key, uint64_t *out) const;
  double f64_or(const std::string &key, double fallback) const;
  bool has_tensor(const std::string &name) const { return tensors_.count(name) != 0; }
  const GgufTensorInfo &info(const std::string &name) const;   // fails when absent

  // Tensor payload as f32 (f16 widened exactly) or as f16 bits (f32 rounded to nearest even).
  std::vector<float> read_f32(const std::string &name);
  std::vector<uint16_t> read_f16_bits(const std::string &name);

  uint32_t version() const { return version_; }
  uint64_t data_start() const { return data_start_; }
  size_t tensor_count() const { return tensors_.size(); }

 private:
  void read_raw(const GgufTensorInfo &info, const std::string &name, std::vector<uint8_t> *bytes);
  std::string path_;
  FILE *fp_ = nullptr;
  uint32_t version_ = 0;
  uint64_t data_start_ = 0, file_size_ = 0;
  std::map<std::string, GgufValue> meta_;
  std::map<std::string, GgufTensorInfo> tensors_;
};

}  // namespace ta
