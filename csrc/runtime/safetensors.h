// Read-only view of safetensors files (memory-mapped): 8-byte little-endian header length, a
// JSON header {name: {dtype, shape, data_offsets}}, then the raw tensor bytes. A model
// directory may hold one file or numbered shards.
//
// Reference: src/vllm/model_executor/model_loader/safetensors.cpp (mmap'd shards, the same format).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b200::rt {

struct TensorView {
  std::string dtype;              // "BF16", "F16", "F32", "F8_E4M3", "U8", "I32", "I64"
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

class SafetensorsDir {
 public:
  // Opens every *.safetensors file of `dir` (or the single file `dir` names).
  explicit SafetensorsDir(const std::string& dir);
  ~SafetensorsDir();
  SafetensorsDir(const SafetensorsDir&) = delete;
  SafetensorsDir& operator=(const SafetensorsDir&) = delete;
  bool has(const std::string& name) const { return tensors_.count(name) > 0; }
  const TensorView& get(const std::string& name) const;   // throws std::runtime_error if absent
  const std::map<std::string, TensorView>& all() const { return tensors_; }

 private:
  struct Mapping {
    void* base = nullptr;
    size_t size = 0;
  };
  void open_file(const std::string& path);
  std::vector<Mapping> maps_;
  std::map<std::string, TensorView> tensors_;
};

}  // namespace b200::rt
