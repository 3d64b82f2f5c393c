// Read-only safetensors access: mmaps `model.safetensors` (or every shard listed in
// `model.safetensors.index.json`) and exposes tensors by name.  The reference does the same
// through candle's VarBuilder (backends/candle/src/lib.rs:170-215,275-280).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace tei {

enum class StDType { F32, F16, BF16, F64, I64, I32, U8, BOOL, OTHER };

struct StTensor {
  StDType dtype = StDType::OTHER;
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;  // points into the mapping
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

class SafeTensors {
 public:
  SafeTensors() = default;
  ~SafeTensors();
  SafeTensors(const SafeTensors&) = delete;
  SafeTensors& operator=(const SafeTensors&) = delete;

  // Opens the weights of a model directory.  Throws std::runtime_error (message starts with
  // "weights not found" when no safetensors file exists).
  void open_dir(const std::string& model_dir);
  void open_file(const std::string& path);

  bool contains(const std::string& name) const { return tensors_.count(name) != 0; }
  const StTensor& get(const std::string& name) const;
  const std::map<std::string, StTensor>& all() const { return tensors_; }

 private:
  struct Mapping {
    void* addr;
    size_t len;
  };
  std::vector<Mapping> maps_;
  std::map<std::string, StTensor> tensors_;
};

}  // namespace tei
