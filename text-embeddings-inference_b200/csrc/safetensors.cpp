#include "safetensors.h"

#include "json.h"

#include <cstring>
#include <fcntl.h>
#include <fstream>
#include <set>
#include <sstream>
#include <stdexcept>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace tei {
namespace {

bool file_exists(const std::string& p) {
  struct stat st;
  return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

StDType parse_dtype(const std::string& s, size_t* elem) {
  if (s == "F32") { *elem = 4; return StDType::F32; }
  if (s == "F16") { *elem = 2; return StDType::F16; }
  if (s == "BF16") { *elem = 2; return StDType::BF16; }
  if (s == "F64") { *elem = 8; return StDType::F64; }
  if (s == "I64") { *elem = 8; return StDType::I64; }
  if (s == "I32") { *elem = 4; return StDType::I32; }
  if (s == "U8") { *elem = 1; return StDType::U8; }
  if (s == "BOOL") { *elem = 1; return StDType::BOOL; }
  *elem = 0;
  return StDType::OTHER;
}

}  // namespace

SafeTensors::~SafeTensors() {
  for (auto& m : maps_) ::munmap(m.addr, m.len);
}

void SafeTensors::open_file(const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error("weights not found: cannot open " + path);
  struct stat st;
  if (::fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    throw std::runtime_error("safetensors: file too small: " + path);
  }
  const size_t len = static_cast<size_t>(st.st_size);
  void* addr = ::mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (addr == MAP_FAILED) throw std::runtime_error("safetensors: mmap failed for " + path);
  maps_.push_back({addr, len});
  const uint8_t* base = static_cast<const uint8_t*>(addr);
  uint64_t hlen = 0;
  std::memcpy(&hlen, base, 8);  // little-endian header length
  if (hlen > len - 8) throw std::runtime_error("safetensors: corrupt header length in " + path);
  const Json header = Json::parse(reinterpret_cast<const char*>(base + 8), static_cast<size_t>(hlen));
  if (!header.is_object()) throw std::runtime_error("safetensors: header is not an object");
  const uint8_t* data0 = base + 8 + hlen;
  const size_t data_len = len - 8 - static_cast<size_t>(hlen);
  for (const auto& kv : header.members()) {
    if (kv.first == "__metadata__") continue;
    const Json& e = kv.second;
    StTensor t;
    size_t elem = 0;
    t.dtype = parse_dtype(e["dtype"].as_string(), &elem);
    for (const Json& d : e["shape"].items()) t.shape.push_back(d.as_int());
    const int64_t b = e["data_offsets"].at(0).as_int();
    const int64_t en = e["data_offsets"].at(1).as_int();
    if (b < 0 || en < b || static_cast<size_t>(en) > data_len) {
      throw std::runtime_error("safetensors: bad data_offsets for " + kv.first);
    }
    t.data = data0 + b;
    t.nbytes = static_cast<size_t>(en - b);
    if (elem != 0 && static_cast<size_t>(t.numel()) * elem != t.nbytes) {
      throw std::runtime_error("safetensors: shape/size mismatch for " + kv.first);
    }
    tensors_[kv.first] = t;
  }
}

void SafeTensors::open_dir(const std::string& model_dir) {
  const std::string single = model_dir + "/model.safetensors";
  const std::string index = model_dir + "/model.safetensors.index.json";
  if (file_exists(single)) {
    open_file(single);
    return;
  }
  if (file_exists(index)) {
    std::ifstream in(index);
    std::stringstream ss;
    ss << in.rdbuf();
    const Json idx = Json::parse(ss.str());
    std::set<std::string> shards;
    for (const auto& kv : idx["weight_map"].members()) shards.insert(kv.second.as_string());
    if (shards.empty()) throw std::runtime_error("weights not found: empty weight_map in " + index);
    for (const auto& s : shards) open_file(model_dir + "/" + s);
    return;
  }
  throw std::runtime_error("weights not found: no model.safetensors under " + model_dir);
}

const StTensor& SafeTensors::get(const std::string& name) const {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) throw std::runtime_error("cannot find tensor " + name);
  return it->second;
}

}  // namespace tei
