#include "runtime/safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <filesystem>
#include <stdexcept>

#include "util/json.h"

namespace fs = std::filesystem;

namespace b200::rt {

SafetensorsDir::SafetensorsDir(const std::string& dir) {
  std::vector<std::string> files;
  if (fs::is_regular_file(dir)) {
    files.push_back(dir);
  } else if (fs::is_directory(dir)) {
    for (auto& e : fs::directory_iterator(dir))
      if (e.is_regular_file() && e.path().extension() == ".safetensors") files.push_back(e.path().string());
  }
  if (files.empty()) throw std::runtime_error("no .safetensors file in " + dir);
  std::sort(files.begin(), files.end());
  for (auto& f : files) open_file(f);
}

SafetensorsDir::~SafetensorsDir() {
  for (auto& m : maps_)
    if (m.base) munmap(m.base, m.size);
}

void SafetensorsDir::open_file(const std::string& path) {
  int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error("cannot open " + path);
  struct stat st {};
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    throw std::runtime_error("not a safetensors file: " + path);
  }
  void* base = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (base == MAP_FAILED) throw std::runtime_error("mmap failed for " + path);
  maps_.push_back({base, (size_t)st.st_size});
  const uint8_t* p = static_cast<const uint8_t*>(base);
  uint64_t hlen = 0;
  std::memcpy(&hlen, p, 8);
  if (hlen == 0 || 8 + hlen > (uint64_t)st.st_size) throw std::runtime_error("corrupt safetensors header: " + path);
  Json header = Json::parse(std::string(reinterpret_cast<const char*>(p + 8), (size_t)hlen));
  const uint8_t* data0 = p + 8 + hlen;
  const size_t data_size = (size_t)st.st_size - 8 - (size_t)hlen;
  for (auto& kv : header.members()) {
    if (kv.first == "__metadata__") continue;
    TensorView t;
    t.dtype = kv.second["dtype"].as_string();
    for (auto& d : kv.second["shape"].items()) t.shape.push_back(d.as_int());
    const auto& off = kv.second["data_offsets"];
    const size_t a = (size_t)off[0].as_int(), b = (size_t)off[1].as_int();
    if (b < a || b > data_size) throw std::runtime_error("tensor " + kv.first + " lies outside " + path);
    t.data = data0 + a;
    t.nbytes = b - a;
    tensors_[kv.first] = std::move(t);
  }
}

const TensorView& SafetensorsDir::get(const std::string& name) const {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) throw std::runtime_error("checkpoint has no tensor named " + name);
  return it->second;
}

}  // namespace b200::rt
