// Memory and stream services of the native runtime. The implementation (tensor.cpp) is the one
// translation unit that includes libtorch: buffers are ATen tensors (the caching CUDA allocator,
// the pinned-host allocator), streams are c10 CUDA streams. Everything else in the runtime sees
// raw pointers, which is also what the kernel library takes.
//
// The reference's counterpart is its own vt:: tensor runtime (include/vt/tensor.h, src/vt/cuda/
// cuda_backend.cu); here that layer is PyTorch's C++ frontend.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

namespace b200::rt {

struct Device {
  bool cuda = false;
  int index = 0;
  static Device parse(const std::string& s);   // "cpu", "cuda", "cuda:3"
  std::string str() const;
};

// Owning handle of `nbytes` of memory on a device (or pinned host memory).
class Buffer {
 public:
  Buffer() = default;
  void* data() const { return data_; }
  template <class T> T* as() const { return static_cast<T*>(data_); }
  size_t nbytes() const { return nbytes_; }
  explicit operator bool() const { return data_ != nullptr; }

 private:
  friend Buffer alloc(size_t, Device, bool);
  friend Buffer alloc_pinned(size_t);
  std::shared_ptr<void> keep_;   // the ATen tensor that owns the memory
  void* data_ = nullptr;
  size_t nbytes_ = 0;
};

bool cuda_available();
void set_device(Device d);
Buffer alloc(size_t nbytes, Device d, bool zero = false);
Buffer alloc_pinned(size_t nbytes);            // page-locked host memory (plain host memory without CUDA)
void* current_stream(Device d);                // cudaStream_t of the device's current stream; nullptr on CPU
// dst <- src, `n` bytes; asynchronous on the device's current stream when either side is a GPU.
void copy(void* dst, Device dst_dev, const void* src, Device src_dev, size_t n);
void memset_zero(void* p, Device d, size_t n);
void synchronize(Device d);                    // waits for the current stream
void free_and_total_memory(Device d, size_t* free_bytes, size_t* total_bytes);

// CUDA events for the asynchronous device->host copy of sampled ids.
class Event {
 public:
  explicit Event(Device d);
  ~Event();
  void record();          // on the device's current stream
  void synchronize();
 private:
  void* ev_ = nullptr;
  int stream_dev_ = 0;
};

}  // namespace b200::rt
