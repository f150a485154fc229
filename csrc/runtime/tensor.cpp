#include "runtime/tensor.h"

#include <ATen/ATen.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

namespace b200::rt {

Device Device::parse(const std::string& s) {
  Device d;
  if (s.rfind("cuda", 0) == 0) {
    d.cuda = true;
    auto c = s.find(':');
    d.index = c == std::string::npos ? 0 : std::stoi(s.substr(c + 1));
  } else if (s != "cpu" && !s.empty()) {
    throw std::invalid_argument("unknown device '" + s + "' (cpu, cuda, cuda:N)");
  }
  return d;
}
std::string Device::str() const { return cuda ? "cuda:" + std::to_string(index) : "cpu"; }

bool cuda_available() { return at::hasCUDA() && c10::cuda::device_count() > 0; }

void set_device(Device d) {
  if (d.cuda) c10::cuda::set_device((c10::DeviceIndex)d.index);
}

Buffer alloc(size_t nbytes, Device d, bool zero) {
  auto opt = at::TensorOptions().dtype(at::kByte).device(d.cuda ? at::Device(at::kCUDA, (c10::DeviceIndex)d.index)
                                                                : at::Device(at::kCPU));
  const int64_t n = (int64_t)(nbytes ? nbytes : 1);
  auto* t = new at::Tensor(zero ? at::zeros({n}, opt) : at::empty({n}, opt));
  Buffer b;
  b.keep_ = std::shared_ptr<void>(t, [](void* p) { delete static_cast<at::Tensor*>(p); });
  b.data_ = t->data_ptr();
  b.nbytes_ = nbytes;
  return b;
}

Buffer alloc_pinned(size_t nbytes) {
  auto opt = at::TensorOptions().dtype(at::kByte).device(at::kCPU).pinned_memory(cuda_available());
  const int64_t n = (int64_t)(nbytes ? nbytes : 1);
  auto* t = new at::Tensor(at::zeros({n}, opt));
  Buffer b;
  b.keep_ = std::shared_ptr<void>(t, [](void* p) { delete static_cast<at::Tensor*>(p); });
  b.data_ = t->data_ptr();
  b.nbytes_ = nbytes;
  return b;
}

void* current_stream(Device d) {
  if (!d.cuda) return nullptr;
  return (void*)c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)d.index).stream();
}

void copy(void* dst, Device dd, const void* src, Device sd, size_t n) {
  if (n == 0) return;
  if (!dd.cuda && !sd.cuda) {
    std::memmove(dst, src, n);
    return;
  }
  const Device g = dd.cuda ? dd : sd;
  cudaMemcpyKind kind = dd.cuda && sd.cuda ? cudaMemcpyDeviceToDevice
                        : dd.cuda          ? cudaMemcpyHostToDevice
                                           : cudaMemcpyDeviceToHost;
  if (cudaMemcpyAsync(dst, src, n, kind, (cudaStream_t)current_stream(g)) != cudaSuccess)
    throw std::runtime_error(std::string("cudaMemcpyAsync failed: ") + cudaGetErrorString(cudaGetLastError()));
}

void memset_zero(void* p, Device d, size_t n) {
  if (!d.cuda) {
    std::memset(p, 0, n);
    return;
  }
  if (cudaMemsetAsync(p, 0, n, (cudaStream_t)current_stream(d)) != cudaSuccess)
    throw std::runtime_error("cudaMemsetAsync failed");
}

void synchronize(Device d) {
  if (!d.cuda) return;
  if (cudaStreamSynchronize((cudaStream_t)current_stream(d)) != cudaSuccess)
    throw std::runtime_error(std::string("stream synchronisation failed: ") +
                             cudaGetErrorString(cudaGetLastError()));
}

void free_and_total_memory(Device d, size_t* f, size_t* t) {
  *f = *t = 0;
  if (!d.cuda) return;
  set_device(d);
  cudaMemGetInfo(f, t);
}

Event::Event(Device d) {
  if (d.cuda) {
    cudaEvent_t e;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess) ev_ = e;
    stream_dev_ = d.index;
  }
}
Event::~Event() {
  if (ev_) cudaEventDestroy((cudaEvent_t)ev_);
}
void Event::record() {
  if (ev_) cudaEventRecord((cudaEvent_t)ev_, c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)stream_dev_).stream());
}
void Event::synchronize() {
  if (ev_) cudaEventSynchronize((cudaEvent_t)ev_);
}

}  // namespace b200::rt
