// Host-side helpers shared by all kernel launchers: tensor-map encoding through the
// driver entry point, a per-device status word that kernels write when a bounded wait
// runs out, and device-property queries.
#include <cstdlib>
#include <cudaTypedefs.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
  });
  return fn;
}

bool encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype,
                    size_t elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                    uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool encode_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype,
                    size_t elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                    uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                    uint32_t b2, CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  if (!fn) return false;
  (void)elem_bytes;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Limit, in SM clock cycles, of the waits on another GPU's progress (the gather / scatter
// counters of the fused tensor-parallel kernels). Process-wide; kernels take it as a parameter at
// launch, so a change applies to the launches that follow.
static std::atomic<long long> g_peer_wait_cycles{kPeerWaitCycles};
long long peer_wait_cycles() { return g_peer_wait_cycles.load(std::memory_order_relaxed); }

int* device_status_word() {
  static std::mutex mu;
  static std::unordered_map<int, int*> words;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(dev);
  if (it != words.end()) return it->second;
  int* p = nullptr;
  if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, sizeof(int));
  words[dev] = p;
  return p;
}

}  // namespace b200

extern "C" {

int b200_num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && cached[dev]) return cached[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64) cached[dev] = n;
  return n;
}

// Reads (and clears) the status word of the current device. Synchronises the whole device
// first: a pageable cudaMemcpy alone orders only against the legacy default stream, and kernels
// launched on non-blocking streams could still be running their bounded waits.
int b200_read_status() {
  int* w = b200::device_status_word();
  if (!w) return -1;
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

void* b200_status_ptr() { return b200::device_status_word(); }

// Sets the peer-wait limit (cycles; <= 0 restores the default of about 9 s) and returns the
// previous one. Serving sets it from the step deadline; tests set it to about a millisecond to
// make a wait on a counter that nothing raises run out.
long long b200_set_peer_wait_cycles(long long cycles) {
  return b200::g_peer_wait_cycles.exchange(cycles > 0 ? cycles : b200::kPeerWaitCycles);
}

const char* b200_kernel_arch() { return "sm_100a"; }

}  // extern "C"
