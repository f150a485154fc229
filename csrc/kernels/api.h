// C entry points of the sm_100a kernel library. Every launcher takes raw device pointers
// and the stream to launch on, returns 0 on success and a negative code on a rejected
// argument (-1 shape/alignment, -2 launch failure, -3 tensor-map encode failure,
// -4 size beyond a stated maximum). No launcher synchronises the device.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int b200_num_sms();
int b200_read_status();
void* b200_status_ptr();
const char* b200_kernel_arch();

// C[M,N] = A[M,K] * W[N,K]^T (+bias[N]) (+residual[M,N]); bf16 in, bf16 or f32 out.
// force_path: 0 auto, 1 tiled kernel, 2 swap-AB split-K kernel, 3 BN=128, 4 BN=256.
int b200_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                   int out_f32, const void* bias, const void* residual, int ldr, int M, int N,
                   int K, void* workspace, size_t ws_bytes, int force_path, cudaStream_t stream);

// Tensor-parallel prologue / epilogue of a GEMM (see gemm_bf16.cu and tp_fused.cu).
typedef struct B200TpGemm {
  int world, rank, rows_per_rank;
  int scatter;                 // 1: epilogue scatters bf16 partial rows to their owner rank
  int gather;                  // 1: producer waits for gathered rows before loading A
  void* peer_recv[8];          // receive buffers [2][world][rows_per_rank][N], one per rank
  void* peer_rs_flags[8];      // arrival counters [2][rows_per_rank / 32], one per rank
  long long recv_parity_stride;
  int rs_flag_parity_stride;
  const void* a_alt;           // gather: the parity-1 copy of A (A itself is the parity-0 copy)
  const void* ag_flags;        // local gather counters [2][groups]
  int ag_flag_parity_stride;
  const void* op_counter;      // local device word, bumped by b200_tp_reduce_norm_gather
  int out_f32;                 // gather mode: fp32 output (lm_head)
  int scatter_splits;          // scatter mode, M <= 256: k-splits, each its own source slot
  int act_fuse;                // gather mode, M > 256: 0, or activation kind + 1 for the gated
                               // epilogue (out[M, N / 2] = act(gate) * up, W rows interleaved)
} B200TpGemm;

int b200_gemm_bf16_tp(const void* A, int lda, const void* W, int ldw, void* out, int ldo, int M,
                      int N, int K, const B200TpGemm* tp, int* expected_rs, cudaStream_t stream);

// ---- small-M GEMM that allocates nothing ------------------------------------------------
// This entry point has no counterpart in the reference project. It exists for callers that
// need a decode-sized GEMM (M <= 256) but may not allocate at that point: a plug-in inside
// another runtime's callback, a thread kept away from the framework's caching allocator, a
// plain C host without torch. out[M,N] (bf16, row stride ldo) = A[M,K] * W[N,K]^T, the same
// split-K kernels as b200_gemm_bf16, with the fp32 partial sums kept in an array that is part
// of the module image (B200_GEMM_STATIC_SCRATCH_BYTES per device) instead of a workspace.
//   * All calls on a device share that array: calls that can overlap in time race. Serialise.
//   * Nothing in the array needs clearing between calls.
//   * The first call on a device resolves the array's address (cudaGetSymbolAddress) and sets
//     a kernel attribute; make it before any stream capture on that device.
//   * Refused with -4 when M > 256 or 2*M*N*4 bytes exceed the array; -1 for misaligned
//     arguments; b200_gemm_bf16_smallm_static_error() names the reason (thread-local).
//   * b200_gemm_bf16_smallm_static_status() copies out this path's own sticky error word
//     (non-zero after a bounded wait inside the kernel ran out); it synchronises the device.
#define B200_GEMM_STATIC_SCRATCH_BYTES (8u << 20)
int b200_gemm_bf16_smallm_static(const void* A, int lda, const void* W, int ldw, void* out,
                                 int ldo, int M, int N, int K, cudaStream_t stream);
const char* b200_gemm_bf16_smallm_static_error(void);
int b200_gemm_bf16_smallm_static_status(int* out);

#ifdef __cplusplus
}
#endif
