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

#ifdef __cplusplus
}
#endif
