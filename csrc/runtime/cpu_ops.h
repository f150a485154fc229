// Entry points of the thread-pool CPU kernels (csrc/cpu/cpu_ops.cpp, built into _cpu.so): bf16
// tensors as uint16_t, fp32 accumulation, results independent of the thread count.
#pragma once
#include <cstdint>

extern "C" {
void b200cpu_set_threads(int n);
int b200cpu_num_threads();
void b200cpu_matmul_bt(const uint16_t* A, int64_t lda, const uint16_t* W, int64_t ldw, void* out, int64_t ldo,
                       int out_f32, const uint16_t* bias, const uint16_t* residual, int64_t ldr, int M, int N, int K);
void b200cpu_rmsnorm(const uint16_t* x, int64_t ldx, const uint16_t* w, float eps, uint16_t* residual, int64_t ldr,
                     uint16_t* out, int64_t ldo, int T, int H, int gemma);
void b200cpu_act_and_mul(const uint16_t* x, int64_t ldx, uint16_t* out, int64_t ldo, int T, int I, int kind);
void b200cpu_embedding(const int64_t* ids, const uint16_t* table, uint16_t* out, int64_t ldo, int T, int H,
                       int64_t vocab_start, int64_t rows, float scale);
void b200cpu_rope_kv(uint16_t* qkv, int64_t ld, const int64_t* positions, const float* table, int T, int Hq, int Hkv,
                     int D, int rot, int neox, const uint16_t* q_norm, const uint16_t* k_norm, float eps, int gemma,
                     const int64_t* slot_mapping, uint16_t* kv_cache, int block_size);
void b200cpu_paged_attention(const uint16_t* q, int64_t ldq, const uint16_t* kv_cache, const int32_t* block_table,
                             int64_t max_blocks, const int32_t* seq_lens, const int32_t* q_start, int R, int Hq, int Hkv,
                             int D, int block_size, float scale, float softcap, int window, uint16_t* out, int64_t ldo);
}
