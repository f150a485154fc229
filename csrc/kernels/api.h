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
// Allocates the per-device scratch of the launchers (stream-K partials) for the current device.
// Call once per device before the first stream capture. 0 on success.
int b200_init_device();
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

// ---- argument structs of the multi-kernel entry points -----------------------------------
// Weights of one layer (device pointers; q_norm / k_norm may be null).
typedef struct B200DenseLayerWeights {
  const void* ln1;
  const void* qkv;        // [(Hq + 2 Hkv) D, H]
  const void* q_norm;
  const void* k_norm;
  const void* o;          // [H, Hq D]
  const void* ln2;
  const void* gate_up;    // [2 I, H], interleaved in blocks of 128 if gate_up_interleaved
  const void* down;       // [H, I]
  void* kv_cache;         // [num_blocks, 2, block_size, Hkv, D]
  // fp8 != 0: qkv / o / gate_up / down are e4m3 [N, K] with one fp32 scale per output channel;
  // the activations are quantised row by row (one scale per token) in the kernel that makes them
  int fp8;
  const float* qkv_scale;
  const float* o_scale;
  const float* gate_up_scale;
  const float* down_scale;
} B200DenseLayerWeights;

// Shapes, step metadata (device pointers into the packed step buffer) and activation buffers.
typedef struct B200DenseStep {
  int T, H, Hq, Hkv, D, rot, inter, block_size;
  int neox, gemma, act_kind, gate_up_interleaved;
  float eps, scale, softcap;
  int window;
  long long num_blocks;
  const void* positions;
  const void* cos_sin;
  const void* slot_mapping;
  const void* block_table;
  int max_blocks;
  const void* seq_lens;
  int num_decodes, decode_splits, decode_tc;
  void* decode_tmp_o;
  void* decode_tmp_lse;
  int num_prefills, num_tiles, num_prefill_tokens;
  const void* prefill_q_start;
  const void* tile_req;
  const void* tile_q0;
  void* hidden;           // [T, H] in: previous block's output (or the embeddings); out: this block's
  void* resid;            // [T, H] residual stream
  void* normed;           // [T, H]
  void* qkv_buf;          // [T, (Hq + 2 Hkv) D]
  void* attn;             // [T, Hq D]
  void* gate_up_buf;      // [T, 2 I]
  void* act;              // [T, I]
  void* gemm_ws;
  unsigned long long gemm_ws_bytes;
  int first_layer;        // the residual stream starts here: resid = hidden, no add
  void* fp8_act;          // fp8 weights: [T, max(H, Hq D, I)] bytes of quantised activations
  void* fp8_scales;       // fp8 weights: [T] fp32 per-token scales
} B200DenseStep;

// Peer-mapped buffers of the fused tensor-parallel path (see tp_fused.cu): per rank a receive
// buffer, a gathered-activation buffer and the counters, each with two parities.
typedef struct B200TpLayers {
  int world, rank;
  int rpr_max;                 // capacity of a rank's row shard (multiple of 32)
  int max_tokens;              // capacity of the gathered buffer (multiple of 32)
  void* recv[8];               // [2][world * k-splits][rpr][H] bf16
  void* rs_flags[8];           // [2][rpr_max / 32]
  void* x_full[8];             // [2][max_tokens][H] bf16
  void* ag_flags[8];           // [2][max_tokens / 32]
  void* op_counter;            // local
  void* done_counter;          // local
  void* residual;              // local shard [rpr_max][H]
  const void* final_norm;      // the norm after the last block
} B200TpLayers;

// Owner-side reduce of the fused tensor-parallel path (tp_fused.cu).
typedef struct B200TpReduce {
  int world, rank, rows_per_rank, M, H;
  const void* recv;
  long long recv_parity_stride;
  void* rs_flags;
  int rs_flag_parity_stride;
  int expected_rs;
  int nsrc;
  void* residual;
  const void* norm_w;
  float eps;
  int gemma;
  void* peer_x[8];
  long long x_parity_stride;
  void* peer_ag_flags[8];
  int ag_flag_parity_stride;
  int ag_groups;
  void* op_counter;
  void* done_counter;
} B200TpReduce;

// One-shot all-reduce (+ residual + RMSNorm) for decode-sized batches: every rank reads all ranks'
// partial rows over peer pointers. peer_partial[r]: rank r's partial [M, H] of THIS op (the caller
// alternates two buffers per rank); peer_flags[r]: rank r's array of `world` monotonic arrival
// counters; seq / done_counter: local uint32 words, zero at start. norm_w null: plain sum.
// mc_partial: the partial buffer of this op through an NVSwitch multicast mapping (then the sum is
// one multimem.ld_reduce per 16 bytes, reduced in the switch), or null for peer loads.
typedef struct B200TpOneShot {
  int world, rank, M, H;
  const void* peer_partial[8];
  void* peer_flags[8];
  const void* mc_partial;
  void* seq;
  void* done_counter;
  void* residual;
  const void* norm_w;
  void* out;
  float eps;
  int gemma;
} B200TpOneShot;

// Row-owner scatter of the MoE combine (moe.cu): the same receive slots and counters as the
// scatter epilogue of the GEMM.
typedef struct B200MoeScatter {
  int world, rank, rows_per_rank;
  void* peer_recv[8];
  void* peer_rs_flags[8];
  long long recv_parity_stride;
  int rs_flag_parity_stride;
  const void* op_counter;
} B200MoeScatter;

// A fused-chain program (recipe.cu): rows x width bf16 values, up to four shared-memory row
// registers, a list of steps over them. Operand rows are addressed as
// ptr + (row / heads) * ld + (row % heads) * width + col, in elements of the operand's type
// (bf16, or bytes for fp8 output); ld = 0 for a vector or scalar operand.
#define B200_CHAIN_MAX_STEPS 16
#define B200_CHAIN_MAX_OPERANDS 12
typedef struct B200ChainStep {
  int op, dst, a, b;
  int operand, operand2, operand3;
  int flag;
  float f;
} B200ChainStep;
typedef struct B200ChainOperand {
  void* ptr;
  long long ld, col;
} B200ChainOperand;
typedef struct B200Chain {
  int n_steps, n_regs, width, heads;
  long long rows;
  B200ChainStep steps[B200_CHAIN_MAX_STEPS];
  B200ChainOperand operands[B200_CHAIN_MAX_OPERANDS];
} B200Chain;

// ---- every other launcher, by source file ----------------------------------------------
// ---- attn_decode.cu
int b200_attn_decode_splits(int B, int Hkv, int G, int D, int max_seq_len);
int b200_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kv_cache, int block_size, int Hq, int Hkv, int D, const void* block_table, int max_blocks, const void* seq_lens, int B, float scale, float softcap, int window, int splits, void* tmp_o, void* tmp_lse, cudaStream_t stream);
int b200_attn_decode_merge(const void* tmp_o, const void* tmp_lse, void* out, int ldo, int B, int Hq, int D, int splits, cudaStream_t stream);
int b200_merge_attn_states(const void* a, const void* lse_a, const void* b, const void* lse_b, void* out, void* lse_out, int T, int H, int D, cudaStream_t stream);
// ---- attn_decode_tc.cu
int b200_attn_decode_tc(const void* q, int ldq, void* out, int ldo, const void* kv_cache, int64_t num_blocks, int block_size, int Hq, int Hkv, int D, const void* block_table, int max_blocks, const void* seq_lens, int B, float scale, float softcap, int window, int splits, void* tmp_o, void* tmp_lse, cudaStream_t stream);
// ---- attn_prefill.cu
int b200_attn_prefill(const void* q, int ldq, void* out, int ldo, void* lse, const void* kv_cache, int64_t num_blocks, int block_size, int Hq, int Hkv, int D, const void* block_table, int max_blocks, const void* seq_lens, const void* q_start, const void* tile_req, const void* tile_q0, int num_tiles, int total_q, float scale, float softcap, int window, int causal, cudaStream_t stream);
// ---- common.cu
long long b200_set_peer_wait_cycles(long long cycles);
// ---- gdn.cu
int b200_gdn_conv1d_fwd(const void* x, long ldx, const void* w, void* conv_state, const int* qsl, const int* slots, const int* has_init, void* out, long ldo, int n_seq, int total_tokens, int C, cudaStream_t stream);
int b200_gdn_conv1d_update(const void* x, long ldx, const void* w, void* conv_state, const int* slots, void* out, long ldo, int B, int C, cudaStream_t stream);
int b200_gdn_post_conv(const void* xc, long ld, int T, int Hk, int Hv, int Dk, const void* a, const void* b, long ldab, const float* A_log, const float* dt_bias, void* q_out, void* k_out, float* g, float* beta, float eps, cudaStream_t stream);
int b200_gdn_packed_decode(const void* xc, long ld, const void* a, const void* b, long ldab, const float* A_log, const float* dt_bias, float* state, const int* slots, void* out, int B, int Hk, int Hv, int Dk, int Dv, float eps, cudaStream_t stream);
int b200_rmsnorm_gated(const void* x, long ldx, const void* z, long ldz, const void* w, void* out, long ldo, long R, int D, float eps, int gate_kind, int heads, cudaStream_t stream);
// ---- gdn_scan.cu
int b200_gdn_chunk_scan(const void* q, const void* k, const void* v, long ldv, int v_col0, const float* g, const float* beta, int T, int Hk, int Hv, const int* chunk_tok0, const int* chunk_len, int NT, const int* seq_chunk0, const int* slots, const int* has_init, int n_seq, float* state, void* u, void* w, void* qs, void* pbuf, float* gc, void* out, cudaStream_t stream);
// ---- gemm_bf16.cu
int b200_gemm_bf16_gated(const void* A, int lda, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int kind, int force_path, cudaStream_t stream);
int b200_gemm_fp8_pair(const void* A, int lda, const void* W, int ldw, void* out, int ldo, const float* a_scale, const float* w_scale, int w_scale_per_channel, const void* bias, int M, int N, int K, cudaStream_t stream);
int b200_gemm_bf16_batched(const void* A, int lda, int a_batch_cols, const void* W, int ldw, void* out, int ldo, long long out_batch_stride, int M, int N, int K, int batch, cudaStream_t stream);
// ---- gemm_quant.cu
int b200_gemm_fp8(const void* A, int lda, const void* W, int ldw, void* out, int ldo, const float* a_scale, const float* w_scale, int w_scale_per_channel, const void* bias, int M, int N, int K, cudaStream_t stream);
int b200_nvfp4_dequant(const void* packed, const void* sf, const float* gscale, void* out, long N, int K, cudaStream_t stream);
int b200_fp8_init_device();
int b200_quant_fp8_dynamic(const void* x, long ldx, void* scratch, void* out, long ldo, long T, int H, cudaStream_t stream);
int b200_quant_fp8(const void* x, long ldx, const void* norm_w, float eps, int gemma, const float* scale, void* out, long ldo, long T, int H, cudaStream_t stream);
int b200_quant_nvfp4_gated(const void* x, long ldx, const void* gate, long ldg, const float* gscale, void* out, void* sf, long T, int K, int swizzle, cudaStream_t stream);
int b200_rmsnorm_quant_nvfp4(const void* x, long ldx, void* residual, const void* weight, float eps, int gemma, const float* gscale, void* out, void* sf, void* normed, long T, int K, int swizzle, cudaStream_t stream);
int b200_quant_nvfp4(const void* x, long ldx, const float* gscale, void* out, void* sf, long T, int K, int mode, int swizzle, cudaStream_t stream);
// ---- gemm_w4a16.cu
// NVFP4 x NVFP4 (W4A4) on the block-scaled tensor-core path; scales in the 128 x 4 chunk layout
// (b200_nvfp4_sf_to_chunks / b200_quant_nvfp4 with swizzle = 1). K a multiple of 256.
int b200_gemm_nvfp4(const void* aq, const void* sfa, const float* g_a, const void* wq, const void* sfw, const float* g_w, void* out, int ldo, const void* bias, int M, int N, int K, int n_tile, void* workspace, size_t ws_bytes, cudaStream_t stream);
int b200_nvfp4_sf_to_chunks(const void* sf, long rows, int K, int pad_rows, void* out, cudaStream_t stream);
int b200_gemm_w4a16(const void* A, int lda, const void* wq, const void* sf, const float* gscale, void* out, int ldo, const void* bias, int M, int N, int K, void* workspace, size_t ws_bytes, cudaStream_t stream);
// ---- layer.cu
void b200_dense_layer_abi(int* out4);
int b200_dense_attn_half(const B200DenseLayerWeights* w, const B200DenseStep* s, cudaStream_t stream);
int b200_dense_layer(const B200DenseLayerWeights* w, const B200DenseStep* s, cudaStream_t stream);
void b200_tp_layers_abi(int* out2);
int b200_dense_layers_tp(const B200DenseLayerWeights* w, int num_layers, const B200DenseStep* s, const B200TpLayers* c, cudaStream_t stream);
// ---- mla.cu
int b200_mla_decode(const void* qabs, void* out, int ldo, const void* cache, int64_t num_blocks, int block_size, int Hq, const void* block_table, int max_blocks, const void* seq_lens, int B, float scale, int splits, void* tmp_o, void* tmp_lse, cudaStream_t stream);
int b200_mla_gather_latent(const void* cache, const void* block_table, int max_blocks, const void* seq_lens, const void* dense_base, int block_size, void* dense, int num_reqs, int max_req_blocks, cudaStream_t stream);
int b200_mla_assemble_kv(const void* kvb, const void* dense, void* cache, int N, int H, int block_size, cudaStream_t stream);
int b200_mla_pad_q(const void* q, long ldq, void* out, int T, int H, cudaStream_t stream);
int b200_mla_copy_qpe(const void* q, long ldq, void* qabs, int T, int H, cudaStream_t stream);
// ---- moe.cu
int b200_moe_router_topk(const void* logits_f32, int ld, int T, int E, int k, int renorm, int scoring, const void* e_bias, int n_group, int topk_group, float routed_scale, void* topk_ids, void* topk_w, cudaStream_t stream);
int b200_moe_sort(const void* topk_ids, int T, int k, int e0, int e1, void* meta, void* sorted_token, void* pair_pos, void* chunk_expert, void* chunk_row0, void* chunk_n, int max_chunks, cudaStream_t stream);
int b200_moe_gather(const void* x, int ldx, const void* sorted_token, const void* meta, int E, void* xs, int H, int max_rows, cudaStream_t stream);
int b200_moe_grouped_gemm(const void* xs, int max_rows, const void* W, int E, int N, int K, void* out, const void* chunk_expert, const void* chunk_row0, const void* chunk_n, const void* meta, int max_chunks, cudaStream_t stream);
int b200_moe_grouped_gemm_gated(const void* xs, int max_rows, const void* W, int E, int N, int K, void* out, const void* chunk_expert, const void* chunk_row0, const void* chunk_n, const void* meta, int max_chunks, int kind, cudaStream_t stream);
int b200_moe_combine(const void* y, const void* pair_pos, const void* topk_w, int T, int k, int H, const void* shared, const void* shared_gate, void* out, const B200MoeScatter* sc, cudaStream_t stream);
int b200_shared_gate(const void* x, int ldx, const void* w, int T, int H, void* out, cudaStream_t stream);
// ---- norm_act.cu
int b200_rmsnorm(const void* x, int ldx, void* residual, const void* w, void* out, int ldo, int T, int H, float eps, int gemma, cudaStream_t stream);
int b200_quant_fp8_rowwise(const void* x, long ldx, void* residual, const void* norm_w, float eps, int gemma, int mode, int kind_flags, void* out, long ldo, void* scales, int T, int K, cudaStream_t stream);
int b200_layernorm(const void* x, const void* w, const void* b, void* out, int T, int H, float eps, cudaStream_t stream);
int b200_act_and_mul(const void* x, int ldx, void* out, int T, int I, int kind, cudaStream_t stream);
int b200_eltwise(const void* a, const void* b, void* out, size_t n, int kind, float scalar, cudaStream_t stream);
int b200_cast_bf16_f32(const void* a, void* out, size_t n, cudaStream_t stream);
int b200_cast_f32_bf16(const void* a, void* out, size_t n, cudaStream_t stream);
int b200_embedding(const void* ids, const void* table, void* out, int T, int H, int64_t vocab_start, int64_t vocab_rows, int64_t vocab_total, float scale, cudaStream_t stream);
int b200_gather_rows(const void* x, const void* idx, void* out, int n_out, int n_src, int row_bytes, cudaStream_t stream);
// ---- rope_cache.cu
int b200_rope_kv(void* qkv, int ld, int q_off, int k_off, int v_off, int q_head_stride, int Hq, int Hkv, int D, int rot, const void* positions, const void* cos_sin, const void* q_norm_w, const void* k_norm_w, float eps, int gemma, int neox, const void* slot_mapping, void* kv_cache, int block_size, void* q_out, int T, cudaStream_t stream);
int b200_reshape_and_cache(const void* k, int ldk, const void* v, int ldv, const void* slots, void* cache, int block_size, int Hkv, int D, int T, cudaStream_t stream);
int b200_concat_and_cache_mla(const void* kv_c, int ldc, const void* k_pe, int ldr, const void* slots, void* cache, int Lc, int Lr, int T, cudaStream_t stream);
int b200_rope_table(const void* inv_freq_f64, void* out_f32, int max_pos, int half, float mscale, cudaStream_t stream);
// ---- sample.cu
int b200_argmax_blocks_per_row(int n, int V);
int b200_argmax(const void* logits, int ld, int n, int V, void* out_i64, void* scratch_f, void* scratch_i, cudaStream_t stream);
int b200_argmax_candidates(const void* logits, int ld, int n, int V, int v_valid, int index_base, void* cand_out, void* scratch_f, void* scratch_i, cudaStream_t stream);
int b200_argmax_combine(const void* cand, int n, int world, int V_total, void* out_i64, cudaStream_t stream);
int b200_apply_temperature(void* logits, int ld, int n, int V, const void* temp, cudaStream_t stream);
int b200_apply_penalties(void* logits, int ld, int V, const void* rows, const void* toks, const void* out_cnt, int n_entries, const void* rep, const void* freq, const void* pres, cudaStream_t stream);
int b200_sparse_edit(void* logits, int ld, int V, const void* rows, const void* toks, const void* vals, int n_entries, int mode, cudaStream_t stream);
int b200_apply_bitmask(void* logits, int ld, int V, const void* mask, int n_mask_rows, const void* row_ids, cudaStream_t stream);
int b200_apply_min_p(void* logits, int ld, int n, int V, const void* min_p, cudaStream_t stream);
int b200_apply_top_k_top_p(void* logits, int ld, int n, int V, const void* top_k, const void* top_p, cudaStream_t stream);
int b200_softmax(const void* logits, int ld, void* out, int ldo, int n, int V, int log_mode, cudaStream_t stream);
int b200_random_sample(const void* probs, int ld, int n, int V, const void* seeds, const void* steps, void* out_i64, cudaStream_t stream);
int b200_merge_greedy_random(const void* g, const void* r, const void* temp, void* out, int n, cudaStream_t stream);
int b200_token_rank(const void* logprobs, int ld, int n, int V, const void* toks, void* out_lp, void* out_rank, cudaStream_t stream);
int b200_greedy_reject(const void* target_argmax, const void* draft, const void* cu_draft, int n, int max_spec, void* out, cudaStream_t stream);
int b200_splice_sampled(void* input_ids, const void* dst_idx, const void* src_row, const void* last_sampled, int n, cudaStream_t stream);
int b200_scatter_sampled(void* last_sampled, const void* row_of, const void* sampled, int n, cudaStream_t stream);
uint64_t b200_splitmix64(uint64_t z);
// ---- recipe.cu
int b200_fused_chain(const B200Chain* prog, cudaStream_t stream);
// ---- tp_fused.cu
int b200_tp_reduce_norm_gather(const B200TpReduce* a, cudaStream_t stream);
int b200_tp_oneshot_allreduce_norm(const B200TpOneShot* a, cudaStream_t stream);
int b200_tp_first_norm(const void* hidden, void* residual_shard, const void* w, void* x_full, long long x_parity_stride, void* ag_flags, int ag_flag_parity_stride, int ag_groups, void* rs_flags, int rs_flag_parity_stride, int rank, int rows_per_rank, int M, int H, float eps, int gemma, void* op_counter, void* done_counter, cudaStream_t stream);
int b200_tp_gather_rows(const void* x_base, long long x_parity_stride, int H, const void* idx, int n, const void* ag_flags, int ag_flag_parity_stride, const void* op_counter, int M, void* out, cudaStream_t stream);
void* b200_symm_alloc(size_t bytes);
int b200_symm_free(void* p);
int b200_ipc_get_handle(void* p, void* out64);
void* b200_ipc_open(const void* handle64);
int b200_ipc_close(void* p);
int b200_memset_async(void* p, int v, size_t bytes, cudaStream_t stream);

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
