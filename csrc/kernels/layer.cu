// One call per decoder layer: the launch sequence of a pre-norm dense transformer block
// (RMSNorm+residual -> QKV GEMM -> qk-norm/RoPE/KV-cache write -> paged attention (decode rows
// first, then prefill tiles) -> o GEMM -> RMSNorm+residual -> gated MLP) issued from native code.
// The model classes otherwise sequence these launches from Python, ~10 calls per layer; for
// batches where the GPU step is short (data-parallel replicas, tensor-parallel shards, small
// models) that host time is what bounds the step. This entry covers the plain configuration
// (no biases, no sandwich / post norms, no tensor parallelism); everything else keeps the
// per-op path.
//
// Reference: Qwen3DenseModel::ForwardDevice, src/vllm/model_executor/models/qwen3.cpp:135-244
// (the reference's forward is native code throughout).
#include <cstddef>

#include "api.h"
#include "sm100.cuh"

extern "C" {

// force_path bit 8: the weight operand is constant, its first tiles may be fetched before the
// predecessor kernel has finished
static constexpr int kConstW = 0x100;

#define B200_TRY(call)          \
  do {                          \
    int rc_ = (call);           \
    if (rc_ != 0) return rc_ < 0 ? rc_ : -rc_; \
    ++launches;                 \
  } while (0)

// Layout check for bindings: sizes of the two structs and the offsets of their last members.
void b200_dense_layer_abi(int* out4) {
  out4[0] = (int)sizeof(B200DenseLayerWeights);
  out4[1] = (int)sizeof(B200DenseStep);
  out4[2] = (int)offsetof(B200DenseLayerWeights, down_scale);
  out4[3] = (int)offsetof(B200DenseStep, fp8_scales);
}

// Attention half of a block: (add+)RMSNorm -> QKV GEMM -> qk-norm / RoPE / KV-cache write ->
// paged attention (decode rows, then prefill tiles) -> o_proj GEMM into s->hidden. Returns the
// number of launcher calls made or a negative error code.
int b200_dense_attn_half(const B200DenseLayerWeights* w, const B200DenseStep* s, cudaStream_t stream) {
  if (!w || !s || s->T <= 0) return 0;
  int launches = 0;
  const int T = s->T, H = s->H, D = s->D, Hq = s->Hq, Hkv = s->Hkv;
  const int qkv_w = (Hq + 2 * Hkv) * D;
  using bf16 = __nv_bfloat16;
  const bool fp8 = w->fp8 != 0;
  if (fp8 && (!s->fp8_act || !s->fp8_scales || !w->qkv_scale || !w->o_scale)) return -1;
  if (s->first_layer &&
      cudaMemcpyAsync(s->resid, s->hidden, (size_t)T * H * sizeof(bf16), cudaMemcpyDeviceToDevice, stream) !=
          cudaSuccess)
    return -2;
  void* resid_in = s->first_layer ? nullptr : s->resid;
  if (fp8) {
    // (add +) RMSNorm and the row-wise quantisation in one kernel; scales: per token x per channel
    B200_TRY(b200_quant_fp8_rowwise(s->hidden, H, resid_in, w->ln1, s->eps, s->gemma, 1, 0, s->fp8_act, H,
                                    s->fp8_scales, T, H, stream));
    B200_TRY(b200_gemm_fp8(s->fp8_act, H, w->qkv, H, s->qkv_buf, qkv_w, (const float*)s->fp8_scales, w->qkv_scale,
                           3, nullptr, T, qkv_w, H, stream));
  } else {
    B200_TRY(b200_rmsnorm(s->hidden, H, resid_in, w->ln1, s->normed, H, T, H, s->eps, s->gemma, stream));
    B200_TRY(b200_gemm_bf16(s->normed, H, w->qkv, H, s->qkv_buf, qkv_w, 0, nullptr, nullptr, 0, T, qkv_w, H,
                            s->gemm_ws, (size_t)s->gemm_ws_bytes, kConstW, stream));
  }
  B200_TRY(b200_rope_kv(s->qkv_buf, qkv_w, 0, Hq * D, (Hq + Hkv) * D, D, Hq, Hkv, D, s->rot, s->positions,
                        s->cos_sin, w->q_norm, w->k_norm, s->eps, s->gemma, s->neox, s->slot_mapping,
                        w->kv_cache, s->block_size, nullptr, T, stream));
  const int nd = s->num_decodes;
  if (nd > 0) {
    if (s->decode_tc)
      B200_TRY(b200_attn_decode_tc(s->qkv_buf, qkv_w, s->attn, Hq * D, w->kv_cache, s->num_blocks, s->block_size,
                                   Hq, Hkv, D, s->block_table, s->max_blocks, s->seq_lens, nd, s->scale,
                                   s->softcap, s->window, s->decode_splits, s->decode_tmp_o, s->decode_tmp_lse,
                                   stream));
    else
      B200_TRY(b200_attn_decode(s->qkv_buf, qkv_w, s->attn, Hq * D, w->kv_cache, s->block_size, Hq, Hkv, D,
                                s->block_table, s->max_blocks, s->seq_lens, nd, s->scale, s->softcap, s->window,
                                s->decode_splits, s->decode_tmp_o, s->decode_tmp_lse, stream));
  }
  if (s->num_prefills > 0) {
    const bf16* q = reinterpret_cast<const bf16*>(s->qkv_buf) + (size_t)nd * qkv_w;
    bf16* o = reinterpret_cast<bf16*>(s->attn) + (size_t)nd * Hq * D;
    const int32_t* bt = reinterpret_cast<const int32_t*>(s->block_table) + (size_t)nd * s->max_blocks;
    const int32_t* sl = reinterpret_cast<const int32_t*>(s->seq_lens) + nd;
    B200_TRY(b200_attn_prefill(q, qkv_w, o, Hq * D, nullptr, w->kv_cache, s->num_blocks, s->block_size, Hq, Hkv, D,
                               bt, s->max_blocks, sl, s->prefill_q_start, s->tile_req, s->tile_q0, s->num_tiles,
                               s->num_prefill_tokens, s->scale, s->softcap, s->window, 1, stream));
  }
  if (fp8) {
    B200_TRY(b200_quant_fp8_rowwise(s->attn, Hq * D, nullptr, nullptr, 0.f, 0, 0, 0, s->fp8_act, Hq * D,
                                    s->fp8_scales, T, Hq * D, stream));
    B200_TRY(b200_gemm_fp8(s->fp8_act, Hq * D, w->o, Hq * D, s->hidden, H, (const float*)s->fp8_scales, w->o_scale,
                           3, nullptr, T, H, Hq * D, stream));
  } else {
    B200_TRY(b200_gemm_bf16(s->attn, Hq * D, w->o, Hq * D, s->hidden, H, 0, nullptr, nullptr, 0, T, H, Hq * D,
                            s->gemm_ws, (size_t)s->gemm_ws_bytes, kConstW, stream));
  }
  return launches;
}

// Whole block: the attention half, then add+RMSNorm and the gated MLP into s->hidden.
// Returns the number of launcher calls made (>= 1 kernel each), or a negative error code.
int b200_dense_layer(const B200DenseLayerWeights* w, const B200DenseStep* s, cudaStream_t stream) {
  if (!w || !s || s->T <= 0) return 0;
  int launches = b200_dense_attn_half(w, s, stream);
  if (launches < 0) return launches;
  const int T = s->T, H = s->H;
  // ---- MLP block
  const int I = s->inter;
  if (w->fp8) {
    if (!w->gate_up_scale || !w->down_scale) return -1;
    B200_TRY(b200_quant_fp8_rowwise(s->hidden, H, s->resid, w->ln2, s->eps, s->gemma, 1, 0, s->fp8_act, H,
                                    s->fp8_scales, T, H, stream));
    B200_TRY(b200_gemm_fp8(s->fp8_act, H, w->gate_up, H, s->gate_up_buf, 2 * I, (const float*)s->fp8_scales,
                           w->gate_up_scale, 3, nullptr, T, 2 * I, H, stream));
    // act(gate) * up and its quantisation in one kernel
    B200_TRY(b200_quant_fp8_rowwise(s->gate_up_buf, 2 * I, nullptr, nullptr, 0.f, 0, 2,
                                    s->act_kind | (s->gate_up_interleaved ? 0x100 : 0), s->fp8_act, I,
                                    s->fp8_scales, T, I, stream));
    B200_TRY(b200_gemm_fp8(s->fp8_act, I, w->down, I, s->hidden, H, (const float*)s->fp8_scales, w->down_scale, 3,
                           nullptr, T, H, I, stream));
    return launches;
  }
  B200_TRY(b200_rmsnorm(s->hidden, H, s->resid, w->ln2, s->normed, H, T, H, s->eps, s->gemma, stream));
  if (s->gate_up_interleaved && T > 128) {
    B200_TRY(b200_gemm_bf16_gated(s->normed, H, w->gate_up, H, s->act, I, T, 2 * I, H, s->act_kind, 0, stream));
  } else {
    B200_TRY(b200_gemm_bf16(s->normed, H, w->gate_up, H, s->gate_up_buf, 2 * I, 0, nullptr, nullptr, 0, T, 2 * I,
                            H, s->gemm_ws, (size_t)s->gemm_ws_bytes, kConstW, stream));
    B200_TRY(b200_act_and_mul(s->gate_up_buf, 2 * I, s->act, T, I,
                              s->act_kind | (s->gate_up_interleaved ? 0x100 : 0), stream));
  }
  B200_TRY(b200_gemm_bf16(s->act, I, w->down, I, s->hidden, H, 0, nullptr, nullptr, 0, T, H, I, s->gemm_ws,
                          (size_t)s->gemm_ws_bytes, kConstW, stream));
  return launches;
}

// ---- tensor-parallel stack ----------------------------------------------------------------
void b200_tp_layers_abi(int* out2) {
  out2[0] = (int)sizeof(B200TpLayers);
  out2[1] = (int)offsetof(B200TpLayers, final_norm);
}

namespace {
struct TpIssue {
  const B200TpLayers* c;
  const B200DenseStep* s;
  cudaStream_t stream;
  int rpr;                     // rows per rank of this step
  long long recv_parity, x_parity;
  int rs_groups, ag_groups;

  int gather_gemm(const void* W, int N, void* out, int ldo, int out_f32, int act_fuse = 0) const {
    B200TpGemm d{};
    d.act_fuse = act_fuse;
    d.world = c->world; d.rank = c->rank; d.rows_per_rank = rpr;
    d.gather = 1;
    d.a_alt = reinterpret_cast<const __nv_bfloat16*>(c->x_full[c->rank]) + x_parity;
    d.ag_flags = c->ag_flags[c->rank];
    d.ag_flag_parity_stride = ag_groups;
    d.op_counter = c->op_counter;
    d.out_f32 = out_f32;
    return b200_gemm_bf16_tp(c->x_full[c->rank], s->H, W, s->H, out, ldo, s->T, N, s->H, &d, nullptr, stream);
  }
  // partial a[T, K] x W[H, K]^T scattered to the row owners; *expected / *nsrc feed the reduce
  int scatter_gemm(const void* a, int K, const void* W, int* expected, int* nsrc) const {
    B200TpGemm d{};
    d.world = c->world; d.rank = c->rank; d.rows_per_rank = rpr;
    d.scatter = 1;
    for (int r = 0; r < c->world; ++r) { d.peer_recv[r] = c->recv[r]; d.peer_rs_flags[r] = c->rs_flags[r]; }
    d.recv_parity_stride = recv_parity;
    d.rs_flag_parity_stride = rs_groups;
    d.op_counter = c->op_counter;
    int splits = 1;
    if (s->T <= 256) {
      // small batches: split K so that more than H / 128 CTAs stream the weight shard; every
      // (rank, split) pair owns a source slot of the receive buffer
      const int tiles_n = (s->H + 127) / 128, kblocks = (K + 63) / 64;
      splits = b200_num_sms() / tiles_n;
      if (splits > kblocks / 4) splits = kblocks / 4;
      if (splits > c->rpr_max / rpr) splits = c->rpr_max / rpr;
      if (splits > 8) splits = 8;
      if (splits < 1) splits = 1;
      const int kb_per = (kblocks + splits - 1) / splits;
      splits = (kblocks + kb_per - 1) / kb_per;
    }
    d.scatter_splits = splits;
    *nsrc = c->world * splits;
    return b200_gemm_bf16_tp(a, K, W, K, nullptr, s->H, s->T, s->H, K, &d, expected, stream);
  }
  int reduce(int expected, int nsrc, const void* norm_w) const {
    B200TpReduce a{};
    a.world = c->world; a.rank = c->rank; a.rows_per_rank = rpr; a.M = s->T; a.H = s->H;
    a.recv = c->recv[c->rank];
    a.recv_parity_stride = recv_parity;
    a.rs_flags = c->rs_flags[c->rank];
    a.rs_flag_parity_stride = rs_groups;
    a.expected_rs = expected;
    a.nsrc = nsrc;
    a.residual = c->residual;
    a.norm_w = norm_w;
    a.eps = s->eps; a.gemma = s->gemma;
    for (int r = 0; r < c->world; ++r) { a.peer_x[r] = c->x_full[r]; a.peer_ag_flags[r] = c->ag_flags[r]; }
    a.x_parity_stride = x_parity;
    a.ag_flag_parity_stride = ag_groups;
    a.ag_groups = ag_groups;
    a.op_counter = c->op_counter;
    a.done_counter = c->done_counter;
    return b200_tp_reduce_norm_gather(&a, stream);
  }
};
}  // namespace

// All blocks of the fused tensor-parallel forward. On entry the first norm has run
// (b200_tp_first_norm: gathered buffer = norm(embeddings), residual shard initialised); on return
// the gathered buffer holds the final norm's output. s->Hq / Hkv / inter are this rank's shards.
// Returns the number of launcher calls made or a negative error code.
int b200_dense_layers_tp(const B200DenseLayerWeights* w, int num_layers, const B200DenseStep* s,
                         const B200TpLayers* c, cudaStream_t stream) {
  if (!w || !s || !c || s->T <= 0 || num_layers <= 0) return 0;
  if (c->world < 2 || c->world > 8 || (c->rpr_max & 31) || (c->max_tokens & 31) || s->T > c->max_tokens)
    return -1;
  int launches = 0;
  const int T = s->T, H = s->H, D = s->D, Hq = s->Hq, Hkv = s->Hkv, I = s->inter;
  const int qkv_w = (Hq + 2 * Hkv) * D;
  using bf16 = __nv_bfloat16;
  TpIssue tp;
  tp.c = c; tp.s = s; tp.stream = stream;
  tp.rpr = (((T + c->world - 1) / c->world) + 31) & ~31;
  if (tp.rpr > c->rpr_max) return -1;
  tp.recv_parity = (long long)c->world * c->rpr_max * H;
  tp.x_parity = (long long)c->max_tokens * H;
  tp.rs_groups = c->rpr_max / 32;
  tp.ag_groups = c->max_tokens / 32;
  const int nd = s->num_decodes;
  for (int l = 0; l < num_layers; ++l) {
    const B200DenseLayerWeights* L = w + l;
    B200_TRY(tp.gather_gemm(L->qkv, qkv_w, s->qkv_buf, qkv_w, 0));
    B200_TRY(b200_rope_kv(s->qkv_buf, qkv_w, 0, Hq * D, (Hq + Hkv) * D, D, Hq, Hkv, D, s->rot, s->positions,
                          s->cos_sin, L->q_norm, L->k_norm, s->eps, s->gemma, s->neox, s->slot_mapping,
                          L->kv_cache, s->block_size, nullptr, T, stream));
    if (nd > 0) {
      if (s->decode_tc)
        B200_TRY(b200_attn_decode_tc(s->qkv_buf, qkv_w, s->attn, Hq * D, L->kv_cache, s->num_blocks, s->block_size,
                                     Hq, Hkv, D, s->block_table, s->max_blocks, s->seq_lens, nd, s->scale,
                                     s->softcap, s->window, s->decode_splits, s->decode_tmp_o,
                                     s->decode_tmp_lse, stream));
      else
        B200_TRY(b200_attn_decode(s->qkv_buf, qkv_w, s->attn, Hq * D, L->kv_cache, s->block_size, Hq, Hkv, D,
                                  s->block_table, s->max_blocks, s->seq_lens, nd, s->scale, s->softcap,
                                  s->window, s->decode_splits, s->decode_tmp_o, s->decode_tmp_lse, stream));
    }
    if (s->num_prefills > 0) {
      const bf16* q = reinterpret_cast<const bf16*>(s->qkv_buf) + (size_t)nd * qkv_w;
      bf16* o = reinterpret_cast<bf16*>(s->attn) + (size_t)nd * Hq * D;
      const int32_t* bt = reinterpret_cast<const int32_t*>(s->block_table) + (size_t)nd * s->max_blocks;
      const int32_t* sl = reinterpret_cast<const int32_t*>(s->seq_lens) + nd;
      B200_TRY(b200_attn_prefill(q, qkv_w, o, Hq * D, nullptr, L->kv_cache, s->num_blocks, s->block_size, Hq, Hkv,
                                 D, bt, s->max_blocks, sl, s->prefill_q_start, s->tile_req, s->tile_q0,
                                 s->num_tiles, s->num_prefill_tokens, s->scale, s->softcap, s->window, 1, stream));
    }
    int expected = 0, nsrc = 0;
    B200_TRY(tp.scatter_gemm(s->attn, Hq * D, L->o, &expected, &nsrc));
    B200_TRY(tp.reduce(expected, nsrc, L->ln2));
    if (s->gate_up_interleaved && T > 256 && ((2 * I) & 255) == 0) {
      // the gated activation runs in the GEMM's epilogue (CTA-pair tiles hold gate and up halves)
      B200_TRY(tp.gather_gemm(L->gate_up, 2 * I, s->act, I, 0, s->act_kind + 1));
    } else {
      B200_TRY(tp.gather_gemm(L->gate_up, 2 * I, s->gate_up_buf, 2 * I, 0));
      B200_TRY(b200_act_and_mul(s->gate_up_buf, 2 * I, s->act, T, I,
                                s->act_kind | (s->gate_up_interleaved ? 0x100 : 0), stream));
    }
    B200_TRY(tp.scatter_gemm(s->act, I, L->down, &expected, &nsrc));
    B200_TRY(tp.reduce(expected, nsrc, l + 1 < num_layers ? w[l + 1].ln1 : c->final_norm));
  }
  return launches;
}

}  // extern "C"
