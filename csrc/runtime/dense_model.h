// Native decoder (Llama / Mistral / Qwen3 shapes: pre-norm blocks, RMSNorm, rotary embeddings,
// grouped-query attention over the paged KV cache, gated MLP, no biases; Qwen3-MoE: the same
// attention with a routed mixture of experts in place of the MLP): weights
// read from safetensors into device memory, forward pass as a sequence of launcher calls —
// the sm_100a kernel library on a GPU (one native call per block, csrc/kernels/layer.cu), the
// thread-pool CPU kernels (csrc/cpu) otherwise. No interpreter is involved anywhere.
//
// Reference: Qwen3DenseModel::ForwardDevice, src/vllm/model_executor/models/qwen3.cpp:135-244;
// weight naming and merging: src/vllm/model_executor/models/qwen3_weights.cpp, llama.cpp.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "runtime/tensor.h"

namespace b200 {
class Json;
}

namespace b200::rt {

struct DenseConfig {
  std::string architecture;
  int vocab_size = 0, hidden = 0, inter = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0;
  float eps = 1e-6f;
  int max_position = 8192;
  bool tie_embeddings = false, qk_norm = false;
  int act_kind = 0;                    // 0 SiLU, 1 GELU-tanh, 2 GELU-erf
  // rotary embedding
  double theta = 10000.0;
  std::string scaling;                 // "", "linear", "llama3"
  double factor = 1.0, low_freq_factor = 1.0, high_freq_factor = 4.0;
  int original_max_position = 8192;
  int rotary_dim = 0;                  // 0: head_dim
  int eos_token_id = -1, bos_token_id = -1;
  // mixture of experts (Qwen3-MoE): 0 experts = dense MLP
  int num_experts = 0, experts_per_token = 0, moe_inter = 0;
  bool norm_topk_prob = true;

  // Throws std::runtime_error naming what the native runtime does not cover.
  static DenseConfig from_hf(const Json& cfg);
};

// Device pointers into the packed step buffer + shapes of one engine step.
struct StepInputs {
  int num_tokens = 0, num_reqs = 0, num_decodes = 0, num_prefills = 0, num_prefill_tokens = 0, num_tiles = 0;
  int num_logits = 0;
  const int64_t* input_ids = nullptr;
  const int64_t* positions = nullptr;
  const int64_t* slot_mapping = nullptr;
  const int32_t* query_start = nullptr;     // [R + 1]
  const int32_t* seq_lens = nullptr;        // [R]
  const int32_t* block_table = nullptr;     // [R, max_blocks]
  int max_blocks = 0;
  const int32_t* logits_indices = nullptr;
  const int32_t* tile_req = nullptr;
  const int32_t* tile_q0 = nullptr;
  const int32_t* prefill_q_start = nullptr;
};

class DenseModel {
 public:
  DenseModel(const DenseConfig& cfg, Device dev, int max_position);
  void load_weights(const std::string& model_dir);
  void alloc_kv_cache(int64_t num_blocks, int block_size);
  void reserve(int max_tokens, int max_reqs);
  int64_t kv_bytes_per_block(int block_size) const;
  int64_t weight_bytes() const { return weight_bytes_; }
  // fp32 logits [num_logits, vocab] on the model's device for the rows in logits_indices
  float* forward(const StepInputs& in);
  const DenseConfig& config() const { return cfg_; }
  Device device() const { return dev_; }
  int64_t launches() const { return launches_; }

 private:
  struct Layer {
    Buffer ln1, qkv, q_norm, k_norm, o, ln2, gate_up, down, kv_cache;
    Buffer router, w_gate_up, w_down;    // MoE: [E, H], [E, 2 I, H] rows [gate | up], [E, H, I]
  };
  void moe_cuda(const Layer& L, int T);
  void moe_cpu(const Layer& L, int T);
  Buffer upload(const void* src, size_t nbytes);
  void forward_cuda(const StepInputs& in);
  void forward_cpu(const StepInputs& in);
  DenseConfig cfg_;
  Device dev_;
  int max_position_, rot_, block_size_ = 0;
  int64_t num_blocks_ = 0, weight_bytes_ = 0, launches_ = 0;
  bool gate_up_interleaved_ = false;
  float scale_;
  Buffer embed_, lm_head_, final_norm_, rope_table_;
  std::vector<Layer> layers_;
  // activations (sized by reserve)
  int max_tokens_ = 0, max_reqs_ = 0;
  Buffer hidden_, resid_, normed_, qkv_, attn_, gate_up_, act_, last_, logits_, gemm_ws_, decode_tmp_o_,
      decode_tmp_lse_, argmax_ws_;
  int decode_tmp_batch_ = 0, decode_tmp_splits_ = 0;
  // MoE workspace (sized by reserve): router logits, top-k, expert-sorted rows
  Buffer router_logits_, topk_ids_, topk_w_, moe_meta_, sorted_token_, pair_pos_, chunk_expert_, chunk_row0_,
      chunk_n_, xs_, moe_act_, moe_y_;
  int max_chunks_ = 0;
};

}  // namespace b200::rt
