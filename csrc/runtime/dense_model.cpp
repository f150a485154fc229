#include "runtime/dense_model.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "kernels/api.h"
#include "runtime/cpu_ops.h"
#include "runtime/safetensors.h"
#include "util/json.h"

namespace b200::rt {

namespace {
constexpr size_t kGemmWsBytes = 64u << 20;
constexpr int kConstW = 0x100;   // force_path bit: the weight operand is constant

void check(int rc, const char* what) {
  if (rc < 0) throw std::runtime_error(std::string(what) + ": kernel launcher returned " + std::to_string(rc));
}

bool decode_uses_tc(int head_dim, int group, int block_size) {
  if (head_dim != 128 || group > 16 || block_size < 8 || block_size % 8) return false;
  return block_size <= 128 ? (128 % block_size == 0) : (block_size % 128 == 0);
}
}  // namespace

// ------------------------------------------------------------------------------- config
DenseConfig DenseConfig::from_hf(const Json& cfg_in) {
  Json t = cfg_in;
  if (cfg_in.contains("text_config"))
    for (auto& kv : cfg_in["text_config"].members()) t[kv.first] = kv.second;
  DenseConfig c;
  const auto& archs = t["architectures"];
  c.architecture = archs.size() ? archs[0].as_string() : "LlamaForCausalLM";
  static const char* kSupported[] = {"LlamaForCausalLM", "MistralForCausalLM", "Qwen3ForCausalLM",
                                     "Qwen3MoeForCausalLM"};
  bool ok = false;
  for (auto* a : kSupported) ok = ok || c.architecture == a;
  if (!ok)
    throw std::runtime_error("architecture " + c.architecture + " is not covered by the native runtime "
                             "(Llama / Mistral / Qwen3 / Qwen3-MoE families)");
  c.hidden = (int)t["hidden_size"].as_int();
  c.heads = (int)t["num_attention_heads"].as_int();
  c.head_dim = (int)t["head_dim"].as_int(c.heads ? c.hidden / c.heads : 0);
  c.vocab_size = (int)t["vocab_size"].as_int();
  c.inter = (int)t["intermediate_size"].as_int(4 * c.hidden);
  c.layers = (int)t["num_hidden_layers"].as_int();
  c.kv_heads = (int)t["num_key_value_heads"].as_int(c.heads);
  c.eps = (float)t["rms_norm_eps"].as_double(1e-6);
  c.max_position = (int)t["max_position_embeddings"].as_int(8192);
  c.tie_embeddings = t["tie_word_embeddings"].as_bool(false);
  c.qk_norm = c.architecture == "Qwen3ForCausalLM" || c.architecture == "Qwen3MoeForCausalLM";
  if (c.architecture == "Qwen3MoeForCausalLM") {
    c.num_experts = (int)t["num_experts"].as_int();
    c.experts_per_token = (int)t["num_experts_per_tok"].as_int();
    c.moe_inter = (int)t["moe_intermediate_size"].as_int();
    c.norm_topk_prob = t["norm_topk_prob"].as_bool(true);
    if (c.num_experts <= 0 || c.experts_per_token <= 0 || c.experts_per_token > c.num_experts || c.moe_inter <= 0)
      throw std::runtime_error("config.json: inconsistent mixture-of-experts shape");
    if (t["mlp_only_layers"].size() > 0 || t["decoder_sparse_step"].as_int(1) != 1)
      throw std::runtime_error("mixed dense / sparse layer patterns are not covered by the native runtime");
  }
  const std::string act = t["hidden_act"].is_string() ? t["hidden_act"].as_string() : "silu";
  if (act == "silu") c.act_kind = 0;
  else if (act == "gelu_tanh" || act == "gelu_pytorch_tanh") c.act_kind = 1;
  else if (act == "gelu") c.act_kind = 2;
  else throw std::runtime_error("activation " + act + " is not covered by the native runtime");
  if (t["attention_bias"].as_bool(false) || t["mlp_bias"].as_bool(false))
    throw std::runtime_error("projection biases are not covered by the native runtime");
  if (t["sliding_window"].as_int(0) > 0 && t["use_sliding_window"].as_bool(c.architecture == "MistralForCausalLM"))
    throw std::runtime_error("sliding-window attention is not covered by the native runtime");
  if (t.contains("quantization_config") && !t["quantization_config"].is_null())
    throw std::runtime_error("quantised checkpoints are not covered by the native runtime");
  if (c.hidden <= 0 || c.heads <= 0 || c.layers <= 0 || c.vocab_size <= 0 || c.head_dim <= 0 ||
      c.heads % c.kv_heads)
    throw std::runtime_error("config.json: inconsistent model shape");
  c.theta = t["rope_theta"].as_double(10000.0);
  const Json* rs = t.find("rope_scaling");
  if (!rs || rs->is_null()) rs = t.find("rope_parameters");
  if (rs && rs->is_object()) {
    std::string ty = (*rs)["rope_type"].is_string() ? (*rs)["rope_type"].as_string() : (*rs)["type"].as_string();
    if ((*rs)["rope_theta"].is_number()) c.theta = (*rs)["rope_theta"].as_double();
    if (ty == "default" || ty.empty()) {
    } else if (ty == "linear") {
      c.scaling = "linear";
      c.factor = (*rs)["factor"].as_double(1.0);
    } else if (ty == "llama3") {
      c.scaling = "llama3";
      c.factor = (*rs)["factor"].as_double(8.0);
      c.low_freq_factor = (*rs)["low_freq_factor"].as_double(1.0);
      c.high_freq_factor = (*rs)["high_freq_factor"].as_double(4.0);
      c.original_max_position = (int)(*rs)["original_max_position_embeddings"].as_int(8192);
    } else {
      throw std::runtime_error("rope scaling '" + ty + "' is not covered by the native runtime");
    }
  }
  if (t["partial_rotary_factor"].is_number())
    c.rotary_dim = (int)(t["partial_rotary_factor"].as_double(1.0) * c.head_dim);
  const Json& eos = t["eos_token_id"];
  c.eos_token_id = eos.is_array() ? (int)eos[0].as_int(-1) : (int)eos.as_int(-1);
  c.bos_token_id = (int)t["bos_token_id"].as_int(-1);
  return c;
}

// ------------------------------------------------------------------------------- set-up
DenseModel::DenseModel(const DenseConfig& cfg, Device dev, int max_position)
    : cfg_(cfg), dev_(dev), max_position_(max_position > 0 ? max_position : cfg.max_position) {
  rot_ = cfg.rotary_dim > 0 ? cfg.rotary_dim : cfg.head_dim;
  scale_ = 1.0f / std::sqrt((float)cfg.head_dim);
  // inverse frequencies in fp64 on the host, the [cos | sin] table per position
  const int half = rot_ / 2;
  std::vector<double> inv(half);
  const double two_pi = 6.283185307179586476925287;
  for (int i = 0; i < half; ++i) {
    double f = 1.0 / std::pow(cfg.theta, (2.0 * i) / rot_);
    if (cfg.scaling == "linear") {
      f /= cfg.factor;
    } else if (cfg.scaling == "llama3") {
      const double low_wl = cfg.original_max_position / cfg.low_freq_factor;
      const double high_wl = cfg.original_max_position / cfg.high_freq_factor;
      const double wl = two_pi / f;
      if (wl >= high_wl && wl <= low_wl) {
        const double smooth = (cfg.original_max_position / wl - cfg.low_freq_factor) /
                              (cfg.high_freq_factor - cfg.low_freq_factor);
        f = (1 - smooth) * f / cfg.factor + smooth * f;
      } else if (wl > low_wl) {
        f /= cfg.factor;
      }
    }
    inv[i] = f;
  }
  set_device(dev_);
  rope_table_ = alloc((size_t)max_position_ * rot_ * sizeof(float), dev_);
  if (dev_.cuda) {
    Buffer dinv = upload(inv.data(), inv.size() * sizeof(double));
    check(b200_rope_table(dinv.data(), rope_table_.data(), max_position_, half, 1.0f,
                          (cudaStream_t)current_stream(dev_)), "rope_table");
    synchronize(dev_);
  } else {
    float* tab = rope_table_.as<float>();
    for (int p = 0; p < max_position_; ++p)
      for (int i = 0; i < half; ++i) {
        const double ph = (double)p * inv[i];
        tab[(size_t)p * rot_ + i] = (float)std::cos(ph);
        tab[(size_t)p * rot_ + half + i] = (float)std::sin(ph);
      }
  }
}

Buffer DenseModel::upload(const void* src, size_t nbytes) {
  Buffer b = alloc(nbytes, dev_);
  copy(b.data(), dev_, src, Device{}, nbytes);
  if (dev_.cuda) synchronize(dev_);      // the source may be a temporary
  return b;
}

void DenseModel::load_weights(const std::string& model_dir) {
  SafetensorsDir st(model_dir);
  const DenseConfig& c = cfg_;
  const size_t H = (size_t)c.hidden, D = (size_t)c.head_dim;
  auto bf16 = [&](const std::string& name, std::vector<int64_t> shape) -> const TensorView& {
    const TensorView& t = st.get(name);
    if (t.dtype != "BF16") throw std::runtime_error(name + ": dtype " + t.dtype + " (the native runtime takes bf16 checkpoints)");
    if (t.shape != shape) throw std::runtime_error(name + ": unexpected shape");
    return t;
  };
  weight_bytes_ = 0;
  auto put = [&](const void* p, size_t n) {
    weight_bytes_ += (int64_t)n;
    return upload(p, n);
  };
  const TensorView& emb = bf16("model.embed_tokens.weight", {c.vocab_size, c.hidden});
  embed_ = put(emb.data, emb.nbytes);
  if (c.tie_embeddings || !st.has("lm_head.weight")) {
    lm_head_ = embed_;
  } else {
    const TensorView& lm = bf16("lm_head.weight", {c.vocab_size, c.hidden});
    lm_head_ = put(lm.data, lm.nbytes);
  }
  const TensorView& fn = bf16("model.norm.weight", {c.hidden});
  final_norm_ = put(fn.data, fn.nbytes);
  // On a GPU the merged gate / up projection is stored in blocks of [128 gate | 128 up] rows so
  // that the GEMM epilogue can apply the gated activation.
  gate_up_interleaved_ = dev_.cuda && c.inter % 128 == 0;
  layers_.clear();
  layers_.resize(c.layers);
  std::vector<uint8_t> stage;
  for (int l = 0; l < c.layers; ++l) {
    const std::string p = "model.layers." + std::to_string(l) + ".";
    Layer& L = layers_[l];
    const TensorView& q = bf16(p + "self_attn.q_proj.weight", {(int64_t)c.heads * c.head_dim, c.hidden});
    const TensorView& k = bf16(p + "self_attn.k_proj.weight", {(int64_t)c.kv_heads * c.head_dim, c.hidden});
    const TensorView& v = bf16(p + "self_attn.v_proj.weight", {(int64_t)c.kv_heads * c.head_dim, c.hidden});
    stage.resize(q.nbytes + k.nbytes + v.nbytes);
    std::memcpy(stage.data(), q.data, q.nbytes);
    std::memcpy(stage.data() + q.nbytes, k.data, k.nbytes);
    std::memcpy(stage.data() + q.nbytes + k.nbytes, v.data, v.nbytes);
    L.qkv = put(stage.data(), stage.size());
    const TensorView& o = bf16(p + "self_attn.o_proj.weight", {c.hidden, (int64_t)c.heads * c.head_dim});
    L.o = put(o.data, o.nbytes);
    const size_t row = H * 2;
    if (c.num_experts > 0) {
      const int E = c.num_experts, I = c.moe_inter;
      const TensorView& rt = bf16(p + "mlp.gate.weight", {E, c.hidden});
      L.router = put(rt.data, rt.nbytes);
      const size_t gu_bytes = (size_t)2 * I * row, dn_bytes = (size_t)c.hidden * I * 2;
      // experts are uploaded one at a time into the stacked device tensors (no host copy of all)
      L.w_gate_up = alloc((size_t)E * gu_bytes, dev_);
      L.w_down = alloc((size_t)E * dn_bytes, dev_);
      weight_bytes_ += (int64_t)E * (int64_t)(gu_bytes + dn_bytes);
      const bool stacked = st.has(p + "mlp.experts.gate_proj.weight");   // [E, I, H] / [E, H, I] tensors
      const TensorView* sg = stacked ? &bf16(p + "mlp.experts.gate_proj.weight", {E, I, c.hidden}) : nullptr;
      const TensorView* su = stacked ? &bf16(p + "mlp.experts.up_proj.weight", {E, I, c.hidden}) : nullptr;
      const TensorView* sd = stacked ? &bf16(p + "mlp.experts.down_proj.weight", {E, c.hidden, I}) : nullptr;
      for (int e = 0; e < E; ++e) {
        const uint8_t *gp, *up, *dp;
        const size_t half = (size_t)I * row;
        if (stacked) {
          gp = sg->data + (size_t)e * half;
          up = su->data + (size_t)e * half;
          dp = sd->data + (size_t)e * dn_bytes;
        } else {
          const std::string q2 = p + "mlp.experts." + std::to_string(e) + ".";
          gp = bf16(q2 + "gate_proj.weight", {I, c.hidden}).data;
          up = bf16(q2 + "up_proj.weight", {I, c.hidden}).data;
          dp = bf16(q2 + "down_proj.weight", {c.hidden, I}).data;
        }
        uint8_t* gu_dst = L.w_gate_up.as<uint8_t>() + (size_t)e * gu_bytes;
        copy(gu_dst, dev_, gp, Device{}, half);
        copy(gu_dst + half, dev_, up, Device{}, half);
        copy(L.w_down.as<uint8_t>() + (size_t)e * dn_bytes, dev_, dp, Device{}, dn_bytes);
      }
      if (dev_.cuda) synchronize(dev_);
    } else {
      const TensorView& g = bf16(p + "mlp.gate_proj.weight", {c.inter, c.hidden});
      const TensorView& u = bf16(p + "mlp.up_proj.weight", {c.inter, c.hidden});
      stage.resize(g.nbytes + u.nbytes);
      if (gate_up_interleaved_) {
        for (int b = 0; b < c.inter / 128; ++b) {
          std::memcpy(stage.data() + (size_t)(2 * b) * 128 * row, g.data + (size_t)b * 128 * row, 128 * row);
          std::memcpy(stage.data() + (size_t)(2 * b + 1) * 128 * row, u.data + (size_t)b * 128 * row, 128 * row);
        }
      } else {
        std::memcpy(stage.data(), g.data, g.nbytes);
        std::memcpy(stage.data() + g.nbytes, u.data, u.nbytes);
      }
      L.gate_up = put(stage.data(), stage.size());
      const TensorView& dn = bf16(p + "mlp.down_proj.weight", {c.hidden, c.inter});
      L.down = put(dn.data, dn.nbytes);
    }
    const TensorView& n1 = bf16(p + "input_layernorm.weight", {c.hidden});
    const TensorView& n2 = bf16(p + "post_attention_layernorm.weight", {c.hidden});
    L.ln1 = put(n1.data, n1.nbytes);
    L.ln2 = put(n2.data, n2.nbytes);
    if (c.qk_norm && st.has(p + "self_attn.q_norm.weight")) {
      const TensorView& qn = bf16(p + "self_attn.q_norm.weight", {c.head_dim});
      const TensorView& kn = bf16(p + "self_attn.k_norm.weight", {c.head_dim});
      L.q_norm = put(qn.data, qn.nbytes);
      L.k_norm = put(kn.data, kn.nbytes);
    }
  }
  (void)D;
}

int64_t DenseModel::kv_bytes_per_block(int block_size) const {
  return (int64_t)cfg_.layers * 2 * block_size * cfg_.kv_heads * cfg_.head_dim * 2;
}

void DenseModel::alloc_kv_cache(int64_t num_blocks, int block_size) {
  num_blocks_ = num_blocks;
  block_size_ = block_size;
  const size_t per_layer = (size_t)num_blocks * 2 * block_size * cfg_.kv_heads * cfg_.head_dim * 2;
  for (auto& L : layers_) L.kv_cache = alloc(per_layer, dev_, /*zero=*/true);
}

void DenseModel::reserve(int max_tokens, int max_reqs) {
  const DenseConfig& c = cfg_;
  max_tokens_ = max_tokens;
  max_reqs_ = max_reqs;
  const size_t T = (size_t)max_tokens, qkv_w = (size_t)(c.heads + 2 * c.kv_heads) * c.head_dim;
  hidden_ = alloc(T * c.hidden * 2, dev_);
  resid_ = alloc(T * c.hidden * 2, dev_);
  normed_ = alloc(T * c.hidden * 2, dev_);
  qkv_ = alloc(T * qkv_w * 2, dev_);
  attn_ = alloc(T * c.heads * c.head_dim * 2, dev_);
  gate_up_ = alloc(T * 2 * c.inter * 2, dev_);
  act_ = alloc(T * c.inter * 2, dev_);
  last_ = alloc((size_t)max_reqs * c.hidden * 2, dev_);
  logits_ = alloc((size_t)max_reqs * c.vocab_size * sizeof(float), dev_);
  if (dev_.cuda) gemm_ws_ = alloc(kGemmWsBytes, dev_);
  if (c.num_experts > 0) {
    const size_t P = T * c.experts_per_token, E = (size_t)c.num_experts;
    max_chunks_ = (int)(E + (P + 255) / 256);
    router_logits_ = alloc(T * E * sizeof(float), dev_);
    topk_ids_ = alloc(P * 4, dev_);
    topk_w_ = alloc(P * 4, dev_);
    moe_meta_ = alloc((3 * E + 2) * 4, dev_, true);
    sorted_token_ = alloc(P * 4, dev_, true);
    pair_pos_ = alloc(P * 4, dev_, true);
    chunk_expert_ = alloc((size_t)max_chunks_ * 4, dev_, true);
    chunk_row0_ = alloc((size_t)max_chunks_ * 4, dev_, true);
    chunk_n_ = alloc((size_t)max_chunks_ * 4, dev_, true);
    xs_ = alloc((P + 256) * c.hidden * 2, dev_, true);
    moe_act_ = alloc((P + 256) * c.moe_inter * 2, dev_, true);
    moe_y_ = alloc((P + 256) * c.hidden * 2, dev_, true);
  }
}

// ------------------------------------------------------------------------------- forward
float* DenseModel::forward(const StepInputs& in) {
  if (in.num_tokens <= 0) return logits_.as<float>();
  if (in.num_tokens > max_tokens_ || in.num_logits > max_reqs_)
    throw std::runtime_error("step exceeds the reserved activation buffers");
  set_device(dev_);
  if (dev_.cuda) forward_cuda(in);
  else forward_cpu(in);
  return logits_.as<float>();
}

void DenseModel::forward_cuda(const StepInputs& in) {
  const DenseConfig& c = cfg_;
  cudaStream_t s = (cudaStream_t)current_stream(dev_);
  const int T = in.num_tokens, H = c.hidden, Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim;
  check(b200_embedding(in.input_ids, embed_.data(), hidden_.data(), T, H, 0, c.vocab_size, c.vocab_size, 1.0f, s),
        "embedding");
  ++launches_;
  B200DenseStep st{};
  st.T = T; st.H = H; st.Hq = Hq; st.Hkv = Hkv; st.D = D; st.rot = rot_; st.inter = c.inter;
  st.block_size = block_size_;
  st.neox = 1; st.gemma = 0; st.act_kind = c.act_kind; st.gate_up_interleaved = gate_up_interleaved_ ? 1 : 0;
  st.eps = c.eps; st.scale = scale_; st.softcap = 0.f; st.window = 0;
  st.num_blocks = num_blocks_;
  st.positions = in.positions; st.cos_sin = rope_table_.data(); st.slot_mapping = in.slot_mapping;
  st.block_table = in.block_table; st.max_blocks = in.max_blocks; st.seq_lens = in.seq_lens;
  const int nd = in.num_decodes, G = Hq / Hkv;
  const bool tc = decode_uses_tc(D, G, block_size_);
  int splits = 1;
  if (nd > 0) {
    const int max_len = in.max_blocks * block_size_;
    if (tc) {
      const int ctas = nd * Hkv > 0 ? nd * Hkv : 1;
      const int want = (2 * b200_num_sms()) / ctas;
      const int tiles = (max_len + 127) / 128;
      splits = want;
      if (splits > tiles / 2) splits = tiles / 2;
      if (splits > 32) splits = 32;
      if (splits < 1) splits = 1;
    } else {
      splits = b200_attn_decode_splits(nd, Hkv, G, D, max_len);
      if (splits < 1) splits = 1;
    }
    if (splits > 1 && (nd > decode_tmp_batch_ || splits > decode_tmp_splits_)) {
      decode_tmp_batch_ = nd > decode_tmp_batch_ ? nd : decode_tmp_batch_;
      decode_tmp_splits_ = splits > decode_tmp_splits_ ? splits : decode_tmp_splits_;
      decode_tmp_o_ = alloc((size_t)decode_tmp_batch_ * Hq * decode_tmp_splits_ * D * sizeof(float), dev_);
      decode_tmp_lse_ = alloc((size_t)decode_tmp_batch_ * Hq * decode_tmp_splits_ * sizeof(float), dev_);
    }
  }
  st.num_decodes = nd; st.decode_splits = splits; st.decode_tc = tc ? 1 : 0;
  st.decode_tmp_o = decode_tmp_o_.data(); st.decode_tmp_lse = decode_tmp_lse_.data();
  st.num_prefills = in.num_prefills; st.num_tiles = in.num_tiles; st.num_prefill_tokens = T - nd;
  st.prefill_q_start = in.prefill_q_start; st.tile_req = in.tile_req; st.tile_q0 = in.tile_q0;
  st.hidden = hidden_.data(); st.resid = resid_.data(); st.normed = normed_.data();
  st.qkv_buf = qkv_.data(); st.attn = attn_.data(); st.gate_up_buf = gate_up_.data(); st.act = act_.data();
  st.gemm_ws = gemm_ws_.data(); st.gemm_ws_bytes = gemm_ws_.nbytes();
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = layers_[l];
    B200DenseLayerWeights w{};
    w.ln1 = L.ln1.data(); w.qkv = L.qkv.data(); w.q_norm = L.q_norm.data(); w.k_norm = L.k_norm.data();
    w.o = L.o.data(); w.ln2 = L.ln2.data(); w.gate_up = L.gate_up.data(); w.down = L.down.data();
    w.kv_cache = L.kv_cache.data();
    st.first_layer = l == 0;
    if (c.num_experts > 0) {
      const int rc = b200_dense_attn_half(&w, &st, s);
      check(rc, "attention half");
      launches_ += rc;
      check(b200_rmsnorm(hidden_.data(), H, resid_.data(), L.ln2.data(), normed_.data(), H, T, H, c.eps, 0, s),
            "post-attention norm");
      ++launches_;
      moe_cuda(L, T);
    } else {
      const int rc = b200_dense_layer(&w, &st, s);
      check(rc, "dense_layer");
      launches_ += rc;
    }
  }
  check(b200_rmsnorm(hidden_.data(), H, resid_.data(), final_norm_.data(), normed_.data(), H, T, H, c.eps, 0, s),
        "final norm");
  const int n = in.num_logits;
  check(b200_gather_rows(normed_.data(), in.logits_indices, last_.data(), n, T, H * 2, s), "gather_rows");
  check(b200_gemm_bf16(last_.data(), H, lm_head_.data(), H, logits_.data(), c.vocab_size, 1, nullptr, nullptr, 0, n,
                       c.vocab_size, H, gemm_ws_.data(), gemm_ws_.nbytes(), kConstW, s), "lm_head");
  launches_ += 3;
}

void DenseModel::forward_cpu(const StepInputs& in) {
  const DenseConfig& c = cfg_;
  const int T = in.num_tokens, H = c.hidden, Hq = c.heads, Hkv = c.kv_heads, D = c.head_dim, I = c.inter;
  const int qkv_w = (Hq + 2 * Hkv) * D;
  auto* hidden = hidden_.as<uint16_t>();
  auto* resid = resid_.as<uint16_t>();
  auto* normed = normed_.as<uint16_t>();
  auto* qkv = qkv_.as<uint16_t>();
  auto* attn = attn_.as<uint16_t>();
  auto* gate_up = gate_up_.as<uint16_t>();
  auto* act = act_.as<uint16_t>();
  b200cpu_embedding(in.input_ids, embed_.as<uint16_t>(), hidden, H, T, H, 0, c.vocab_size, 1.0f);
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = layers_[l];
    if (l == 0) {
      std::memcpy(resid, hidden, (size_t)T * H * 2);
      b200cpu_rmsnorm(hidden, H, L.ln1.as<uint16_t>(), c.eps, nullptr, 0, normed, H, T, H, 0);
    } else {
      b200cpu_rmsnorm(hidden, H, L.ln1.as<uint16_t>(), c.eps, resid, H, normed, H, T, H, 0);
    }
    b200cpu_matmul_bt(normed, H, L.qkv.as<uint16_t>(), H, qkv, qkv_w, 0, nullptr, nullptr, 0, T, qkv_w, H);
    b200cpu_rope_kv(qkv, qkv_w, in.positions, rope_table_.as<float>(), T, Hq, Hkv, D, rot_, 1,
                    L.q_norm.as<uint16_t>(), L.k_norm.as<uint16_t>(), c.eps, 0, in.slot_mapping,
                    L.kv_cache.as<uint16_t>(), block_size_);
    b200cpu_paged_attention(qkv, qkv_w, L.kv_cache.as<uint16_t>(), in.block_table, in.max_blocks, in.seq_lens,
                            in.query_start, in.num_reqs, Hq, Hkv, D, block_size_, scale_, 0.f, 0, attn, Hq * D);
    b200cpu_matmul_bt(attn, Hq * D, L.o.as<uint16_t>(), Hq * D, hidden, H, 0, nullptr, nullptr, 0, T, H, Hq * D);
    b200cpu_rmsnorm(hidden, H, L.ln2.as<uint16_t>(), c.eps, resid, H, normed, H, T, H, 0);
    if (c.num_experts > 0) {
      moe_cpu(L, T);
      continue;
    }
    b200cpu_matmul_bt(normed, H, L.gate_up.as<uint16_t>(), H, gate_up, 2 * I, 0, nullptr, nullptr, 0, T, 2 * I, H);
    b200cpu_act_and_mul(gate_up, 2 * I, act, I, T, I, c.act_kind);
    b200cpu_matmul_bt(act, I, L.down.as<uint16_t>(), I, hidden, H, 0, nullptr, nullptr, 0, T, H, I);
  }
  b200cpu_rmsnorm(hidden, H, final_norm_.as<uint16_t>(), c.eps, resid, H, normed, H, T, H, 0);
  auto* last = last_.as<uint16_t>();
  for (int i = 0; i < in.num_logits; ++i)
    std::memcpy(last + (size_t)i * H, normed + (size_t)in.logits_indices[i] * H, (size_t)H * 2);
  b200cpu_matmul_bt(last, H, lm_head_.as<uint16_t>(), H, logits_.data(), c.vocab_size, 1, nullptr, nullptr, 0,
                    in.num_logits, c.vocab_size, H);
}


// ------------------------------------------------------------------------------- experts
// Router GEMM (fp32 logits) -> softmax top-k -> device-side sort by expert -> gather -> grouped
// gate/up GEMM with the gated activation in its epilogue -> grouped down GEMM -> weighted combine
// into hidden_. Reference: src/vt/cuda/cuda_moe.cu:62,406 and qwen3_moe.cpp.
void DenseModel::moe_cuda(const Layer& L, int T) {
  const DenseConfig& c = cfg_;
  cudaStream_t s = (cudaStream_t)current_stream(dev_);
  const int H = c.hidden, E = c.num_experts, k = c.experts_per_token, I = c.moe_inter, P = T * k;
  check(b200_gemm_bf16(normed_.data(), H, L.router.data(), H, router_logits_.data(), E, 1, nullptr, nullptr, 0, T, E,
                       H, gemm_ws_.data(), gemm_ws_.nbytes(), kConstW, s), "router");
  check(b200_moe_router_topk(router_logits_.data(), E, T, E, k, c.norm_topk_prob ? 1 : 0, 0, nullptr, 1, 1, 1.0f,
                             topk_ids_.data(), topk_w_.data(), s), "router_topk");
  check(b200_moe_sort(topk_ids_.data(), T, k, 0, E, moe_meta_.data(), sorted_token_.data(), pair_pos_.data(),
                      chunk_expert_.data(), chunk_row0_.data(), chunk_n_.data(), max_chunks_, s), "moe_sort");
  check(b200_moe_gather(normed_.data(), H, sorted_token_.data(), moe_meta_.data(), E, xs_.data(), H, P, s),
        "moe_gather");
  int chunks = E + (P + 255) / 256;
  if (chunks > max_chunks_) chunks = max_chunks_;
  check(b200_moe_grouped_gemm_gated(xs_.data(), P, L.w_gate_up.data(), E, 2 * I, H, moe_act_.data(),
                                    chunk_expert_.data(), chunk_row0_.data(), chunk_n_.data(), moe_meta_.data(),
                                    chunks, c.act_kind, s), "experts gate/up");
  check(b200_moe_grouped_gemm(moe_act_.data(), P, L.w_down.data(), E, H, I, moe_y_.data(), chunk_expert_.data(),
                              chunk_row0_.data(), chunk_n_.data(), moe_meta_.data(), chunks, s), "experts down");
  check(b200_moe_combine(moe_y_.data(), pair_pos_.data(), topk_w_.data(), T, k, H, nullptr, nullptr, hidden_.data(),
                         nullptr, s), "moe_combine");
  launches_ += 7;
}

// The same block on the host: the thread-pool GEMM per expert over its gathered rows; fp32
// accumulation per token in ascending expert order, one bf16 rounding at the end.
void DenseModel::moe_cpu(const Layer& L, int T) {
  const DenseConfig& c = cfg_;
  const int H = c.hidden, E = c.num_experts, k = c.experts_per_token, I = c.moe_inter;
  const uint16_t* x = normed_.as<uint16_t>();
  float* logits = router_logits_.as<float>();
  b200cpu_matmul_bt(x, H, L.router.as<uint16_t>(), H, logits, E, 1, nullptr, nullptr, 0, T, E, H);
  std::vector<std::vector<int>> rows_of(E);
  std::vector<std::vector<float>> weight_of(E);
  std::vector<float> score(E);
  for (int t = 0; t < T; ++t) {
    const float* lr = logits + (size_t)t * E;
    float mx = lr[0];
    for (int e = 1; e < E; ++e) mx = std::max(mx, lr[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { score[e] = std::exp(lr[e] - mx); sum += score[e]; }
    for (int e = 0; e < E; ++e) score[e] /= sum;
    int ids[64];
    float w[64], wsum = 0.f;
    std::vector<char> taken(E, 0);
    for (int j = 0; j < k && j < 64; ++j) {       // ties go to the lowest expert index
      int best = -1;
      for (int e = 0; e < E; ++e)
        if (!taken[e] && (best < 0 || score[e] > score[best])) best = e;
      taken[best] = 1;
      ids[j] = best;
      w[j] = score[best];
      wsum += w[j];
    }
    for (int j = 0; j < k && j < 64; ++j) {
      rows_of[ids[j]].push_back(t);
      weight_of[ids[j]].push_back(c.norm_topk_prob && wsum > 0 ? w[j] / wsum : w[j]);
    }
  }
  std::vector<float> acc((size_t)T * H, 0.f);
  std::vector<uint16_t> xs, gu, a, y;
  const size_t gu_elems = (size_t)2 * I * H, dn_elems = (size_t)H * I;
  for (int e = 0; e < E; ++e) {
    const int n = (int)rows_of[e].size();
    if (n == 0) continue;
    xs.resize((size_t)n * H);
    gu.resize((size_t)n * 2 * I);
    a.resize((size_t)n * I);
    y.resize((size_t)n * H);
    for (int r = 0; r < n; ++r) std::memcpy(xs.data() + (size_t)r * H, x + (size_t)rows_of[e][r] * H, (size_t)H * 2);
    b200cpu_matmul_bt(xs.data(), H, L.w_gate_up.as<uint16_t>() + (size_t)e * gu_elems, H, gu.data(), 2 * I, 0, nullptr,
                      nullptr, 0, n, 2 * I, H);
    b200cpu_act_and_mul(gu.data(), 2 * I, a.data(), I, n, I, c.act_kind);
    b200cpu_matmul_bt(a.data(), I, L.w_down.as<uint16_t>() + (size_t)e * dn_elems, I, y.data(), H, 0, nullptr, nullptr, 0,
                      n, H, I);
    for (int r = 0; r < n; ++r) {
      float* dst = acc.data() + (size_t)rows_of[e][r] * H;
      const float wt = weight_of[e][r];
      const uint16_t* src = y.data() + (size_t)r * H;
      for (int i = 0; i < H; ++i) {
        uint32_t bits = (uint32_t)src[i] << 16;
        float v;
        std::memcpy(&v, &bits, 4);
        dst[i] += wt * v;
      }
    }
  }
  uint16_t* out = hidden_.as<uint16_t>();
  for (size_t i = 0; i < acc.size(); ++i) {
    uint32_t bits;
    std::memcpy(&bits, &acc[i], 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {          // NaN stays NaN
      out[i] = (uint16_t)((bits >> 16) | 0x40);
    } else {
      bits += 0x7fffu + ((bits >> 16) & 1);            // round to nearest even
      out[i] = (uint16_t)(bits >> 16);
    }
  }
}

}  // namespace b200::rt
