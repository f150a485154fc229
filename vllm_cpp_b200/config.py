"""Typed configuration: model architecture (from a HF ``config.json`` or a named synthetic
shape), engine arguments and the parallel layout.

Reference surface: ``include/vllm/transformers_utils/hf_config.h`` (typed config incl.
``text_config`` nesting and RoPE parameter normalisation), ``include/vllm/entrypoints/
model_loader.h:36-75`` (EngineParams) and ``include/vllm/config/scheduler.h``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class RopeConfig:
    theta: float = 10000.0
    rotary_dim: Optional[int] = None          # None => head_dim
    neox: bool = True                         # False => GPT-J (interleaved pairs)
    scaling_type: Optional[str] = None        # llama3 | yarn | deepseek_yarn | linear | dynamic | longrope | mrope
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    attn_factor: float = 1.0
    short_factor: Optional[list] = None       # longrope
    long_factor: Optional[list] = None
    mrope_section: Optional[list] = None
    alpha: Optional[float] = None             # dynamic NTK alpha
    config_max_position: int = 0              # the checkpoint's max_position_embeddings (longrope magnitude scale)
    short_mscale: Optional[float] = None      # longrope: explicit magnitude scales, when the checkpoint gives them
    long_mscale: Optional[float] = None
    truncate: bool = True                     # YaRN: round the correction range outward to whole dimensions
    extrapolation_factor: float = 1.0         # YaRN: weight of the unscaled frequencies inside the ramp
    apply_yarn_scaling: bool = True           # YaRN: False keeps only attn_factor as the magnitude scale


@dataclass
class ModelConfig:
    architecture: str = "LlamaForCausalLM"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    rope: RopeConfig = field(default_factory=RopeConfig)
    qk_norm: bool = False                     # per-head RMSNorm on q and k (Qwen3)
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    sliding_window: int = 0
    attention_chunk_size: int = 0             # chunked-local attention ("chunked_attention" layers)
    # layer pattern / extras for the non-plain families
    layer_types: Optional[list] = None        # per-layer "full_attention" | "sliding_attention" | "chunked_attention" | "linear_attention"
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    embed_scale: float = 1.0
    gemma_norm: bool = False                  # (1 + w) RMSNorm weights
    sandwich_norm: bool = False               # post-attention / post-mlp norms (Gemma2/3, GLM4)
    post_norm: bool = False                   # OLMo2-style: norm after the block, not before
    residual_multiplier: float = 1.0          # Granite
    attention_multiplier: Optional[float] = None
    logits_scaling: float = 1.0
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    num_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    first_k_dense_replace: int = 0
    routed_scaling_factor: float = 1.0
    scoring_func: str = "softmax"
    topk_method: str = "greedy"
    n_group: int = 1
    mtp_num_hidden_layers: int = 0            # decoder blocks of the multi-token-prediction head (0: none in the checkpoint)
    topk_group: int = 1
    # MLA
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # Gated DeltaNet (Qwen3.5 / 3.6)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    full_attention_interval: int = 4
    attn_output_gate: bool = False
    partial_rotary_factor: float = 1.0
    # quantisation
    quant: Optional[str] = None               # None | "nvfp4" | "fp8"
    dtype: str = "bfloat16"
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    raw: dict = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_hybrid(self) -> bool:
        return bool(self.layer_types) and "linear_attention" in self.layer_types


def _rope_from_hf(cfg: dict, head_dim: int) -> RopeConfig:
    r = RopeConfig(theta=float(cfg.get("rope_theta", 10000.0)))
    prf = cfg.get("partial_rotary_factor")
    if prf is not None and prf < 1.0:
        r.rotary_dim = int(head_dim * prf)
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or None
    if rs:
        if "rope_theta" in rs:
            r.theta = float(rs["rope_theta"])
        if "partial_rotary_factor" in rs and rs["partial_rotary_factor"] < 1.0:
            r.rotary_dim = int(head_dim * rs["partial_rotary_factor"])
        t = rs.get("rope_type", rs.get("type"))
        if t and t != "default":
            r.scaling_type = t
        r.factor = float(rs.get("factor", 1.0))
        r.low_freq_factor = float(rs.get("low_freq_factor", 1.0))
        r.high_freq_factor = float(rs.get("high_freq_factor", 4.0))
        # Phi-3 keeps the original window beside rope_scaling, not inside it
        r.original_max_position = int(rs.get("original_max_position_embeddings",
                                             cfg.get("original_max_position_embeddings",
                                                     cfg.get("max_position_embeddings", 8192))))
        r.config_max_position = int(cfg.get("max_position_embeddings", 0) or 0)
        r.beta_fast = float(rs.get("beta_fast", 32.0))
        r.beta_slow = float(rs.get("beta_slow", 1.0))
        r.mscale = float(rs.get("mscale", 1.0))
        r.mscale_all_dim = float(rs.get("mscale_all_dim", 0.0))
        r.attn_factor = float(rs.get("attn_factor", 1.0))
        r.short_factor = rs.get("short_factor")
        r.long_factor = rs.get("long_factor")
        r.mrope_section = rs.get("mrope_section")
        r.alpha = rs.get("alpha")
        r.short_mscale, r.long_mscale = rs.get("short_mscale"), rs.get("long_mscale")
        r.truncate = bool(rs.get("truncate", True))
        r.extrapolation_factor = float(rs.get("extrapolation_factor", 1.0))
        r.apply_yarn_scaling = bool(rs.get("apply_yarn_scaling", True))
    return r


def model_config_from_hf(cfg: dict) -> ModelConfig:
    """Builds a ModelConfig from a HF ``config.json`` dict (``text_config`` nesting honoured)."""
    arch = (cfg.get("architectures") or ["LlamaForCausalLM"])[0]
    t = dict(cfg)
    if "text_config" in cfg:
        t.update(cfg["text_config"])
    hidden = int(t["hidden_size"])
    heads = int(t["num_attention_heads"])
    head_dim = int(t.get("head_dim") or hidden // heads)
    m = ModelConfig(
        architecture=arch, vocab_size=int(t["vocab_size"]), hidden_size=hidden,
        intermediate_size=int(t.get("intermediate_size", 4 * hidden)),
        num_layers=int(t["num_hidden_layers"]), num_heads=heads,
        num_kv_heads=int(t.get("num_key_value_heads", heads)), head_dim=head_dim,
        rms_norm_eps=float(t.get("rms_norm_eps", t.get("layer_norm_eps", 1e-6))),
        max_position_embeddings=int(t.get("max_position_embeddings", 8192)),
        tie_word_embeddings=bool(t.get("tie_word_embeddings", False)),
        rope=_rope_from_hf(t, head_dim), attention_bias=bool(t.get("attention_bias", False)),
        mlp_bias=bool(t.get("mlp_bias", False)), hidden_act=t.get("hidden_act", "silu"),
        sliding_window=int(t.get("sliding_window") or 0), layer_types=t.get("layer_types"),
        attention_chunk_size=int(t.get("attention_chunk_size") or 0),
        raw=cfg)
    eos = t.get("eos_token_id")
    m.eos_token_id = eos[0] if isinstance(eos, list) else eos
    m.bos_token_id = t.get("bos_token_id")
    a = arch
    if a in ("Qwen3ForCausalLM", "Qwen3MoeForCausalLM"):
        m.qk_norm = True
    if a in ("Qwen3MoeForCausalLM",):
        m.num_experts = int(t["num_experts"])
        m.num_experts_per_tok = int(t["num_experts_per_tok"])
        m.moe_intermediate_size = int(t["moe_intermediate_size"])
        m.norm_topk_prob = bool(t.get("norm_topk_prob", True))
    if a in ("DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM", "Glm4MoeLiteForCausalLM"):
        m.kv_lora_rank = int(t["kv_lora_rank"])
        m.q_lora_rank = int(t.get("q_lora_rank") or 0)
        m.qk_nope_head_dim = int(t["qk_nope_head_dim"])
        m.qk_rope_head_dim = int(t["qk_rope_head_dim"])
        m.v_head_dim = int(t["v_head_dim"])
        m.num_experts = int(t.get("n_routed_experts", 0))
        m.num_experts_per_tok = int(t.get("num_experts_per_tok", 0))
        m.moe_intermediate_size = int(t.get("moe_intermediate_size", 0))
        m.num_shared_experts = int(t.get("n_shared_experts") or 0)
        m.first_k_dense_replace = int(t.get("first_k_dense_replace", 0))
        m.routed_scaling_factor = float(t.get("routed_scaling_factor", 1.0))
        m.norm_topk_prob = bool(t.get("norm_topk_prob", False))
        m.scoring_func = t.get("scoring_func", "softmax")
        m.topk_method = t.get("topk_method", "greedy")
        m.n_group = int(t.get("n_group") or 1)
        m.mtp_num_hidden_layers = int(t.get("mtp_num_hidden_layers") or 0)
        m.topk_group = int(t.get("topk_group") or 1)
        m.rope.neox = False
        if m.rope.scaling_type == "yarn":
            m.rope.scaling_type = "deepseek_yarn"
    if a.startswith("Gemma"):
        m.gemma_norm = True
        m.embed_scale = hidden ** 0.5
        m.hidden_act = "gelu_tanh"
        m.attn_logit_softcap = float(t.get("attn_logit_softcapping") or 0.0)
        m.final_logit_softcap = float(t.get("final_logit_softcapping") or 0.0)
        m.sandwich_norm = a in ("Gemma2ForCausalLM", "Gemma3ForCausalLM")
        m.qk_norm = a == "Gemma3ForCausalLM"
        if t.get("query_pre_attn_scalar"):
            m.attention_multiplier = float(t["query_pre_attn_scalar"]) ** -0.5
        m.tie_word_embeddings = True
    if a == "GraniteForCausalLM":
        m.residual_multiplier = float(t.get("residual_multiplier", 1.0))
        m.attention_multiplier = float(t.get("attention_multiplier", head_dim ** -0.5))
        m.embed_scale = float(t.get("embedding_multiplier", 1.0))
        m.logits_scaling = float(t.get("logits_scaling", 1.0))
    if a in ("Olmo2ForCausalLM", "Olmo3ForCausalLM"):
        m.post_norm = True
        m.qk_norm = True
    if a in ("Glm4ForCausalLM",):
        m.sandwich_norm = True
        m.rope.neox = False
        m.attention_bias = bool(t.get("attention_bias", True))
    if a in ("Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration",
             "Qwen3NextForCausalLM"):
        m.qk_norm = True
        m.gemma_norm = True
        m.attn_output_gate = True
        m.linear_num_key_heads = int(t.get("linear_num_key_heads", 16))
        m.linear_num_value_heads = int(t.get("linear_num_value_heads", 32))
        m.linear_key_head_dim = int(t.get("linear_key_head_dim", 128))
        m.linear_value_head_dim = int(t.get("linear_value_head_dim", 128))
        m.linear_conv_kernel_dim = int(t.get("linear_conv_kernel_dim", 4))
        m.full_attention_interval = int(t.get("full_attention_interval", 4))
        if not m.layer_types:
            m.layer_types = ["full_attention" if (i + 1) % m.full_attention_interval == 0
                             else "linear_attention" for i in range(m.num_layers)]
        if "num_experts" in t and t["num_experts"]:
            m.num_experts = int(t["num_experts"])
            m.num_experts_per_tok = int(t["num_experts_per_tok"])
            m.moe_intermediate_size = int(t["moe_intermediate_size"])
            m.shared_expert_intermediate_size = int(t.get("shared_expert_intermediate_size", 0))
            m.num_shared_experts = 1 if m.shared_expert_intermediate_size else 0
            m.shared_expert_gate = True
    q = t.get("quantization_config") or {}
    if q:
        method = (q.get("quant_method") or "").lower()
        algo = (q.get("quant_algo") or "").lower()
        if "nvfp4" in json.dumps(q).lower() or algo == "nvfp4":
            m.quant = "nvfp4"
        elif method == "fp8" or algo == "fp8":
            m.quant = "fp8"
    return m


def load_model_config(model_dir: str) -> ModelConfig:
    with open(os.path.join(model_dir, "config.json")) as f:
        return model_config_from_hf(json.load(f))


# ------------------------------------------------------------------ named synthetic shapes
def synthetic_config(name: str) -> ModelConfig:
    """Architectures of the benchmark configurations (random-init weights). A ``+fp8`` or ``+nvfp4``
    suffix selects that weight quantisation (``llama-3.1-8b+fp8``), ``+bf16`` none."""
    n = name.lower()
    if "+" in n:
        base, q = n.rsplit("+", 1)
        if q not in ("fp8", "nvfp4", "bf16"):
            raise ValueError(f"unknown quantisation suffix '+{q}'")
        cfg = synthetic_config(base)
        cfg.quant = None if q == "bf16" else q
        return cfg
    if n in ("qwen3-0.6b", "qwen3_0_6b"):
        return ModelConfig(architecture="Qwen3ForCausalLM", vocab_size=151936, hidden_size=1024,
                           intermediate_size=3072, num_layers=28, num_heads=16, num_kv_heads=8,
                           head_dim=128, rms_norm_eps=1e-6, max_position_embeddings=40960,
                           tie_word_embeddings=True, qk_norm=True, rope=RopeConfig(theta=1e6))
    if n in ("llama-3.1-8b", "llama3.1-8b", "llama_3_1_8b"):
        return ModelConfig(architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=4096,
                           intermediate_size=14336, num_layers=32, num_heads=32, num_kv_heads=8,
                           head_dim=128, rms_norm_eps=1e-5, max_position_embeddings=131072,
                           rope=RopeConfig(theta=5e5, scaling_type="llama3", factor=8.0,
                                           low_freq_factor=1.0, high_freq_factor=4.0,
                                           original_max_position=8192))
    if n in ("qwen3-coder-30b-a3b", "qwen3-30b-a3b"):
        return ModelConfig(architecture="Qwen3MoeForCausalLM", vocab_size=151936, hidden_size=2048,
                           intermediate_size=6144, num_layers=48, num_heads=32, num_kv_heads=4,
                           head_dim=128, rms_norm_eps=1e-6, max_position_embeddings=262144,
                           qk_norm=True, rope=RopeConfig(theta=1e7), num_experts=128,
                           num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True)
    if n in ("deepseek-v2-lite",):
        return ModelConfig(architecture="DeepseekV2ForCausalLM", vocab_size=102400,
                           hidden_size=2048, intermediate_size=10944, num_layers=27, num_heads=16,
                           num_kv_heads=16, head_dim=192, rms_norm_eps=1e-6,
                           max_position_embeddings=163840,
                           rope=RopeConfig(theta=10000.0, neox=False, scaling_type="deepseek_yarn",
                                           factor=40.0, original_max_position=4096, beta_fast=32,
                                           beta_slow=1, mscale=0.707, mscale_all_dim=0.707,
                                           rotary_dim=64),
                           num_experts=64, num_experts_per_tok=6, moe_intermediate_size=1408,
                           num_shared_experts=2, first_k_dense_replace=1, norm_topk_prob=False,
                           kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                           v_head_dim=128)
    if n in ("qwen3.6-27b", "qwen3_6_27b"):
        L = 64
        return ModelConfig(architecture="Qwen3_5ForConditionalGeneration", vocab_size=248320,
                           hidden_size=5120, intermediate_size=17408, num_layers=L, num_heads=24,
                           num_kv_heads=4, head_dim=256, rms_norm_eps=1e-6,
                           max_position_embeddings=262144, qk_norm=True, gemma_norm=True,
                           attn_output_gate=True,
                           rope=RopeConfig(theta=1e7, rotary_dim=64),
                           layer_types=["full_attention" if (i + 1) % 4 == 0 else
                                        "linear_attention" for i in range(L)],
                           linear_num_key_heads=16, linear_num_value_heads=48,
                           linear_key_head_dim=128, linear_value_head_dim=128,
                           linear_conv_kernel_dim=4, quant="nvfp4")
    if n.startswith("tiny"):
        # small shapes for tests: tiny-dense, tiny-moe, tiny-mla, tiny-gdn
        base = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_layers=2,
                    num_heads=4, num_kv_heads=2, head_dim=64, rms_norm_eps=1e-6,
                    max_position_embeddings=2048, rope=RopeConfig(theta=1e4))
        if n == "tiny-dense":
            return ModelConfig(architecture="LlamaForCausalLM", **base)
        if n == "tiny-qwen3":
            return ModelConfig(architecture="Qwen3ForCausalLM", qk_norm=True,
                               tie_word_embeddings=True, **base)
        if n == "tiny-opt":
            return ModelConfig(architecture="OPTForCausalLM", hidden_act="relu", tie_word_embeddings=True,
                               **{**base, "num_kv_heads": 4})
        if n == "tiny-mla":
            base.update(head_dim=192, num_heads=4, num_kv_heads=4)
            return ModelConfig(architecture="DeepseekV2ForCausalLM", num_experts=8, num_experts_per_tok=2,
                               moe_intermediate_size=128, num_shared_experts=1, first_k_dense_replace=1,
                               norm_topk_prob=False, kv_lora_rank=512, qk_nope_head_dim=128,
                               qk_rope_head_dim=64, v_head_dim=128,
                               **{**base, "rope": RopeConfig(theta=1e4, neox=False, rotary_dim=64)})
        if n == "tiny-gdn":
            base.update(num_layers=4, head_dim=256, num_heads=2, num_kv_heads=1)
            return ModelConfig(architecture="Qwen3_5ForConditionalGeneration", qk_norm=True,
                               gemma_norm=True, attn_output_gate=True,
                               layer_types=["full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                                            for i in range(4)],
                               linear_num_key_heads=2, linear_num_value_heads=4,
                               linear_key_head_dim=128, linear_value_head_dim=128,
                               linear_conv_kernel_dim=4, tie_word_embeddings=True,
                               **{**base, "rope": RopeConfig(theta=1e4, rotary_dim=64)})
        if n == "tiny-gdn-moe":
            base.update(num_layers=4, head_dim=256, num_heads=2, num_kv_heads=1)
            return ModelConfig(architecture="Qwen3_5MoeForConditionalGeneration", qk_norm=True,
                               gemma_norm=True, attn_output_gate=True,
                               layer_types=["full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                                            for i in range(4)],
                               linear_num_key_heads=2, linear_num_value_heads=4,
                               linear_key_head_dim=128, linear_value_head_dim=128,
                               linear_conv_kernel_dim=4, tie_word_embeddings=True,
                               num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                               shared_expert_intermediate_size=256, num_shared_experts=1,
                               shared_expert_gate=True, norm_topk_prob=True,
                               **{**base, "rope": RopeConfig(theta=1e4, rotary_dim=64)})
        if n == "tiny-moe":
            return ModelConfig(architecture="Qwen3MoeForCausalLM", qk_norm=True, num_experts=8,
                               num_experts_per_tok=2, moe_intermediate_size=128, **base)
    raise KeyError(f"unknown synthetic model shape: {name}")


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    enable_expert_parallel: bool = False
    rank: int = 0
    local_rank: int = 0
    fused_collectives: bool = True      # False => GEMM kernel + NCCL call (the baseline mode)
    # True: rank 0 owns the scheduler and publishes every step to the other ranks, which run
    # ``LLM.serve_as_worker()`` and never see a request (serving). False: every rank runs its own
    # scheduler and must be fed identical requests (offline batches driven by one script per rank).
    driver_worker: bool = False
    # Expert-parallel load balancing (parallel/eplb.py): redundant physical expert slots (the
    # total must divide over the ranks), steps between rebalances, steps of load history used.
    enable_eplb: bool = False
    eplb_redundant_experts: int = 0
    eplb_interval: int = 3000
    eplb_window: int = 1000
    # Decode context parallelism (KV of one sequence split over ranks). Only 1 is implemented:
    # long prompts are handled by chunked prefill over the paged cache. The field exists so that
    # KV-cache specs and attention metadata carry the degree (reference: dcp_world_size = 1 fixed
    # in src/vllm/v1/core/sched/scheduler.cpp:78-79).
    dcp_world_size: int = 1

    def __post_init__(self):
        if self.dcp_world_size != 1:
            raise ValueError("decode context parallelism is not implemented: dcp_world_size must be 1")

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size


@dataclass
class EngineArgs:
    model: Optional[str] = None                 # directory / .gguf, or None with model_config set
    model_config: Optional[ModelConfig] = None
    block_size: int = 32
    num_blocks: int = 0                         # 0 => size from gpu_memory_utilization
    gpu_memory_utilization: float = 0.90
    max_model_len: int = 0                      # 0 => config.max_position_embeddings
    max_num_seqs: int = 8
    max_num_batched_tokens: int = 0             # 0 => dense 2048 / MoE 4096 (8192 at >= 32 seqs)
    enable_prefix_caching: Optional[bool] = None  # None => on unless hybrid
    scheduling_policy: str = "fcfs"
    async_scheduling: Optional[bool] = None
    # spec_decode.SpeculativeConfig; method "ngram" is wired through the engine (prompt-lookup
    # drafts, argmax verification), the other methods have their building blocks only
    speculative_config: Optional[object] = None
    # device "cpu": "torch" = the fp32 PyTorch oracle the GPU path is compared with,
    # "native" = the C++ thread-pool backend (csrc/cpu)
    cpu_backend: str = "torch"
    # CPU only: keep the linear-layer weights in GGUF blocks ("q8_0" | "q4_0") and run the GEMMs on
    # the packed form (integer block dot products); None keeps bf16 weights
    cpu_weight_quant: Optional[str] = None
    enable_cuda_graphs: bool = True
    seed: int = 0
    device: str = "cuda"
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    tokenizer: Optional[str] = None
    kv_transfer_config: Optional[dict] = None

    def resolve_max_num_batched_tokens(self, cfg: ModelConfig) -> int:
        if self.max_num_batched_tokens > 0:
            return self.max_num_batched_tokens
        if cfg.is_moe:
            return 8192 if self.max_num_seqs >= 32 else 4096
        return 2048

    def resolve_prefix_caching(self, cfg: ModelConfig) -> bool:
        if self.enable_prefix_caching is not None:
            return self.enable_prefix_caching
        return not cfg.is_hybrid
