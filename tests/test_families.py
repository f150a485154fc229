"""Every switch of the dense family block, through its own HF config: Gemma-2 (GeGLU, soft-caps,
sandwich norms, alternating sliding-window layers), Gemma-3 (per-head qk-norm), Phi-3 (LongRoPE
factors), Granite (embedding / residual / attention / logits multipliers), OLMo-2 (post-norm,
qk-norm), GLM-4 (partial interleaved RoPE, sandwich norms, attention bias), Mistral, Qwen3.

CPU part: each config builds, generates and is deterministic on the fp32 oracle. GPU part
(``-m gpu``): the kernels' logits of a prefill step against the oracle's, numerically, and greedy
agreement. Reference: src/vllm/model_executor/models/{gemma2,gemma3,phi3,granite,olmo2,glm4}.cpp."""
import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, model_config_from_hf
from vllm_cpp_b200.engine import LLM, SamplingParams

BASE = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, max_position_embeddings=2048,
            rope_theta=10000.0)

FAMILIES = {
    "mistral": dict(architectures=["MistralForCausalLM"]),
    "qwen3": dict(architectures=["Qwen3ForCausalLM"], tie_word_embeddings=True),
    "gemma2": dict(architectures=["Gemma2ForCausalLM"], attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                   query_pre_attn_scalar=64, sliding_window=32,
                   layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
    "gemma3": dict(architectures=["Gemma3ForCausalLM"], query_pre_attn_scalar=64, sliding_window=32,
                   layer_types=["sliding_attention", "sliding_attention", "full_attention"]),
    "phi3": dict(architectures=["Phi3ForCausalLM"], max_position_embeddings=4096,
                 rope_scaling=dict(type="longrope", short_factor=[1.0 + 0.01 * i for i in range(32)],
                                   long_factor=[1.5 + 0.02 * i for i in range(32)],
                                   original_max_position_embeddings=1024)),
    "granite": dict(architectures=["GraniteForCausalLM"], residual_multiplier=0.22, attention_multiplier=0.0625,
                    embedding_multiplier=12.0, logits_scaling=8.0),
    "olmo2": dict(architectures=["Olmo2ForCausalLM"]),
    "glm4": dict(architectures=["Glm4ForCausalLM"], partial_rotary_factor=0.5, attention_bias=True),
    # chunked-local attention (Llama-4 style layer pattern): a query attends inside its own 32-token chunk
    "chunked": dict(architectures=["LlamaForCausalLM"], attention_chunk_size=32,
                    layer_types=["chunked_attention", "chunked_attention", "full_attention"]),
}


def config_of(name):
    return model_config_from_hf({**BASE, **FAMILIES[name]})


def prompts_of(cfg):
    g = torch.Generator().manual_seed(9)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 9, 41)]


def build(cfg, device, **kw):
    return LLM(EngineArgs(model_config=cfg, device=device, block_size=16, num_blocks=128, max_model_len=512,
                          max_num_seqs=4, max_num_batched_tokens=256, **kw))


@pytest.mark.parametrize("name", sorted(FAMILIES))
def test_family_config_runs_on_the_oracle(name):
    cfg = config_of(name)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a = [o.outputs[0].token_ids for o in build(cfg, "cpu").generate(prompts_of(cfg), sp)]
    b = [o.outputs[0].token_ids for o in build(cfg, "cpu").generate(prompts_of(cfg), sp)]
    assert a == b and all(len(x) == 6 for x in a)
    assert all(0 <= t < cfg.vocab_size for x in a for t in x)


def test_chunked_local_attention_changes_the_result_and_groups_the_layers():
    """The chunk mask is live (long prompts decode differently from the same weights with full
    attention) and chunked layers get their own KV-cache group."""
    cfg = config_of("chunked")
    assert cfg.attention_chunk_size == 32
    plain = model_config_from_hf({**BASE, "architectures": ["LlamaForCausalLM"]})
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a, b = build(cfg, "cpu"), build(plain, "cpu")
    assert [len(g[0]) for g in a.model.kv_cache_groups(16)] == [1, 2]
    assert a.model._layer_window(0) == -32 and a.model._layer_window(2) == 0
    pa = [o.outputs[0].token_ids for o in a.generate(prompts_of(cfg), sp)]
    pb = [o.outputs[0].token_ids for o in b.generate(prompts_of(cfg), sp)]
    assert pa != pb
    # a prompt that fits in one chunk sees the same keys either way
    short = [[5, 6, 7, 8, 9]]
    assert [o.outputs[0].token_ids[0] for o in a.generate(short, sp)] == \
           [o.outputs[0].token_ids[0] for o in b.generate(short, sp)]


def test_family_switches_are_read_from_the_config():
    g2, gr, ol, gl, p3 = (config_of(n) for n in ("gemma2", "granite", "olmo2", "glm4", "phi3"))
    assert g2.sandwich_norm and g2.gemma_norm and g2.attn_logit_softcap == 50.0 and g2.final_logit_softcap == 30.0
    assert g2.sliding_window == 32 and g2.hidden_act == "gelu_tanh"
    assert gr.residual_multiplier == 0.22 and gr.logits_scaling == 8.0 and gr.embed_scale == 12.0
    assert ol.post_norm and ol.qk_norm
    assert gl.sandwich_norm and not gl.rope.neox and gl.rope.rotary_dim == 32 and gl.attention_bias
    assert p3.rope.scaling_type == "longrope" and len(p3.rope.long_factor) == 32


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(FAMILIES))
def test_family_gpu_logits_and_tokens_match_the_oracle(name):
    """Prefill logits of the kernels against the fp32 oracle (relative error over the matrix and
    a per-row bound, so one wrong row cannot hide), then greedy agreement."""
    from vllm_cpp_b200 import ops
    cfg = config_of(name)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    logits = {}
    toks = {}
    for dev in ("cuda", "cpu"):
        llm = build(cfg, dev, enable_cuda_graphs=False)
        for p in prompts_of(cfg):
            llm.add_request(p, sp)
        llm.step()                                            # one step: all three prompts prefill
        logits[dev] = llm.runner._logits[:3].float().cpu().clone()
        out = {}
        while llm.has_unfinished_requests():
            for st in llm.step():
                out[st.request_id] = st.outputs[0].token_ids
        toks[dev] = [out[k] for k in sorted(out)]
    g, c = logits["cuda"], logits["cpu"]
    rel = ((g - c).norm() / c.norm()).item()
    row = ((g - c).abs().amax(dim=1) / c.abs().amax(dim=1)).max().item()
    assert rel < 3e-2, f"{name}: relative error {rel}"
    assert row < 8e-2, f"{name}: worst row error {row}"
    assert [x[0] for x in toks["cuda"]] == [x[0] for x in toks["cpu"]]
    hit = sum(sum(1 for a, b in zip(x, y) if a == b) for x, y in zip(toks["cuda"], toks["cpu"]))
    assert hit / sum(len(x) for x in toks["cpu"]) > 0.7
    assert ops.read_status() == 0
