"""Native CPU ops beyond the dense decoder (MoE, Gated DeltaNet, MLA, block-quantised GEMM) against
the PyTorch fp32 restatements the GPU kernels are also tested against."""
import numpy as np
import pytest
import torch

from vllm_cpp_b200.ops import cpu_native as N
from vllm_cpp_b200.ops import gdn as G
from vllm_cpp_b200.ops import mla as MLA
from vllm_cpp_b200.ops import moe as M


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("scoring,bias,groups", [("softmax", False, (1, 1)), ("sigmoid", True, (4, 2)),
                                                 ("softmax", False, (4, 2))])
@pytest.mark.parametrize("renorm", [True, False])
def test_router_topk(scoring, bias, groups, renorm):
    T, E, k = 37, 16, 4
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(3))
    logits[5, 2] = logits[5, 9]                      # a tie: the lower index wins
    eb = torch.randn(E, generator=torch.Generator().manual_seed(4)) * 0.1 if bias else None
    ids, w = N.moe_router_topk(logits, k, renorm, scoring, eb, groups[0], groups[1], 2.5)
    rid, rw = M.ref_router_topk(logits, k, renorm, scoring, eb, groups[0], groups[1], 2.5)
    assert torch.equal(ids, rid)
    torch.testing.assert_close(w, rw, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("e0,el", [(0, 8), (4, 4)])
def test_moe_experts_match_reference(e0, el):
    T, H, I, E, k = 19, 64, 48, 8, 2
    x = _bf(T, H, seed=1)
    wgu = _bf(E, 2 * I, H, scale=0.1, seed=2)
    wd = _bf(E, H, I, scale=0.1, seed=3)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(5))
    ids, w = M.ref_router_topk(logits, k)
    got = N.moe_experts(x, ids, w, wgu[e0:e0 + el], wd[e0:e0 + el], e0=e0)
    want = M.ref_moe_block(x, ids, w, wgu[e0:e0 + el], wd[e0:e0 + el], e0=e0)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max() + 1e-6


def test_gdn_conv1d_and_state():
    C, slots_n = 96, 5
    qsl, slots, has_init = [0, 7, 8, 8, 20], [3, 0, 1, 4], [1, 0, 1, 1]
    x = _bf(20, C, seed=1)
    w = _bf(C, 4, scale=0.5, seed=2)
    st = _bf(slots_n, C, 3, seed=3)
    want, want_st = G.ref_conv1d(x, w, st, qsl, slots, has_init)
    got_st = st.clone()
    got = N.gdn_conv1d(x, w, got_st, qsl, slots, has_init)
    assert (got.float() - want.float()).abs().max() < 2e-2
    assert torch.equal(got_st, want_st)


def test_gdn_post_conv_recurrent_and_gated_norm():
    T, Hk, Hv = 12, 2, 4
    xc = _bf(T, 2 * Hk * 128 + Hv * 128, seed=1)
    a, b = _bf(T, Hv, seed=2), _bf(T, Hv, seed=3)
    A_log, dt_bias = torch.randn(Hv) * 0.1, torch.randn(Hv) * 0.1
    q, k, g, beta = N.gdn_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias)
    rq, rk, rg, rb = G.ref_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias)
    assert (q.float() - rq.float()).abs().max() < 1e-2 and (k.float() - rk.float()).abs().max() < 1e-2
    torch.testing.assert_close(g, rg, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(beta, rb, rtol=1e-4, atol=1e-5)
    # two sequences: one continues a stored state, one starts from zero
    qsl, slots, has_init = [0, 5, 12], [2, 0], [1, 0]
    state = torch.randn(3, Hv, 128, 128, generator=torch.Generator().manual_seed(7)) * 0.05
    v = xc[:, 2 * Hk * 128:].view(T, Hv, 128)
    st = state.clone()
    out = N.gdn_recurrent(rq, rk, v, rg, rb, st, qsl, slots, has_init)
    for i in range(2):
        s0 = state[slots[i]] if has_init[i] else torch.zeros_like(state[0])
        bgn, end = qsl[i], qsl[i + 1]
        o, s1 = G.ref_recurrent(rq[bgn:end], rk[bgn:end], v[bgn:end], rg[bgn:end], rb[bgn:end], s0)
        torch.testing.assert_close(out[bgn:end], o, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(st[slots[i]], s1, rtol=2e-4, atol=2e-4)
    assert torch.equal(st[1], state[1])                       # an unused slot is untouched
    core = out.reshape(T, -1).to(torch.bfloat16)
    z, gw = _bf(T, Hv * 128, seed=9), _bf(128, seed=10)
    got = N.rmsnorm_gated(core, z, gw, heads=Hv)
    want = G.ref_rmsnorm_gated(core, z, gw, heads=Hv)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max() + 1e-6


def test_mla_attention_prefill_and_decode_rows():
    H, bs, nb = 2, 16, 12
    cache = _bf(nb, bs, 576, scale=0.3, seed=1)
    w_kvb = _bf(H * 256, 512, scale=0.05, seed=2)
    # request 0: 20 cached rows, 20 new (prefill); request 1: 37 cached rows, 1 new (decode)
    seq_lens = torch.tensor([20, 37])
    query_start = torch.tensor([0, 20, 21])
    block_table = torch.tensor([[3, 7, 0, 0], [1, 4, 9, 0]], dtype=torch.int32)
    q = _bf(21, H, 192, scale=0.5, seed=3)
    want = MLA.ref_mla_attention(q, cache, block_table, seq_lens, query_start, w_kvb, H, 0.07, bs)
    got = N.mla_attention(q, cache, block_table, seq_lens, query_start, w_kvb, H, 0.07, bs)
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("kind", [N.Q8_0, N.Q4_0])
def test_block_quant_gemm_keeps_weights_packed(kind):
    from vllm_cpp_b200.loader.gguf import dequantize
    M_, Nn, K = 5, 24, 128
    a = _bf(M_, K, seed=1)
    w = torch.randn(Nn, K, generator=torch.Generator().manual_seed(2)) * 0.1
    wq = N.quantize_blocks(w, kind)
    ggml_type = {N.Q8_0: 8, N.Q4_0: 2}[kind]
    wd = torch.from_numpy(dequantize(wq.numpy().reshape(-1), ggml_type, (Nn, K)).astype(np.float32))
    # the packed weights decode close to the source (Q8_0 fine, Q4_0 coarse)
    assert (wd - w).abs().max() < (0.005 if kind == N.Q8_0 else 0.06)
    got = N.gemm_quant(a, wq, kind, out_dtype=torch.float32)
    want = a.float() @ wd.t()
    # activations are rounded to int8 per block: ~0.4 % relative error per term
    assert (got - want).norm() / want.norm() < 1e-2


@pytest.mark.parametrize("shape", ["tiny-mla", "tiny-gdn", "tiny-gdn-moe", "tiny-moe"])
def test_engine_on_native_cpu_ops_matches_the_pytorch_oracle(shape, monkeypatch):
    """The CPU execution path of the MLA / GDN / MoE models runs on the native ops; with
    B200_CPU_ORACLE=1 the same engine runs their PyTorch restatements. Same greedy tokens."""
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    res = {}
    for oracle in ("1", "0"):
        monkeypatch.setenv("B200_CPU_ORACLE", oracle)
        cfg = synthetic_config(shape)
        llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=100, max_model_len=256,
                             max_num_seqs=4, max_num_batched_tokens=64))
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 9, 33)]
        out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
        res[oracle] = [o.outputs[0].token_ids for o in out]
    assert res["0"] == res["1"]


@pytest.mark.parametrize("fmt", ["q8_0", "q4_0"])
def test_engine_computes_on_packed_gguf_blocks(fmt):
    """cpu_weight_quant keeps the linear weights in GGUF blocks and the native backend multiplies
    the packed form; against the same weights decoded to bf16 the greedy tokens agree."""
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    from vllm_cpp_b200.models.backend import BlockQuantWeight
    cfg = synthetic_config("tiny-qwen3")
    kw = dict(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256, max_num_seqs=4,
              max_num_batched_tokens=64, cpu_backend="native")
    packed = LLM(EngineArgs(cpu_weight_quant=fmt, **kw))
    assert isinstance(packed.model.layers[0]["qkv"], BlockQuantWeight)
    # reference engine: the same blocks decoded to bf16 tensors
    dense = LLM(EngineArgs(**kw))
    for Lp, Ld in zip(packed.model.layers, dense.model.layers):
        for k, w in Lp.items():
            if isinstance(w, BlockQuantWeight):
                Ld[k] = w.dequant()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a = [o.outputs[0].token_ids for o in packed.generate(prompts, sp)]
    b = [o.outputs[0].token_ids for o in dense.generate(prompts, sp)]
    assert [x[0] for x in a] == [x[0] for x in b]
    hit = sum(sum(1 for p, q in zip(x, y) if p == q) for x, y in zip(a, b))
    assert hit >= 0.7 * sum(len(x) for x in b)


def test_requantising_decoded_q8_0_blocks_is_lossless():
    w = torch.randn(16, 128, generator=torch.Generator().manual_seed(4))
    first = N.quantize_blocks(w, N.Q8_0)
    from vllm_cpp_b200.loader.gguf import dequantize
    dec = torch.from_numpy(dequantize(first.numpy().reshape(-1), 8, (16, 128)).astype(np.float32))
    again = N.quantize_blocks(dec, N.Q8_0)
    assert torch.equal(first, again)
