"""Multi-head latent attention: absorbed tcgen05 decode kernel, batched small-M GEMM, prefill
helpers, and the DeepSeek-V2-shaped model through the engine (CPU oracle, GPU vs CPU)."""
import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams


def _rel(a, b):
    from _numerics import rel_err
    return rel_err(a, b, row_tol=0.15, abs_tol=0.1)


def _prompts(cfg, lens, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def _run(dev, cfg, prompts, budget, max_tokens=6):
    llm = LLM(EngineArgs(model_config=cfg, device=dev, block_size=16, num_blocks=128, max_model_len=512,
                         max_num_seqs=4, max_num_batched_tokens=budget))
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    return [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]


def test_mla_cpu_chunked_prefill_matches_unchunked():
    cfg = synthetic_config("tiny-mla")
    prompts = _prompts(cfg, (70, 5, 33))
    assert _run("cpu", cfg, prompts, 256) == _run("cpu", cfg, prompts, 32)


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,bs,splits,ctx", [(3, 16, 16, 1, [700, 1, 129]), (5, 4, 32, 3, [64, 1000, 5, 300, 128]),
                                                (2, 16, 128, 2, [2000, 513])])
def test_mla_decode_kernel(B, H, bs, splits, ctx):
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.ops import mla as M
    torch.manual_seed(0)
    nb = sum(-(-c // bs) for c in ctx) + 2
    cache = (torch.randn(nb, bs, 576, device="cuda") * 0.5).to(torch.bfloat16)
    mb = max(-(-c // bs) for c in ctx)
    bt = torch.zeros(B, mb, dtype=torch.int32, device="cuda")
    perm = torch.randperm(nb - 1)[: nb - 1] + 1
    k = 0
    for b, c in enumerate(ctx):
        n = -(-c // bs)
        bt[b, :n] = perm[k:k + n].to(torch.int32)
        k += n
    sl = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    qabs = (torch.randn(B, H, 576, device="cuda") * 0.3).to(torch.bfloat16)
    out = torch.empty(B, H * 512, dtype=torch.bfloat16, device="cuda")
    M.mla_decode(qabs, cache, bt, sl, out, 0.07, bs, splits=splits)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    exp = M.ref_mla_decode_absorbed(qabs, cache, bt, sl, 0.07, bs)
    assert _rel(out.view(B, H, 512), exp) < 2e-2


@pytest.mark.gpu
def test_gemm_batched_and_prefill_helpers():
    from vllm_cpp_b200.ops import mla as M
    torch.manual_seed(1)
    T, H = 300, 6
    a = (torch.randn(T, H * 192 + 64, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(H, 512, 128, device="cuda") * 0.1).to(torch.bfloat16)
    out = torch.zeros(T, H * 576, dtype=torch.bfloat16, device="cuda")
    M.gemm_batched(a, 192, w, out, 576, T, 512, 128, H)
    for h in range(H):
        exp = a[:, h * 192: h * 192 + 128].float() @ w[h].float().t()
        assert _rel(out[:, h * 576: h * 576 + 512], exp) < 1e-2
        assert (out[:, h * 576 + 512: (h + 1) * 576] == 0).all()
    M.copy_qpe(a, out, T, H)
    assert torch.equal(out.view(T, H, 576)[:, :, 512:], a[:, : H * 192].view(T, H, 192)[:, :, 128:])
    qpad = torch.empty(T, H * 256, dtype=torch.bfloat16, device="cuda")
    M.pad_q(a, qpad, T, H)
    qp = qpad.view(T, H, 256)
    assert torch.equal(qp[:, :, :192], a[:, : H * 192].view(T, H, 192)) and (qp[:, :, 192:] == 0).all()
    # gather + assemble
    bs, lens = 16, [40, 16, 7]
    nb = 12
    cache = torch.randn(nb, bs, 576, device="cuda").to(torch.bfloat16)
    bt = torch.tensor([[3, 5, 1], [7, 0, 0], [9, 0, 0]], dtype=torch.int32, device="cuda")
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    base = torch.tensor([0, 48, 64], dtype=torch.int32, device="cuda")
    dense = torch.zeros(80, 576, dtype=torch.bfloat16, device="cuda")
    M.gather_latent(cache, bt, sl, base, bs, dense, 3, 3)
    assert torch.equal(dense[:48], cache[[3, 5, 1]].reshape(48, 576))
    assert torch.equal(dense[48:64], cache[7]) and torch.equal(dense[64:80], cache[9])
    kvb = torch.randn(80, H, 256, device="cuda").to(torch.bfloat16)
    tmp = torch.empty(5, 2, bs, H, 256, dtype=torch.bfloat16, device="cuda")
    M.assemble_kv(kvb, dense, tmp, 80, H, bs)
    K = tmp[:, 0].reshape(80, H, 256)
    V = tmp[:, 1].reshape(80, H, 256)
    assert torch.equal(K[:, :, :128], kvb[:, :, :128]) and torch.equal(V[:, :, :128], kvb[:, :, 128:])
    assert torch.equal(K[:, :, 128:192], dense[:, None, 512:].expand(80, H, 64))
    assert (K[:, :, 192:] == 0).all() and (V[:, :, 128:] == 0).all()


@pytest.mark.gpu
def test_mla_model_gpu_vs_cpu():
    from vllm_cpp_b200 import ops
    cfg = synthetic_config("tiny-mla")
    prompts = _prompts(cfg, (150, 9, 70))
    cpu = _run("cpu", cfg, prompts, 256, 8)
    for budget in (256, 64):
        gpu = _run("cuda", cfg, prompts, budget, 8)
        assert ops.read_status() == 0
        assert [a[0] for a in gpu] == [a[0] for a in cpu]
        hit = sum(sum(1 for p, q in zip(a, b) if p == q) for a, b in zip(gpu, cpu))
        assert hit / sum(len(a) for a in gpu) > 0.7
