"""MoE kernels (router top-k, expert sort, tcgen05 grouped GEMM, combine) and the Qwen3-MoE
model end to end, against the fp32 PyTorch restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from vllm_cpp_b200 import ops  # noqa: E402
from vllm_cpp_b200.ops import moe as M  # noqa: E402

DEV = "cuda"


def _rel(a, b):
    from _numerics import rel_err
    return rel_err(a, b, row_tol=0.15, abs_tol=0.1)


@pytest.mark.parametrize("T,E,k", [(7, 128, 8), (300, 64, 6), (33, 8, 2)])
def test_router_topk_softmax_renorm(T, E, k):
    torch.manual_seed(0)
    logits = torch.randn(T, E, device=DEV)
    logits[0, 3] = logits[0, 5] = 9.0          # tie: the lower index must win first
    ids, w = M.router_topk(logits, k, renorm=True)
    eids, ew = M.ref_router_topk(logits, k, renorm=True)
    assert torch.equal(ids, eids)
    assert torch.allclose(w, ew, atol=1e-6, rtol=1e-5)
    assert ids[0, 0].item() == 3 and ids[0, 1].item() == 5


def test_router_grouped_sigmoid_bias():
    torch.manual_seed(1)
    T, E, k = 40, 64, 6
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1
    ids, w = M.router_topk(logits, k, renorm=True, scoring="sigmoid", e_bias=bias, n_group=8,
                           topk_group=4, routed_scale=2.5)
    eids, ew = M.ref_router_topk(logits, k, renorm=True, scoring="sigmoid", e_bias=bias,
                                 n_group=8, topk_group=4, routed_scale=2.5)
    assert torch.equal(ids.sort(-1).values, eids.sort(-1).values)
    assert torch.allclose(w.sum(-1), ew.sum(-1), atol=1e-5)


def local_pairs(ids, e0, el):
    return int(((ids >= e0) & (ids < e0 + el)).sum().item())


@pytest.mark.parametrize("T,E,k,H,I,e0,el", [(5, 8, 2, 256, 128, 0, 8), (300, 16, 4, 512, 256, 0, 16),
                                             (700, 8, 2, 256, 128, 4, 4), (64, 128, 8, 2048, 768, 0, 128)])
def test_moe_block_matches_reference(T, E, k, H, I, e0, el):
    """sort + gather + grouped GEMM (gate_up) + silu*mul + grouped GEMM (down) + combine;
    with e0/el a subset of experts is local (expert parallel partial sums)."""
    torch.manual_seed(2)
    x = (torch.randn(T, H, device=DEV) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(el, 2 * I, H, device=DEV) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(el, H, I, device=DEV) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, device=DEV)
    ids, w = M.router_topk(logits, k)
    ws = M.MoeWorkspace(torch.device(DEV), T, k, el, H, I)
    M.moe_sort(ids, e0, e0 + el, ws)
    P = T * k
    M.moe_gather(x, ws, el, P)
    M.grouped_gemm(ws.xs, wgu, ws.gu, ws, P)
    ops.act_and_mul(ws.gu[:P], 0, out=ws.act[:P])
    # the gated grouped GEMM (both halves in TMEM, activation in the epilogue) gives the same bits
    unfused = ws.act[:local_pairs(ids, e0, el)].clone()
    ws.act.zero_()
    M.grouped_gemm_gated(ws.xs, wgu, ws.act, ws, P, kind=0)
    assert torch.equal(ws.act[:unfused.shape[0]], unfused)
    M.grouped_gemm(ws.act, wd, ws.y, ws, P)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    M.combine(ws.y, ws, w, out)
    exp = M.ref_moe_block(x, ids, w, wgu, wd, e0=e0)
    assert ops.read_status() == 0
    assert _rel(out, exp) < 2e-2
    # bookkeeping: every local pair has a slot, counts add up
    local = ((ids >= e0) & (ids < e0 + el)).sum().item()
    assert ws.meta[2 * el].item() == local
    assert (ws.pair_pos.view(T, k)[(ids >= e0) & (ids < e0 + el)] >= 0).all()


def test_moe_engine_gpu_vs_cpu():
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-moe")
    cfg.head_dim = 128
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (90, 7, 200)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)

    def run(dev):
        llm = LLM(EngineArgs(model_config=cfg, device=dev, block_size=16, num_blocks=128,
                             max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256))
        return [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]

    gpu, cpu = run("cuda"), run("cpu")
    assert ops.read_status() == 0
    assert [a[0] for a in gpu] == [a[0] for a in cpu]
    hit = sum(sum(1 for p, q in zip(a, b) if p == q) for a, b in zip(gpu, cpu))
    assert hit / sum(len(a) for a in gpu) > 0.7
