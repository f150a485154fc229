"""Native CPU backend (csrc/cpu) against the PyTorch oracle: op by op, thread-count invariance,
and a whole model through the engine."""
import pytest
import torch

from vllm_cpp_b200.ops import cpu_native as CN
from vllm_cpp_b200.ops import reference as ref


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)).item()


@pytest.mark.parametrize("M,N,K", [(1, 64, 128), (5, 100, 72), (17, 33, 260), (64, 512, 1024)])
def test_matmul(M, N, K):
    a, w = _rand(M, K), _rand(N, K, scale=0.05, seed=1)
    bias, res = _rand(N, seed=2), _rand(M, N, seed=3)
    out = CN.gemm(a, w, bias, res)
    assert _rel(out, ref.gemm(a, w, bias, res)) < 1e-2
    out32 = CN.gemm(a, w, out_dtype=torch.float32)
    assert _rel(out32, ref.gemm(a, w, out_dtype=torch.float32)) < 1e-4


def test_results_do_not_depend_on_thread_count():
    a, w = _rand(9, 520), _rand(301, 520, scale=0.05, seed=1)
    outs = []
    for n in (1, 3, 8):
        CN.set_num_threads(n)
        assert CN.num_threads() == n
        outs.append(CN.gemm(a, w, out_dtype=torch.float32))
    CN.set_num_threads(0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_norm_act_embedding():
    x, w, r = _rand(7, 256), _rand(256, seed=1), _rand(7, 256, seed=2)
    r2 = r.clone()
    out = CN.rmsnorm(x, w, 1e-6, residual=r2, gemma=True)
    exp, newr = ref.rmsnorm(x, w, 1e-6, r, True)
    assert torch.equal(r2, newr)
    assert _rel(out, exp) < 1e-2
    gu = _rand(5, 2 * 96, seed=3)
    for kind in (0, 1, 2):
        assert _rel(CN.act_and_mul(gu, kind), ref.act_and_mul(gu, kind)) < 1e-2
    table = _rand(50, 32, seed=4)
    ids = torch.tensor([3, 49, 60, 10])
    e = CN.embedding(ids, table[10:], vocab_start=10)
    assert torch.equal(e[0], torch.zeros(32, dtype=torch.bfloat16)) and torch.equal(e[1], table[49])
    assert torch.equal(e[2], torch.zeros(32, dtype=torch.bfloat16)) and torch.equal(e[3], table[10])


@pytest.mark.parametrize("neox,rot,norm", [(True, 64, True), (False, 32, False)])
def test_rope_cache_attention(neox, rot, norm):
    torch.manual_seed(0)
    Hq, Hkv, D, bs = 4, 2, 64, 16
    lens = [37, 5, 20]
    qlens = [37, 1, 4]
    T = sum(qlens)
    nb = [(l + bs - 1) // bs for l in lens]
    cache = torch.zeros(sum(nb) + 1, 2, bs, Hkv, D, dtype=torch.bfloat16)
    cache_ref = cache.clone()
    bt = torch.zeros(3, max(nb), dtype=torch.int32)
    nxt = 1
    for r in range(3):
        for j in range(nb[r]):
            bt[r, j] = nxt
            nxt += 1
    # context already in the cache for requests 1 and 2
    ctx = _rand(*cache.shape, seed=5)
    cache.copy_(ctx)
    cache_ref.copy_(ctx)
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=6)
    pos, slots, qs = [], [], [0]
    for r in range(3):
        for i in range(qlens[r]):
            p = lens[r] - qlens[r] + i
            pos.append(p)
            slots.append(int(bt[r, p // bs]) * bs + p % bs)
        qs.append(qs[-1] + qlens[r])
    pos, slots = torch.tensor(pos), torch.tensor(slots)
    table = ref.rope_table(ref.rope_inv_freq(rot, 1e4), 64)
    qn = _rand(D, seed=7) if norm else None
    kn = _rand(D, seed=8) if norm else None
    q_ref, k_ref, v_ref = ref.rope_kv(qkv, pos, table, Hq, Hkv, D, rot, neox, qn, kn, 1e-6, False)
    ref.write_kv_cache(cache_ref, k_ref, v_ref, slots, bs)
    mine = qkv.clone()
    CN.rope_kv(mine, pos, table, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, rot_dim=rot, neox=neox,
              q_norm=qn, k_norm=kn, eps=1e-6, gemma=False, slot_mapping=slots, kv_cache=cache, block_size=bs)
    assert _rel(mine[:, : Hq * D], q_ref.reshape(T, -1)) < 1e-2
    assert _rel(cache, cache_ref) < 1e-2
    sl, qst = torch.tensor(lens, dtype=torch.int32), torch.tensor(qs, dtype=torch.int32)
    q = q_ref.reshape(T, -1).contiguous()
    for window, cap in ((0, 0.0), (9, 20.0)):
        out = CN.paged_attention(q, cache_ref, bt, sl, qst, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                block_size=bs, scale=D ** -0.5, softcap=cap, window=window)
        exp = ref.paged_attention(q, cache_ref, bt, sl, qst, Hq, Hkv, D, bs, D ** -0.5, cap, window)
        assert _rel(out, exp) < 1e-2


def test_engine_on_native_backend_matches_oracle():
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-qwen3")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 7, 19)]
    outs = {}
    for be in ("torch", "native"):
        llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, max_model_len=128,
                             max_num_seqs=4, max_num_batched_tokens=32, num_blocks=64, cpu_backend=be))
        assert (llm.model.be.name == "cpu-native") == (be == "native")
        outs[be] = [o.outputs[0].token_ids
                    for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))]
    same = sum(a == b for x, y in zip(outs["torch"], outs["native"]) for a, b in zip(x, y))
    assert [x[0] for x in outs["torch"]] == [x[0] for x in outs["native"]]
    assert same >= 0.75 * 24


def test_gemm_tiers_agree():
    """The GEMM tiers this machine offers (scalar, AVX2, AVX-512 BF16, AMX tiles; the cap is read
    once per process, so each runs in a child) give the same product up to fp32 summation order."""
    import os
    import subprocess
    import sys
    code = (
        "import torch, sys\n"
        "from vllm_cpp_b200.ops import cpu_native as CN\n"
        "g = torch.Generator().manual_seed(3)\n"
        "a = torch.randn(37, 1056, generator=g).to(torch.bfloat16)\n"
        "w = (torch.randn(203, 1056, generator=g) * 0.05).to(torch.bfloat16)\n"
        "b = torch.randn(203, generator=g).to(torch.bfloat16)\n"
        "out = CN.gemm(a, w, b, out_dtype=torch.float32)\n"
        "torch.save((CN.lib().b200cpu_simd_tier(), out), sys.argv[1])\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = {}
    for cap in ("scalar", "avx2", "avx512", ""):
        path = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"b200_tier_{os.getpid()}_{cap or 'best'}.pt")
        env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        if cap:
            env["B200CPU_SIMD"] = cap
        else:
            env.pop("B200CPU_SIMD", None)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=300)
        tier, out = torch.load(path)
        os.remove(path)
        outs[tier] = out
    assert 0 in outs                                   # the scalar tier always exists
    base = outs[0]
    for tier, out in outs.items():
        assert ((out - base).abs().max() / base.abs().max()).item() < 2e-6, tier
    if 2 in outs:
        assert torch.equal(outs[2], outs[0])           # AVX2 sums in the scalar tier's order
