"""Numerics of every sm_100a kernel against the fp32 PyTorch restatement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from vllm_cpp_b200 import ops  # noqa: E402
from vllm_cpp_b200.ops import reference as ref  # noqa: E402

DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


from _numerics import rel_err as _rel_err  # noqa: E402


def test_library_loaded_and_status_clean():
    assert ops.num_sms() >= 100
    assert ops.read_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (512, 1024, 512), (300, 520, 328),
                                   (1024, 4096, 4096), (4096, 6144, 4096), (257, 128, 8192)])
@pytest.mark.parametrize("path", [3, 4])
def test_gemm_tiled(M, N, K, path):
    torch.manual_seed(0)
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.gemm(a, w, force_path=path)
    exp = ref.gemm(a, w)
    assert _rel_err(out, exp) < 6e-3
    assert ops.read_status() == 0


@pytest.mark.parametrize("M,N,K", [(1280, 4096, 4096), (1280, 4096, 14336), (384, 4096, 4096),
                                   (1000, 6144, 4096), (130, 512, 8192), (520, 4104, 1024),
                                   (128, 256, 64)])
@pytest.mark.parametrize("path", [0, 5, 6])
def test_gemm_stream_k(M, N, K, path):
    """Stream-K: tiles are cut along K across CTAs and fixed up through fp32 partials. Run twice:
    the second launch only works if the first one cleared every flag it consumed."""
    torch.manual_seed(2)
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    r = _rand(M, N)
    exp = ref.gemm(a, w)
    for _ in range(2):
        out = ops.gemm(a, w, force_path=path)
        assert _rel_err(out, exp) < 6e-3
    out = ops.gemm(a, w, residual=r, force_path=path, out_dtype=torch.float32)
    assert _rel_err(out, exp + r.float()) < 6e-3
    assert ops.read_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 6144, 4096), (16, 128, 64), (33, 4096, 14336),
                                   (64, 28672, 4096), (200, 1024, 1024), (256, 4096, 4096),
                                   (5, 128256, 1024), (1, 28672, 4096), (17, 32768, 512), (64, 16384, 192)])
def test_gemm_small_m_swap_splitk(M, N, K):
    torch.manual_seed(1)
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.gemm(a, w)
    exp = ref.gemm(a, w)
    assert _rel_err(out, exp) < 6e-3
    assert ops.read_status() == 0


@pytest.mark.parametrize("M,N,K", [(32, 4096, 4096), (64, 28672, 4096), (200, 1024, 1024), (1280, 4096, 4096)])
def test_gemm_const_weight_early_fetch_in_a_chain(M, N, K):
    """``const_w`` lets the GEMM fetch weight tiles before the previous kernel has finished; the
    activations still have to wait for it. A chain norm -> GEMM -> norm -> GEMM, launched back to
    back, must give the same bits as the same chain without the flag."""
    torch.manual_seed(11)
    x0 = _rand(M, K)
    g = _rand(K)
    w1 = _rand(N, K, scale=0.05)
    w2 = _rand(K, N, scale=0.02)

    def chain(flag):
        x = x0
        for _ in range(3):
            h = ops.rmsnorm(x, g, 1e-6)
            y = ops.gemm(h, w1, const_w=flag)
            x = ops.gemm(y, w2, const_w=flag)
        return x

    a, b = chain(False), chain(True)
    assert torch.equal(a, b)
    h = ops.rmsnorm(x0, g, 1e-6)
    assert _rel_err(ops.gemm(h, w1, const_w=True), ref.gemm(h, w1)) < 6e-3
    assert ops.read_status() == 0


def test_gemm_epilogues():
    torch.manual_seed(2)
    for M in (7, 700):
        a, w = _rand(M, 512), _rand(768, 512, scale=0.05)
        bias, res = _rand(768), _rand(M, 768)
        out = ops.gemm(a, w, bias=bias, residual=res)
        assert _rel_err(out, ref.gemm(a, w, bias, res)) < 6e-3
        o32 = ops.gemm(a, w, out_dtype=torch.float32)
        assert o32.dtype == torch.float32
        assert _rel_err(o32, ref.gemm(a, w, out_dtype=torch.float32)) < 2e-3
    # strided activations (a column slice of a wider buffer)
    big = _rand(300, 1024)
    a = big[:, 256:768]
    w = _rand(384, 512, scale=0.05)
    assert _rel_err(ops.gemm(a, w), ref.gemm(a, w)) < 6e-3
    assert ops.read_status() == 0


def test_gemm_deterministic():
    torch.manual_seed(3)
    a, w = _rand(48, 4096), _rand(4096, 4096, scale=0.05)
    o1 = ops.gemm(a, w).clone()
    o2 = ops.gemm(a, w)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("T,H", [(1, 1024), (37, 4096), (5, 5120), (3, 2048)])
def test_rmsnorm(T, H):
    torch.manual_seed(4)
    x, w, r = _rand(T, H), _rand(H), _rand(T, H)
    out = ops.rmsnorm(x, w, 1e-6)
    exp, _ = ref.rmsnorm(x, w, 1e-6)
    assert _rel_err(out, exp) < 5e-3
    r2 = r.clone()
    out = ops.rmsnorm(x, w, 1e-6, residual=r2, gemma=True)
    exp, newr = ref.rmsnorm(x, w, 1e-6, residual=r, gemma=True)
    assert torch.equal(r2, newr)
    assert _rel_err(out, exp) < 5e-3


def test_layernorm_and_eltwise():
    torch.manual_seed(5)
    x, w, b = _rand(9, 768), _rand(768), _rand(768)
    assert _rel_err(ops.layernorm(x, w, b, 1e-5), ref.layernorm(x, w, b, 1e-5)) < 5e-3
    a, c = _rand(16, 512), _rand(16, 512)
    assert _rel_err(ops.add(a, c), (a.float() + c.float())) < 5e-3
    assert torch.equal(ops.relu(a), torch.relu(a))
    assert _rel_err(ops.mul_scalar(a, 0.37), a.float() * 0.37) < 5e-3
    assert _rel_err(ops.softcap(a, 30.0), 30.0 * torch.tanh(a.float() / 30.0)) < 5e-3
    assert _rel_err(ops.sigmoid_mul(a, c), a.float() * torch.sigmoid(c.float())) < 5e-3
    assert torch.equal(ops.cast_bf16(ops.cast_f32(a)), a)


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_act_and_mul(kind):
    torch.manual_seed(6)
    x = _rand(33, 2 * 1408)
    assert _rel_err(ops.act_and_mul(x, kind), ref.act_and_mul(x, kind)) < 5e-3


def test_embedding_and_gather():
    torch.manual_seed(7)
    table = _rand(1000, 256)
    ids = torch.randint(0, 1000, (77,), device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids])
    # vocab shard: rows outside are zero, no error flag
    out = ops.embedding(ids, table[500:], vocab_start=500, vocab_total=1000)
    exp = torch.where((ids >= 500)[:, None], table[ids], torch.zeros_like(table[ids]))
    assert torch.equal(out, exp)
    assert ops.read_status() == 0
    bad = ids.clone()
    bad[3] = 5000
    ops.embedding(bad, table)
    assert ops.read_status() == 3  # flagged, no fault
    assert ops.read_status() == 0
    idx = torch.randint(0, 77, (13,), device=DEV, dtype=torch.int32)
    x = _rand(77, 256)
    assert torch.equal(ops.gather_rows(x, idx), x[idx.long()])


@pytest.mark.parametrize("neox,rot,qk_norm", [(True, 128, False), (True, 128, True),
                                              (False, 64, False), (True, 64, True)])
def test_rope_kv(neox, rot, qk_norm):
    torch.manual_seed(8)
    T, Hq, Hkv, D, bs, nb = 45, 8, 2, 128, 16, 12
    qkv = _rand(T, (Hq + 2 * Hkv) * D)
    pos = torch.randint(0, 500, (T,), device=DEV)
    inv = ref.rope_inv_freq(rot, 1e6).to(DEV)
    table = ops.rope_table(inv, 512)
    assert torch.allclose(table, ref.rope_table(inv, 512), atol=2e-6)
    qn = _rand(D) if qk_norm else None
    kn = _rand(D) if qk_norm else None
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int64)
    slots[5] = -1
    cache = torch.zeros(nb, 2, bs, Hkv, D, device=DEV, dtype=torch.bfloat16)
    eq, ek, ev = ref.rope_kv(qkv, pos, table, Hq, Hkv, D, rot, neox, qn, kn)
    work = qkv.clone()
    ops.rope_kv(work, pos, table, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, rot_dim=rot,
                neox=neox, q_norm=qn, k_norm=kn, slot_mapping=slots, kv_cache=cache, block_size=bs)
    got_q = work[:, : Hq * D].reshape(T, Hq, D)
    assert _rel_err(got_q, eq) < 8e-3
    exp_cache = torch.zeros_like(cache)
    ref.write_kv_cache(exp_cache, ek, ev, slots, bs)
    assert _rel_err(cache[:, 0], exp_cache[:, 0]) < 8e-3
    assert torch.equal(cache[:, 1], exp_cache[:, 1])


def _make_paged(seq_lens, Hkv, D, bs, extra_blocks=3):
    nb_per = [(s + bs - 1) // bs for s in seq_lens]
    total = sum(nb_per) + extra_blocks
    cache = _rand(total, 2, bs, Hkv, D)
    perm = torch.randperm(total, device=DEV).to(torch.int32)
    maxb = max(nb_per)
    bt = torch.zeros(len(seq_lens), maxb, dtype=torch.int32, device=DEV)
    o = 0
    for r, n in enumerate(nb_per):
        bt[r, :n] = perm[o:o + n]
        o += n
    return cache, bt


@pytest.mark.parametrize("D,Hq,Hkv,bs", [(128, 8, 2, 16), (128, 4, 4, 32), (64, 4, 1, 16),
                                         (128, 4, 1, 128), (256, 6, 1, 16), (256, 2, 2, 64)])
def test_attn_prefill(D, Hq, Hkv, bs):
    torch.manual_seed(9)
    q_lens = [200, 17, 128, 333]
    ctx = [0, 40, 256, 77]  # cached prefix per request (chunked prefill / prefix hit)
    seq_lens = [a + b for a, b in zip(q_lens, ctx)]
    cache, bt = _make_paged(seq_lens, Hkv, D, bs)
    T = sum(q_lens)
    q = _rand(T, Hq * D)
    qs = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    treq, tq0 = ref.build_prefill_tiles(q_lens)
    treq = torch.tensor(treq, dtype=torch.int32, device=DEV)
    tq0 = torch.tensor(tq0, dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    lse = torch.empty(T, Hq, dtype=torch.float32, device=DEV)
    out = ops.attn_prefill(q, cache, block_table=bt, seq_lens=sl, q_start=qs, tile_req=treq,
                           tile_q0=tq0, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                           block_size=bs, scale=scale, lse=lse)
    exp, exp_lse = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, scale, return_lse=True)
    assert ops.read_status() == 0
    assert _rel_err(out, exp) < 1.5e-2
    assert torch.allclose(lse, exp_lse, atol=2e-2, rtol=1e-3)


def test_attn_prefill_window_softcap():
    torch.manual_seed(10)
    D, Hq, Hkv, bs = 128, 4, 2, 16
    q_lens, ctx = [300, 64], [100, 500]
    seq_lens = [a + b for a, b in zip(q_lens, ctx)]
    cache, bt = _make_paged(seq_lens, Hkv, D, bs)
    T = sum(q_lens)
    q = _rand(T, Hq * D)
    qs = torch.tensor([0, 300, 364], dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    treq, tq0 = ref.build_prefill_tiles(q_lens)
    kw = dict(block_table=bt, seq_lens=sl, q_start=qs,
              tile_req=torch.tensor(treq, dtype=torch.int32, device=DEV),
              tile_q0=torch.tensor(tq0, dtype=torch.int32, device=DEV), num_q_heads=Hq,
              num_kv_heads=Hkv, head_dim=D, block_size=bs, scale=D ** -0.5)
    out = ops.attn_prefill(q, cache, window=150, softcap=20.0, **kw)
    exp = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5, softcap=20.0,
                              window=150)
    assert _rel_err(out, exp) < 1.5e-2
    assert ops.read_status() == 0


@pytest.mark.parametrize("chunk", [64, 200])
def test_attn_chunked_local(chunk):
    """Chunked-local attention (window < 0): a query sees the keys of its own chunk only, in the
    prefill kernel, the tcgen05 decode kernel and the CUDA-core decode kernel."""
    torch.manual_seed(12)
    D, Hq, Hkv, bs = 128, 8, 2, 16
    q_lens, ctx = [300, 64, 5], [100, 500, 0]
    seq_lens = [a + b for a, b in zip(q_lens, ctx)]
    cache, bt = _make_paged(seq_lens, Hkv, D, bs)
    T = sum(q_lens)
    q = _rand(T, Hq * D)
    qs = torch.tensor([0, 300, 364, 369], dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    treq, tq0 = ref.build_prefill_tiles(q_lens)
    out = ops.attn_prefill(q, cache, block_table=bt, seq_lens=sl, q_start=qs,
                           tile_req=torch.tensor(treq, dtype=torch.int32, device=DEV),
                           tile_q0=torch.tensor(tq0, dtype=torch.int32, device=DEV), num_q_heads=Hq,
                           num_kv_heads=Hkv, head_dim=D, block_size=bs, scale=D ** -0.5, window=-chunk)
    exp = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5, window=-chunk)
    assert _rel_err(out, exp) < 1.5e-2
    # decode: one query per sequence at its last position
    B = len(seq_lens)
    qd = _rand(B, Hq * D)
    qsd = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    expd = ref.paged_attention(qd, cache, bt, sl, qsd, Hq, Hkv, D, bs, D ** -0.5, window=-chunk)
    for cuda_core in (False, True):
        got = ops.attn_decode(qd, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq, num_kv_heads=Hkv,
                              head_dim=D, block_size=bs, scale=D ** -0.5, window=-chunk, splits=2,
                              force_cuda_core=cuda_core)
        assert _rel_err(got, expd) < 1e-2
    assert ops.read_status() == 0


@pytest.mark.parametrize("D,Hq,Hkv,bs,splits", [(128, 32, 8, 16, 0), (128, 4, 1, 16, 1),
                                                (128, 32, 4, 32, 5), (64, 8, 8, 16, 3),
                                                (256, 24, 4, 16, 2), (128, 16, 8, 16, 4)])
def test_attn_decode(D, Hq, Hkv, bs, splits):
    torch.manual_seed(11)
    seq_lens = [1, 15, 16, 17, 700, 1234, 129]
    cache, bt = _make_paged(seq_lens, Hkv, D, bs)
    B = len(seq_lens)
    q = _rand(B, Hq * D)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    qs = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    out = ops.attn_decode(q, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq, num_kv_heads=Hkv,
                          head_dim=D, block_size=bs, scale=D ** -0.5, splits=splits)
    exp = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5)
    assert _rel_err(out, exp) < 1e-2
    out2 = ops.attn_decode(q, cache, block_table=bt, seq_lens=sl, num_q_heads=Hq, num_kv_heads=Hkv,
                           head_dim=D, block_size=bs, scale=D ** -0.5, splits=splits, window=100,
                           softcap=30.0)
    exp2 = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5, window=100,
                               softcap=30.0)
    assert _rel_err(out2, exp2) < 1e-2


@pytest.mark.parametrize("Hq,Hkv,bs,splits", [(32, 8, 32, 1), (16, 4, 16, 3)])
def test_attn_decode_tcgen05_persistent(Hq, Hkv, bs, splits):
    """More (sequence, kv head, split) items than resident CTAs: every CTA walks several items
    (some of them empty) and the rings run across the item boundaries."""
    torch.manual_seed(22)
    D = 128
    B = 100 if Hkv == 8 else 60
    gen = torch.Generator().manual_seed(5)
    seq_lens = torch.randint(0, 600, (B,), generator=gen).tolist()
    seq_lens[3] = 0
    seq_lens[7] = 128
    seq_lens[11] = 1
    cache, bt = _make_paged([max(s, 1) for s in seq_lens], Hkv, D, bs)
    q = _rand(B, Hq * D)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    qs = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kw = dict(block_table=bt, seq_lens=sl, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
              block_size=bs, scale=D ** -0.5, splits=splits)
    exp = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5)
    for _ in range(2):
        out = ops.attn_decode(q, cache, **kw)
        assert ops.read_status() == 0
        assert _rel_err(out, exp) < 1e-2


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("Hq,Hkv,bs,splits", [(32, 8, 16, 0), (4, 1, 32, 1), (32, 4, 16, 3),
                                              (16, 16, 64, 2), (8, 1, 128, 4), (16, 1, 16, 2),
                                              (24, 4, 32, 2)])
def test_attn_decode_tcgen05(Hq, Hkv, bs, splits, D):
    """tcgen05 swapped-operand decode kernel (head_dim 128 and 256) vs the fp32 oracle and vs the
    CUDA-core kernel."""
    torch.manual_seed(21)
    seq_lens = [1, 127, 128, 129, 700, 1234, 0, 31]
    lens_for_cache = [max(s, 1) for s in seq_lens]
    cache, bt = _make_paged(lens_for_cache, Hkv, D, bs)
    B = len(seq_lens)
    q = _rand(B, Hq * D)
    # strided q like the model passes it (a column slice of the merged qkv buffer)
    wide = _rand(B, (Hq + 2 * Hkv) * D)
    wide[:, : Hq * D] = q
    qv = wide[:, : Hq * D]
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    qs = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kw = dict(block_table=bt, seq_lens=sl, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
              block_size=bs, scale=D ** -0.5, splits=splits)
    out = ops.attn_decode(qv, cache, **kw)
    assert ops.read_status() == 0
    exp = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5)
    assert _rel_err(out, exp) < 1e-2
    old = ops.attn_decode(qv, cache, force_cuda_core=True, **kw)
    assert _rel_err(out, old) < 1e-2
    out2 = ops.attn_decode(qv, cache, window=100, softcap=30.0, **kw)
    exp2 = ref.paged_attention(q, cache, bt, sl, qs, Hq, Hkv, D, bs, D ** -0.5, window=100,
                               softcap=30.0)
    assert _rel_err(out2, exp2) < 1e-2
    assert ops.read_status() == 0


def test_merge_attn_states():
    torch.manual_seed(12)
    T, H, D = 9, 4, 128
    a, b = _rand(T, H, D), _rand(T, H, D)
    la = torch.randn(T, H, device=DEV)
    lb = torch.randn(T, H, device=DEV)
    lb[0, 0] = -math.inf
    lo = torch.empty_like(la)
    out = ops.merge_attn_states(a, la, b, lb, lse_out=lo)
    mx = torch.maximum(la, lb)
    wa, wb = torch.exp(la - mx), torch.exp(lb - mx)
    exp = (a.float() * wa[..., None] + b.float() * wb[..., None]) / (wa + wb)[..., None]
    assert _rel_err(out, exp) < 5e-3
    assert torch.allclose(lo, mx + torch.log(wa + wb), atol=1e-4)


# ------------------------------------------------------------------------------- sampling
def test_argmax_tie_break_lowest_index():
    torch.manual_seed(13)
    logits = torch.randn(37, 151936, device=DEV)
    logits[3, 100] = 50.0
    logits[3, 90000] = 50.0
    got = ops.argmax(logits)
    assert torch.equal(got, logits.argmax(-1)) or got[3].item() == 100
    assert got[3].item() == 100
    mask = torch.ones(37, dtype=torch.bool)
    mask[3] = False
    assert torch.equal(got[mask], logits.argmax(-1)[mask])


def test_top_k_top_p_min_p_temperature():
    torch.manual_seed(14)
    n, V = 6, 32000
    logits = torch.randn(n, V, device=DEV) * 3
    k = torch.tensor([0, 1, 50, 0, 20, V], dtype=torch.int32, device=DEV)
    p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 0.3], dtype=torch.float32, device=DEV)
    got = ops.apply_top_k_top_p(logits.clone(), k, p)
    exp = ref.top_k_top_p(logits, k.tolist(), p.tolist())
    assert torch.equal(torch.isinf(got), torch.isinf(exp))
    temp = torch.tensor([0.0, 0.5, 1.0, 2.0, 0.7, 1e-6], device=DEV)
    t = ops.apply_temperature(logits.clone(), temp)
    e = logits.clone()
    for r in range(n):
        if temp[r] >= 1e-5:
            e[r] /= temp[r]
    assert torch.allclose(t, e, rtol=1e-6)
    mp = torch.tensor([0.0, 0.1, 0.5, 0.01, 0.0, 0.2], device=DEV)
    g = ops.apply_min_p(logits.clone(), mp)
    pr = torch.softmax(logits, -1)
    keep = pr >= mp[:, None] * pr.max(-1, keepdim=True).values
    # boundary elements may differ by rounding: compare away from the threshold
    far = (pr / pr.max(-1, keepdim=True).values - mp[:, None]).abs() > 1e-6
    assert torch.equal((~torch.isinf(g))[far], keep[far])


def test_softmax_random_sample_rank():
    torch.manual_seed(15)
    n, V = 4, 5000
    logits = torch.randn(n, V, device=DEV)
    pr = ops.softmax(logits)
    assert torch.allclose(pr, torch.softmax(logits, -1), atol=1e-7, rtol=1e-4)
    lp = ops.softmax(logits, log=True)
    assert torch.allclose(lp, torch.log_softmax(logits, -1), atol=1e-4)
    seeds = torch.tensor([1, 2, 3, 1], dtype=torch.int64, device=DEV).view(torch.int64)
    steps = torch.tensor([0, 0, 5, 0], dtype=torch.int64, device=DEV)
    pr[3] = pr[0]
    s1 = ops.random_sample(pr, seeds, steps)
    s2 = ops.random_sample(pr, seeds, steps)
    assert torch.equal(s1, s2)
    assert s1[0] == s1[3]
    assert ref.race_sample(pr[0].cpu(), 1, 0) == s1[0].item()
    assert ref.race_sample(pr[2].cpu(), 3, 5) == s1[2].item()
    # distribution sanity: many steps on a peaked 4-token row
    probs = torch.zeros(2000, 8, device=DEV)
    probs[:, :4] = torch.tensor([0.5, 0.25, 0.125, 0.125], device=DEV)
    sd = torch.full((2000,), 42, dtype=torch.int64, device=DEV)
    st = torch.arange(2000, dtype=torch.int64, device=DEV)
    draws = ops.random_sample(probs, sd, st)
    freq = torch.bincount(draws, minlength=8).float() / 2000
    assert abs(freq[0].item() - 0.5) < 0.05 and abs(freq[1].item() - 0.25) < 0.05
    toks = torch.tensor([5, 6, 7, 8], device=DEV)
    tl, rk = ops.token_rank(lp, toks)
    assert torch.allclose(tl, lp[torch.arange(n), toks])
    exp_rank = (lp > lp[torch.arange(n), toks][:, None]).sum(-1) + 1
    assert torch.equal(rk.long(), exp_rank)


def test_penalties_bias_mask_bitmask():
    torch.manual_seed(16)
    n, V = 3, 1000
    logits = torch.randn(n, V, device=DEV)
    rows = torch.tensor([0, 0, 2], dtype=torch.int32, device=DEV)
    toks = torch.tensor([5, 9, 7], dtype=torch.int32, device=DEV)
    cnt = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    rep = torch.tensor([1.5, 1.0, 2.0], device=DEV)
    freq = torch.tensor([0.1, 0.0, 0.2], device=DEV)
    pres = torch.tensor([0.3, 0.0, 0.4], device=DEV)
    got = ops.apply_penalties(logits.clone(), rows, toks, cnt, rep, freq, pres)
    exp = logits.clone()
    for r, t, c in zip(rows.tolist(), toks.tolist(), cnt.tolist()):
        v = exp[r, t]
        v = v / rep[r] if v > 0 else v * rep[r]
        v = v - freq[r] * c - (pres[r] if c > 0 else 0.0)
        exp[r, t] = v
    assert torch.allclose(got, exp, atol=1e-6)
    vals = torch.tensor([1.0, -2.0, 3.0], device=DEV)
    got = ops.apply_logit_bias(logits.clone(), rows, toks, vals)
    exp = logits.clone()
    exp[rows.long(), toks.long()] += vals
    assert torch.allclose(got, exp)
    got = ops.apply_token_mask(logits.clone(), rows, toks)
    assert torch.isinf(got[0, 5]) and torch.isinf(got[2, 7]) and not torch.isinf(got[1]).any()
    words = (V + 31) // 32
    mask = torch.randint(-2**31, 2**31 - 1, (2, words), dtype=torch.int32, device=DEV)
    row_ids = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    got = ops.apply_bitmask(logits.clone(), mask, row_ids)
    bits = ((mask[:, :, None] >> torch.arange(32, device=DEV)) & 1).reshape(2, -1)[:, :V].bool()
    assert torch.equal(~torch.isinf(got[2]), bits[0])
    assert torch.equal(~torch.isinf(got[0]), bits[1])
    assert not torch.isinf(got[1]).any()


def test_greedy_rejection():
    draft = torch.tensor([5, 6, 7, 1, 2], device=DEV)
    cu = torch.tensor([0, 3, 5], dtype=torch.int32, device=DEV)
    # request 0: 3 drafts + bonus -> rows 0..3 ; request 1: 2 drafts + bonus -> rows 4..6
    target = torch.tensor([5, 6, 9, 11, 1, 2, 13], device=DEV)
    out = ops.greedy_reject(target, draft, cu, 3)
    assert out.tolist() == [[5, 6, 9, -1], [1, 2, 13, -1]]


@pytest.mark.parametrize("M,I,K,kind", [(1280, 1024, 512, 0), (300, 384, 256, 1), (64, 256, 128, 0), (200, 14336, 4096, 0),
                                        (700, 14336, 4096, 0), (2048, 128, 64, 2)])
def test_gemm_gated_activation(M, I, K, kind):
    """act(gate) * up in the GEMM epilogue (interleaved gate / up rows). With the same tiling and
    no stream-K split it equals the bf16 GEMM followed by the activation kernel bit for bit;
    otherwise (fp32 partial sums added in another order) within bf16 rounding."""
    torch.manual_seed(3)
    a = _rand(M, K)
    wg, wu = _rand(I, K, scale=0.05), _rand(I, K, scale=0.05)
    w_il = ops.interleave_gate_up(wg, wu)
    merged_w = torch.cat([wg, wu], 0)
    exp = ref.act_and_mul(ref.gemm(a, merged_w), kind)
    out = ops.gemm_gated(a, w_il, kind)
    assert ops.read_status() == 0
    assert _rel_err(out, exp) < 2e-2
    if M > 128:
        two_step = ops.act_and_mul(ops.gemm(a, merged_w, force_path=7), kind)
        assert torch.equal(ops.gemm_gated(a, w_il, kind, force_path=7), two_step)
        assert _rel_err(ops.gemm_gated(a, w_il, kind, force_path=9), exp) < 2e-2
    else:
        assert torch.equal(out, ops.act_and_mul(ops.gemm(a, merged_w), kind))
