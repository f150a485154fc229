"""fp8 tcgen05 GEMM, NVFP4 weight expansion + fused W4A16 GEMM, quantisation producers."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from vllm_cpp_b200 import ops  # noqa: E402
from vllm_cpp_b200.ops import quant as Q  # noqa: E402

DEV = "cuda"


def _rel(a, b):
    from _numerics import rel_err
    return rel_err(a, b, row_tol=0.15, abs_tol=0.1)


@pytest.mark.parametrize("M,N,K,per_channel", [(128, 256, 256, False), (300, 520, 384, True), (7, 4096, 4096, False),
                                               (1000, 1024, 2048, True), (1280, 4096, 4096, False),
                                               (520, 4104, 1040, True)])
def test_gemm_fp8(M, N, K, per_channel):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.1
    sa = (a.abs().max() / 448).reshape(1)
    sw = (w.abs().amax(1) / 448) if per_channel else (w.abs().max() / 448).reshape(1)
    a8 = (a / sa).to(torch.float8_e4m3fn)
    w8 = (w / (sw[:, None] if per_channel else sw)).to(torch.float8_e4m3fn)
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    out = Q.gemm_fp8(a8, w8, sa.float(), sw.float().contiguous(), bias=bias)
    exp = (a8.float() @ w8.float().t()) * sa * (sw[None, :] if per_channel else sw) + bias.float()
    assert ops.read_status() == 0
    assert _rel(out, exp) < 1e-2


@pytest.mark.parametrize("M,N,K", [(64, 4096, 14336), (200, 1024, 2048), (256, 6144, 4096), (1280, 1024, 1024),
                                   (9, 520, 1040)])
def test_gemm_fp8_per_token_scales_and_split_k(M, N, K):
    """One activation scale per row and one weight scale per channel; the small-batch shapes take
    the split-K plan (partial sums through the per-device scratch, scales applied by the reduce)."""
    torch.manual_seed(5)
    a = torch.randn(M, K, device=DEV) * (torch.rand(M, 1, device=DEV) * 4 + 0.1)
    w = torch.randn(N, K, device=DEV) * 0.1
    sa = (a.abs().amax(1) / 448).float().contiguous()
    sw = (w.abs().amax(1) / 448).float().contiguous()
    a8 = (a / sa[:, None]).to(torch.float8_e4m3fn)
    w8 = (w / sw[:, None]).to(torch.float8_e4m3fn)
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    exp = (a8.float() @ w8.float().t()) * sa[:, None] * sw[None, :] + bias.float()
    for _ in range(2):                               # the scratch is reused by the next call
        out = Q.gemm_fp8(a8, w8, sa, sw, bias=bias)
        assert ops.read_status() == 0
        assert _rel(out, exp) < 1e-2
    out2 = Q.gemm_fp8(a8, w8, sa, sw)
    assert _rel(out2, exp - bias.float()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (64, 4096, 4096), (256, 1024, 14336), (33, 520, 512),
                                   (700, 1024, 1024)])
def test_nvfp4_weights(M, N, K):
    torch.manual_seed(1)
    w = torch.randn(N, K, device=DEV) * 0.05
    packed, sf, g = Q.ref_quant_nvfp4_weights(w)
    wd = Q.ref_dequant_nvfp4(packed, sf, g)
    # the format itself: 4-bit values (a Frobenius bound; single elements may be off by a sixth of
    # their block's maximum)
    assert ((wd - w).norm() / w.norm()).item() < 0.15
    got = Q.nvfp4_dequant(packed, sf, g)
    assert torch.equal(got.float(), wd.to(torch.bfloat16).float())
    a = (torch.randn(M, K, device=DEV) * 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    out = Q.gemm_w4a16(a, packed, sf, g, bias=bias)
    exp = a.float() @ wd.to(torch.bfloat16).float().t() + bias.float()
    assert ops.read_status() == 0
    assert _rel(out, exp) < 1e-2


def test_quant_fp8_static_and_rmsnorm():
    torch.manual_seed(2)
    x = (torch.randn(37, 512, device=DEV) * 3).to(torch.bfloat16)
    scale = torch.tensor([0.05], device=DEV)
    got = Q.quant_fp8(x, scale)
    exp = (x.float() / 0.05).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert (got.float() - exp.float()).abs().max() <= exp.float().abs().max() * 0.07
    assert (got.view(torch.uint8) == exp.view(torch.uint8)).float().mean() > 0.98
    w = (torch.rand(512, device=DEV) + 0.5).to(torch.bfloat16)
    got = Q.quant_fp8(x, scale, norm_weight=w, eps=1e-6)
    xf = x.float()
    n = (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * w.float()).to(torch.bfloat16).float()
    exp = (n / 0.05).to(torch.float8_e4m3fn)
    assert _rel(got.float(), exp.float()) < 2e-2


def test_quant_nvfp4_activations():
    torch.manual_seed(3)
    T, K = 200, 256
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    gs = (448.0 * 6.0 / x.float().abs().max()).reshape(1).float()
    packed, sf = Q.quant_nvfp4(x, gs)
    deq = Q.ref_dequant_nvfp4(packed, sf, (1.0 / gs))
    fro = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()   # format quality: a norm bound
    assert fro(deq, x) < 0.12
    # fused silu(gate) * up
    gu = torch.randn(T, 2 * K, device=DEV).to(torch.bfloat16)
    y = (torch.nn.functional.silu(gu[:, :K].float()) * gu[:, K:].float()).to(torch.bfloat16)
    gs2 = (448.0 * 6.0 / y.float().abs().max()).reshape(1).float()
    p2, s2 = Q.quant_nvfp4(gu, gs2, silu_mul=True)
    assert fro(Q.ref_dequant_nvfp4(p2, s2, 1.0 / gs2), y) < 0.12
    # swizzled scale layout holds the same bytes
    p3, s3 = Q.quant_nvfp4(x, gs, swizzle=True)
    assert torch.equal(p3, packed)
    t, gidx = 77, 5
    off = ((t // 128) * (K // 64) + gidx // 4) * 512 + (t % 32) * 16 + ((t % 128) // 32) * 4 + gidx % 4
    assert s3[off].item() == sf[t, gidx].item()


@pytest.mark.parametrize("n_tile", [128, 256])
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (64, 768, 1024), (200, 1280, 2048), (16, 5120, 5120),
                                   (1000, 520, 512)])
def test_gemm_nvfp4_w4a4_block_scaled_mma(M, N, K, n_tile):
    """kind::mxf4nvf4 with both operands in NVFP4 and the block scales in tensor memory, against the
    fp32 product of the dequantised operands (the GEMM itself is exact up to the bf16 output)."""
    torch.manual_seed(2)
    x = (torch.randn(M, K, device=DEV) * 0.7).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV) * 0.05
    wp, wsf, g_w = Q.ref_quant_nvfp4_weights(w)
    g_a = (448.0 * 6.0 / x.float().abs().max()).reshape(1)
    ap, sfa = Q.quant_nvfp4(x, g_a, swizzle=True)
    sfa_rows = Q.quant_nvfp4(x, g_a, swizzle=False)[1]
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    out = Q.gemm_nvfp4(ap, sfa, g_a, wp, Q.nvfp4_sf_chunks(wsf, 256), g_w, bias=bias, n_tile=n_tile)
    assert ops.read_status() == 0
    a_deq = Q.ref_dequant_nvfp4(ap, sfa_rows, 1.0 / g_a)
    exp = a_deq @ Q.ref_dequant_nvfp4(wp, wsf, g_w).t() + bias.float()
    assert _rel(out, exp) < 6e-3
    # and the quantisation error of the activations stays what 4 bits allow
    full = x.float() @ Q.ref_dequant_nvfp4(wp, wsf, g_w).t() + bias.float()
    assert ((out.float() - full).norm() / full.norm()).item() < 0.2


def test_nvfp4_fused_producers():
    """RMSNorm -> NVFP4 (with the residual add) and x * sigmoid(gate) -> NVFP4 give the same bytes as
    the separate norm / gate kernel followed by the plain quantiser."""
    torch.manual_seed(5)
    T, K = 70, 512
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    res = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    w = (torch.rand(K, device=DEV) + 0.5).to(torch.bfloat16)
    gs = torch.full((1,), 300.0, device=DEV)
    r1 = res.clone()
    normed = ops.rmsnorm(x, w, 1e-6, residual=r1)
    p_ref, s_ref = Q.quant_nvfp4(normed, gs)
    r2 = res.clone()
    n2 = torch.empty_like(normed)
    p, s = Q.rmsnorm_quant_nvfp4(x, w, 1e-6, gs, residual=r2, normed=n2)
    assert torch.equal(r1, r2)
    # the fused kernel repeats the norm kernel's arithmetic and the quantiser's: the same bytes
    assert torch.equal(n2, normed)
    assert torch.equal(p, p_ref) and torch.equal(s, s_ref)
    deq = Q.ref_dequant_nvfp4(p, s, 1.0 / gs)
    assert ((deq - n2.float()).norm() / n2.float().norm()).item() < 0.12
    # swizzled scales carry the same bytes
    p3, s3 = Q.rmsnorm_quant_nvfp4(x, w, 1e-6, gs, residual=res.clone(), swizzle=True)
    assert torch.equal(p3, p)
    t, gidx = 69, 7
    off = ((t // 128) * (K // 64) + gidx // 4) * 512 + (t % 32) * 16 + ((t % 128) // 32) * 4 + gidx % 4
    assert int(s3[off]) == int(s[t, gidx])
    # gated
    a = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    g = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    gated = ops.sigmoid_mul(a, g)
    pg_ref, sg_ref = Q.quant_nvfp4(gated, gs)
    pg, sg = Q.quant_nvfp4_gated(a, g, gs)
    assert (pg == pg_ref).float().mean() > 0.97 and (sg == sg_ref).float().mean() > 0.97
    assert ops.read_status() == 0


def test_nvfp4_plan_cache_and_autotune(monkeypatch):
    """Tile-width plans: the heuristic for wide and narrow projections, and the timed choice."""
    Q._NVFP4_PLANS.clear()
    assert Q.nvfp4_plan(64, 34816, 5120) == 256
    assert Q.nvfp4_plan(64, 5120, 17408) == 128
    assert Q.nvfp4_plan(4096, 5120, 17408) == 256
    assert (64, 34816, 5120) in Q._NVFP4_PLANS
    monkeypatch.setenv("B200_NVFP4_AUTOTUNE", "1")
    Q._NVFP4_PLANS.clear()
    torch.manual_seed(3)
    M, N, K = 32, 1024, 1024
    x = (torch.randn(M, K, device=DEV) * 0.5).to(torch.bfloat16)
    wp, wsf, g_w = Q.ref_quant_nvfp4_weights(torch.randn(N, K, device=DEV) * 0.05)
    g_a = (448.0 * 6.0 / x.float().abs().max()).reshape(1)
    ap, sfa = Q.quant_nvfp4(x, g_a, swizzle=True)
    sfw = Q.nvfp4_sf_chunks(wsf, 256)
    a = Q.gemm_nvfp4(ap, sfa, g_a, wp, sfw, g_w)
    assert Q._NVFP4_PLANS[(64, N, K)] in (128, 256)
    b = Q.gemm_nvfp4(ap, sfa, g_a, wp, sfw, g_w, n_tile=384 - Q._NVFP4_PLANS[(64, N, K)])
    assert torch.equal(a, b)                  # the tile width changes the schedule, not the sums
    assert ops.read_status() == 0
