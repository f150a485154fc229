"""Fusion recipes on the GPU: the interpreter gives the bytes of the step-by-step composite, and the
bespoke kernels agree with both up to the last bit of a normalised value."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from vllm_cpp_b200 import ops  # noqa: E402
from vllm_cpp_b200.ops import recipes as R  # noqa: E402

DEV = "cuda"


def _inputs(recipe, T, K, D):
    torch.manual_seed(7)
    bf = lambda *s: torch.randn(*s, device=DEV).to(torch.bfloat16)
    t = {"eps": 1e-6, "scale": torch.tensor([0.04], device=DEV), "gscale": torch.tensor([250.0], device=DEV)}
    for name in recipe.inputs:
        t[name] = bf(T, K)
    t["w"] = (torch.rand(D if recipe.per_head else K, device=DEV) + 0.5).to(torch.bfloat16)
    return t


def _same(a, b):
    if isinstance(a, tuple):
        return all(_same(x, y) for x, y in zip(a, b))
    if a.dtype == torch.float8_e4m3fn:
        a, b = a.view(torch.uint8), b.view(torch.uint8)
    return torch.equal(a, b)


def _close(a, b, frac=0.97):
    if isinstance(a, tuple):
        return all(_close(x, y, frac) for x, y in zip(a, b))
    if a.dtype == torch.float8_e4m3fn:
        a, b = a.view(torch.uint8), b.view(torch.uint8)
    if a.dtype == torch.uint8:
        return (a == b).float().mean().item() > frac
    return (a.float() - b.float()).abs().max().item() <= 2 ** -7 * b.float().abs().max().item()


@pytest.mark.parametrize("T,K,D", [(3, 64, 32), (70, 512, 128), (130, 4096, 128), (17, 1024, 64)])
@pytest.mark.parametrize("name", sorted(n for n, r in R.CATALOG.items() if r.interpretable))
def test_interpreter_matches_composite_bytes(name, T, K, D):
    r = R.CATALOG[name]
    base = _inputs(r, T, K, D)
    a = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in base.items()}
    b = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in base.items()}
    want = R.run(r, a, tier="composite")
    got = R.run(r, b, tier="interpreter")
    assert ops.read_status() == 0
    for o in r.outputs:
        assert _same(got[o], want[o]), (name, o)
    if "residual" in base:
        assert torch.equal(a["residual"], b["residual"])
    if r.bespoke:
        c = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in base.items()}
        fused = R.run(r, c, tier="bespoke")
        for o in r.outputs:
            assert _close(fused[o], want[o]), (name, o)


def test_interpreter_swizzled_scales_and_strided_views():
    """NVFP4 scales in the chunk layout of the block-scaled MMA, and gate / up as the two halves of
    one merged projection output (row stride 2K)."""
    r = R.SILU_MUL_QUANT_NVFP4
    torch.manual_seed(1)
    T, K = 150, 256
    gu = torch.randn(T, 2 * K, device=DEV).to(torch.bfloat16)
    t = {"gate": gu[:, :K], "up": gu[:, K:], "gscale": torch.tensor([300.0], device=DEV), "swizzle": True}
    pk_i, sf_i = R.run(r, dict(t), tier="interpreter")["q"]
    pk_b, sf_b = R.run(r, dict(t), tier="bespoke")["q"]
    assert torch.equal(pk_i, pk_b)
    # rows past T of the last 128-row chunk are not written by either
    rows = torch.arange(T, device=DEV)
    for g in (0, 5, 15):
        off = ((rows // 128) * (K // 64) + g // 4) * 512 + (rows % 32) * 16 + ((rows % 128) // 32) * 4 + g % 4
        assert torch.equal(sf_i[off], sf_b[off])
    assert ops.read_status() == 0


def test_run_picks_one_launch_for_a_recipe_without_a_bespoke_kernel():
    r = R.RMSNORM_GATED_QUANT_FP8
    t = _inputs(r, 40, 2048, 128)
    q = R.run(r, dict(t))["q"]                       # default tier: the interpreter
    from vllm_cpp_b200.ops.gdn import ref_rmsnorm_gated
    y = ref_rmsnorm_gated(t["x"], t["z"], t["w"], heads=16).float()
    err = (q.float() * 0.04 - y).norm() / y.norm()
    assert err.item() < 0.05


def test_interpreter_refuses_what_it_cannot_run():
    r = R.RMSNORM_QUANT_FP8
    t = _inputs(r, 4, 36, 36)                         # width not a multiple of 8
    with pytest.raises(RuntimeError):
        R.run(r, t, tier="interpreter")
