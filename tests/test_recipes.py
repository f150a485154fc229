"""Fusion-recipe catalogue: lowering to interpreter programs (CPU) and the PyTorch composite."""
import pytest
import torch

from vllm_cpp_b200.ops import recipes as R


def test_catalogue_lists_every_recipe_with_its_tiers():
    names = set(R.CATALOG)
    assert {"fused_add_rmsnorm_gemma", "fused_add_rmsnorm", "rmsnorm_quant_fp8", "rmsnorm_gated_quant_fp8",
            "silu_mul_quant_nvfp4", "silu_mul_quant_fp8", "sigmoid_gate_quant_nvfp4", "attn_qk_norm_rope",
            "attn_qk_norm_rope_gate"} <= names
    for r in R.CATALOG.values():
        t = R.tiers(r)
        assert t, r.name
        if r.interpretable:
            assert "composite" in t and "interpreter" in t
    assert R.tiers(R.RMSNORM_GATED_QUANT_FP8)[0] == "interpreter"      # no bespoke kernel: one launch all the same
    assert R.tiers(R.SILU_MUL_QUANT_NVFP4)[0] == "bespoke"
    assert R.tiers(R.ATTN_QK_NORM_ROPE) == ("bespoke",)
    rows = R.describe()
    assert len(rows) == len(R.CATALOG) and all(r["reference"] for r in rows)


def test_lowering_reuses_registers_and_orders_loads_and_stores():
    p = R.lower(R.FUSED_ADD_RMSNORM)
    ops = [s[0] for s in p.steps]
    assert ops == [R.OP_LOAD, R.OP_LOAD, R.OP_ADD, R.OP_STORE, R.OP_RMSNORM, R.OP_STORE]
    assert p.n_regs == 2
    # the sum is stored over the residual input, the normalised row to its own output
    assert p.operands[p.steps[3][4]] == "residual" and p.operands[p.steps[5][4]] == "y"
    p = R.lower(R.ADD_RMSNORM_QUANT_NVFP4)
    assert [s[0] for s in p.steps] == [R.OP_LOAD, R.OP_LOAD, R.OP_ADD, R.OP_STORE, R.OP_RMSNORM, R.OP_QUANT_NVFP4]
    assert p.n_regs == 2 and {"q", "q.sf", "gscale", "w"} <= set(p.operands)
    p = R.lower(R.RMSNORM_GATED_QUANT_FP8)
    assert [s[0] for s in p.steps] == [R.OP_LOAD, R.OP_LOAD, R.OP_RMSNORM_GATED, R.OP_QUANT_FP8]
    with pytest.raises(NotImplementedError):
        R.lower(R.ATTN_QK_NORM_ROPE)
    for r in R.CATALOG.values():
        if r.interpretable:
            q = R.lower(r)
            assert len(q.steps) <= R.MAX_STEPS and q.n_regs <= R.MAX_REGS
            for op, dst, a, b, *_ in q.steps:
                assert max(dst, a, b) < q.n_regs


def test_lowering_rejects_a_value_used_before_it_is_made():
    bad = R.FusedRecipe("bad", ("x",), (), (R._s("add", "y", "x", "nope"),), ("y",))
    with pytest.raises(ValueError):
        R.lower(bad)


def test_chain_structs_match_the_c_layout():
    import ctypes
    assert ctypes.sizeof(R.B200ChainStep) == 36
    assert ctypes.sizeof(R.B200ChainOperand) == 24
    assert ctypes.sizeof(R.B200Chain) == 24 + 36 * R.MAX_STEPS + 24 * R.MAX_OPERANDS


def test_torch_composite_of_each_row_recipe():
    torch.manual_seed(0)
    T, K = 5, 64
    bf = lambda *s: torch.randn(*s).to(torch.bfloat16)
    x, res, w = bf(T, K), bf(T, K), (torch.rand(K) + 0.5).to(torch.bfloat16)
    r0 = res.clone()
    out = R.run("fused_add_rmsnorm", {"x": x, "residual": res, "w": w, "eps": 1e-6})
    h = (x.float() + r0.float()).to(torch.bfloat16)
    assert torch.equal(res, h) and torch.equal(out["h"], h)
    hf = h.float()
    want = (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-6) * w.float()).to(torch.bfloat16)
    assert torch.equal(out["y"], want)
    g = R.run("fused_add_rmsnorm_gemma", {"x": x, "residual": r0.clone(), "w": w, "eps": 1e-6})["y"]
    want_g = (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-6) * (w.float() + 1)).to(torch.bfloat16)
    assert torch.equal(g, want_g)
    scale = torch.tensor([0.05])
    q = R.run("silu_mul_quant_fp8", {"gate": x, "up": res, "scale": scale})["q"]
    y = (torch.nn.functional.silu(x.float()) * res.float()).to(torch.bfloat16).float()
    assert q.dtype == torch.float8_e4m3fn and (q.float() * 0.05 - y).abs().max() <= 0.07 * y.abs().max() + 0.05
    # gated norm over heads of 32 columns
    w32 = (torch.rand(32) + 0.5).to(torch.bfloat16)
    q = R.run("rmsnorm_gated_quant_fp8", {"x": x, "z": res, "w": w32, "eps": 1e-6, "scale": scale})["q"]
    from vllm_cpp_b200.ops.gdn import ref_rmsnorm_gated
    y = ref_rmsnorm_gated(x, res, w32, heads=2).float()
    assert (q.float() * 0.05 - y).abs().max() <= 0.07 * y.abs().max() + 0.05
    # NVFP4: packed codes and scales dequantise to the gated product within what 4 bits allow
    from vllm_cpp_b200.ops.quant import ref_dequant_nvfp4
    gs = torch.tensor([200.0])
    pk, sf = R.run("sigmoid_gate_quant_nvfp4", {"x": x, "gate": res, "gscale": gs})["q"]
    y = (x.float() * torch.sigmoid(res.float())).to(torch.bfloat16).float()
    deq = ref_dequant_nvfp4(pk, sf, 1.0 / gs)
    assert pk.shape == (T, K // 2) and sf.shape == (T, K // 16)
    assert ((deq - y).norm() / y.norm()).item() < 0.12


def test_activation_quantiser_reference_rounds_ties_to_the_even_code():
    from vllm_cpp_b200.ops.quant import ref_quant_nvfp4_activations
    # block maximum 6 with gscale 1: scale byte = e4m3(1.0), codes are the values themselves
    vals = torch.tensor([[6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, 0.0, 5.5]])
    pk, sf = ref_quant_nvfp4_activations(vals.to(torch.bfloat16), torch.tensor([1.0]))
    codes = torch.stack([pk[0] & 15, pk[0] >> 4], -1).reshape(-1).tolist()
    assert codes == [7, 0, 2, 2, 4, 4, 6, 6, 9, 10, 11, 12, 13, 14, 0, 7]
    assert sf.view(torch.float8_e4m3fn).float().item() == 1.0
