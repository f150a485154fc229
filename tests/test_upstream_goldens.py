"""Op parity against golden vectors recorded from upstream vLLM.

The reference project ships, with its own parity tests, ``.npy`` inputs and outputs of pinned
upstream ops (``tests/parity/goldens/<case>/manifest.json``: op, arguments, tensors, tolerances).
When a checkout of the reference sits beside this repository (or ``B200_GOLDENS_DIR`` points at the
directory) these tests feed the same inputs to this engine's restatements and CPU kernels and hold
them to the recorded outputs with the recorded tolerances; elsewhere they skip. Only the data
files are read."""
import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch


def _goldens_dir():
    env = os.environ.get("B200_GOLDENS_DIR")
    cands = [Path(env)] if env else []
    here = Path(__file__).resolve()
    if len(here.parents) > 2:
        cands += [here.parents[2] / "reference" / "tests" / "parity" / "goldens"]
    for c in cands:
        if c.is_dir():
            return c
    return None


G = _goldens_dir()
pytestmark = pytest.mark.skipif(G is None, reason="no golden vectors on this machine")


def load(case):
    d = G / case
    if not (d / "manifest.json").exists():
        pytest.skip(f"case {case} not in this set of goldens")
    m = json.loads((d / "manifest.json").read_text())
    t = {}
    for name, spec in m["tensors"].items():
        a = np.load(d / spec["file"])
        if spec["dtype"] == "bf16":
            ten = torch.from_numpy(a.astype(np.int32)).to(torch.int16).view(torch.bfloat16) if a.dtype == np.uint16 \
                else torch.from_numpy(a).to(torch.bfloat16)
        else:
            ten = torch.from_numpy(a)
        t[name] = ten
    return m, t


def close(got, want, tol):
    atol, rtol = (tol or {}).get("atol", 1e-5), (tol or {}).get("rtol", 1e-5)
    g, w = got.float(), want.float()
    assert g.shape == w.shape, (g.shape, w.shape)
    bad = (g - w).abs() > atol + rtol * w.abs()
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} off; worst {(g - w).abs().max().item():.3e}"


# ------------------------------------------------------------------ norms, activations, glue
@pytest.mark.parametrize("case", ["rmsnorm_f32_8x128", "rmsnorm_bf16_8x128", "rmsnorm_gemma_bf16_8x128",
                                  "rmsnorm_fused_residual_f32_8x128"])
def test_rmsnorm(case):
    from vllm_cpp_b200.ops import reference as R
    m, t = load(case)
    a = m["args"]
    if a.get("fused_residual"):
        y, r = R.rmsnorm(t["x"], t["weight"], a["eps"], residual=t["residual_in"], gemma=a.get("gemma", False))
        close(r, t["residual_out"], m["tol"])
    else:
        y = R.rmsnorm(t["x"], t["weight"], a["eps"], gemma=a.get("gemma", False))[0]
    close(y, t["out"], m["tol"])
    if t["x"].dtype == torch.bfloat16 and not a.get("fused_residual"):
        # the CPU backend's kernel on the same vectors
        from vllm_cpp_b200.ops import cpu_native as N
        close(N.rmsnorm(t["x"].contiguous(), t["weight"], a["eps"], None, None, a.get("gemma", False)), t["out"], m["tol"])


def test_silu_and_mul():
    from vllm_cpp_b200.ops import cpu_native as N, reference as R
    m, t = load("silu_and_mul_bf16_8x256")
    close(R.act_and_mul(t["x"], 0), t["out"], m["tol"])
    close(N.act_and_mul(t["x"].contiguous(), 0), t["out"], m["tol"])


def test_embedding_and_matmul():
    from vllm_cpp_b200.models.backend import CpuBackend
    from vllm_cpp_b200.ops import reference as R
    m, t = load("embedding_bf16_32ids")
    close(CpuBackend("cpu").embedding(t["ids"], t["table"]), t["out"], m["tol"])
    m, t = load("matmul_bf16_16x64x32")
    close(R.gemm(t["a"], t["b"].t().contiguous(), out_dtype=torch.float32), t["out"], m["tol"])


@pytest.mark.parametrize("case", ["l2norm_f32_small", "l2norm_f32_realdims"])
def test_l2norm(case):
    m, t = load(case)
    x = t["x"].float()
    close(x * torch.rsqrt((x * x).sum(-1, keepdim=True) + m["args"]["eps"]), t["out"], m["tol"])


@pytest.mark.parametrize("case", ["rmsnorm_gated_f32_small_silu", "rmsnorm_gated_f32_realdims_silu",
                                  "rmsnorm_gated_f32_realdims_sigmoid"])
def test_rmsnorm_gated(case):
    m, t = load(case)
    a = m["args"]
    x, z, w = t["x"].float(), t["gate"].float(), t["weight"].float()
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + a["eps"]) * w
    y = y * (torch.nn.functional.silu(z) if a["activation"] in ("silu", "swish") else torch.sigmoid(z))
    close(y, t["out"], m["tol"])
    # and the engine's restatement (bf16 in / out) within bf16 rounding of it
    from vllm_cpp_b200.ops.gdn import ref_rmsnorm_gated
    got = ref_rmsnorm_gated(t["x"].to(torch.bfloat16), t["gate"].to(torch.bfloat16), t["weight"].to(torch.bfloat16),
                            a["eps"], "silu" if a["activation"] in ("silu", "swish") else "sigmoid")
    assert ((got.float() - t["out"].float()).abs() <= 0.03 * t["out"].float().abs() + 0.03).all()


# ------------------------------------------------------------------ rotary embeddings
@pytest.mark.parametrize("case", ["rope_f32_pos_short", "rope_f32_pos_131k"])
def test_rope_base(case):
    from vllm_cpp_b200.ops import reference as R
    m, t = load(case)
    a = m["args"]
    D, rot, hq, hkv = a["head_size"], a["rotary_dim"], a["num_q_heads"], a["num_kv_heads"]
    inv = R.rope_inv_freq(rot, a["base"])
    table = R.rope_table(inv, int(t["positions"].max()) + 1)
    T = t["positions"].numel()
    qkv = torch.cat([t["q_in"], t["k_in"], torch.zeros(T, hkv * D)], 1)
    q, k, _ = R.rope_kv(qkv, t["positions"], table, hq, hkv, D, rot_dim=rot, neox=True)
    close(q.reshape(T, -1), t["q_out"], m["tol"])
    close(k.reshape(T, -1), t["k_out"], m["tol"])


def _rope_cfg(p, neox):
    from vllm_cpp_b200.config import RopeConfig
    kind = p.get("rope_type", "default")
    c = RopeConfig(theta=p["rope_theta"], rotary_dim=p.get("rope_dim"), neox=neox,
                   scaling_type=None if kind == "default" else kind, factor=p.get("factor", 1.0),
                   low_freq_factor=p.get("low_freq_factor", 1.0), high_freq_factor=p.get("high_freq_factor", 4.0),
                   original_max_position=p.get("original_max_position_embeddings", 8192),
                   beta_fast=p.get("beta_fast", 32.0), beta_slow=p.get("beta_slow", 1.0),
                   attn_factor=p.get("attn_factor", 1.0), short_factor=p.get("short_factor"),
                   long_factor=p.get("long_factor"), mrope_section=p.get("mrope_section"), alpha=p.get("alpha"),
                   truncate=p.get("truncate", True), extrapolation_factor=p.get("extrapolation_factor", 1.0),
                   apply_yarn_scaling=p.get("apply_yarn_scaling", True), short_mscale=p.get("short_mscale"),
                   long_mscale=p.get("long_mscale"))
    return c


LONG_ROPE = ["long_rope_llama3_neox_f32_bands", "long_rope_llama3_neox_f32_equal_factors",
             "long_rope_llama3_gptj_bf16_bands", "long_rope_yarn_neox_bf16", "long_rope_yarn_neox_f32_truncate",
             "long_rope_dynamic_alpha_neox_f32", "long_rope_dynamic_factor1_neox_f32",
             "long_rope_dynamic_factor_gptj_bf16", "long_rope_phi3_neox_f32_short", "long_rope_phi3_neox_bf16_long",
             "long_rope_yarn_mrope_f32_text_1d", "long_rope_yarn_gptj_f32_untruncated_no_mscale",
             "long_rope_phi3_neox_f32_mscale_override"]


@pytest.mark.parametrize("case", LONG_ROPE)
def test_long_context_rope(case):
    """Llama-3 bands, YaRN, dynamic NTK (factor and alpha), Phi-3 LongRoPE: the cos/sin table the
    engine builds and the rotated q / k against upstream's."""
    from vllm_cpp_b200.models.rope import rope_parameters
    from vllm_cpp_b200.ops import reference as R
    m, t = load(case)
    a = m["args"]
    p = a["rope_parameters"]
    cfg = _rope_cfg(p, a["is_neox_style"])
    D, hq, hkv = a["head_size"], a["num_q_heads"], a["num_kv_heads"]
    rot = cfg.rotary_dim or D
    max_pos = a.get("max_model_len", a["max_position"])
    want_table = t["cos_sin_cache"].float()
    if p["rope_type"] == "longrope":
        # upstream keeps both tables back to back ([short ; long], the long one used once a
        # position passes the original window); the engine builds the one its length calls for
        cfg.config_max_position = a["max_position"]
        orig = p["original_max_position_embeddings"]
        inv_s, msc_s, _ = rope_parameters(cfg, D, orig)
        inv_l, msc_l, _ = rope_parameters(cfg, D, a["max_position"])
        close(R.rope_table(inv_s, orig, msc_s)[:, :rot], want_table[:orig], m["tol"])
        close(R.rope_table(inv_l, want_table.shape[0] - orig, msc_l)[:, :rot], want_table[orig:], m["tol"])
        long = bool((t["positions"] > orig).any())
        inv, msc = (inv_l, msc_l) if long else (inv_s, msc_s)
        table = R.rope_table(inv, int(t["positions"].max()) + 1, msc)
    else:
        inv, msc, tlen = rope_parameters(cfg, D, max_pos)
        table = R.rope_table(inv, want_table.shape[0], msc)
        close(table[:, : rot], want_table, m["tol"])
    T = t["positions"].numel()
    qkv = torch.cat([t["q_in"].float(), t["k_in"].float(), torch.zeros(T, hkv * D)], 1)
    q, k, _ = R.rope_kv(qkv, t["positions"], table, hq, hkv, D, rot_dim=rot, neox=a["is_neox_style"])
    close(q.reshape(T, -1), t["q_out"], m["tol"])
    close(k.reshape(T, -1), t["k_out"], m["tol"])


# ------------------------------------------------------------------ Gated DeltaNet
@pytest.mark.parametrize("case", ["causal_conv1d_fwd_f32_small", "causal_conv1d_fwd_f32_realdims"])
def test_causal_conv1d_fwd(case):
    from vllm_cpp_b200.ops.gdn import ref_conv1d
    m, t = load(case)
    n = t["conv_state_in"].shape[0]
    out, st = ref_conv1d(t["x"], t["weight"], t["conv_state_in"].clone(), t["query_start_loc"].tolist(),
                         list(range(n)), t["has_initial_state"].tolist())
    close(out, t["out"], {"atol": 4e-3, "rtol": 8e-3})           # the restatement returns bf16 rows
    close(st, t["conv_state_out"], m["tol"])


@pytest.mark.parametrize("case", ["causal_conv1d_update_f32_small", "causal_conv1d_update_f32_realdims"])
def test_causal_conv1d_update(case):
    from vllm_cpp_b200.ops.gdn import ref_conv1d
    m, t = load(case)
    B = t["x"].shape[0]
    out, st = ref_conv1d(t["x"], t["weight"], t["conv_state_in"].clone(), list(range(B + 1)), list(range(B)), [1] * B)
    close(out, t["out"], {"atol": 4e-3, "rtol": 8e-3})
    close(st, t["conv_state_out"], m["tol"])


@pytest.mark.parametrize("case", ["gdn_prefill_f32_small", "gdn_prefill_f32_small_noinit", "gdn_prefill_f32_realdims"])
def test_gdn_prefill(case):
    """The sequential gated delta rule over variable-length sequences (state [Hv, Dv, Dk])."""
    from vllm_cpp_b200.ops.gdn import ref_recurrent
    m, t = load(case)
    a = m["args"]
    qsl = t["query_start_loc"].tolist()
    assert abs(a["scale"] - a["Dk"] ** -0.5) < 1e-6              # the restatement applies Dk ** -0.5 itself
    outs, states = [], []
    for i in range(len(qsl) - 1):
        b, e = qsl[i], qsl[i + 1]
        q, k = t["q"][b:e], t["k"][b:e]
        s0 = t["state_in"][i] if a.get("with_initial_state", True) and "state_in" in t else \
            torch.zeros_like(t["state_out"][i])
        o, s1 = ref_recurrent(q, k, t["v"][b:e], t["g"][b:e], t["beta"][b:e], s0)
        outs.append(o)
        states.append(s1)
    close(torch.cat(outs, 0), t["out"], m["tol"])
    close(torch.stack(states, 0), t["state_out"], m["tol"])


@pytest.mark.parametrize("case", ["gdn_decode_f32_small", "gdn_decode_f32_realdims"])
def test_gdn_decode(case):
    from vllm_cpp_b200.ops.gdn import ref_recurrent
    m, t = load(case)
    a = m["args"]
    assert abs(a["scale"] - a["Dk"] ** -0.5) < 1e-6
    B = t["v"].shape[0]
    outs, states = [], []
    for i in range(B):
        q, k = t["q_l2"][i: i + 1], t["k_l2"][i: i + 1]
        o, s1 = ref_recurrent(q, k, t["v"][i: i + 1], t["g"][i: i + 1], t["beta"][i: i + 1], t["state_in"][i])
        outs.append(o)
        states.append(s1)
    close(torch.cat(outs, 0), t["out"], m["tol"])
    close(torch.stack(states, 0), t["state_out"], m["tol"])


# ------------------------------------------------------------------ MoE
@pytest.mark.parametrize("case", ["moe_router_topk_f32_small", "moe_router_topk_f32_small_norenorm",
                                  "moe_router_topk_bf16_realratio"])
def test_moe_router(case):
    from vllm_cpp_b200.ops.moe import ref_router_topk
    m, t = load(case)
    a = m["args"]
    ids, w = ref_router_topk(t["logits"].float(), a["top_k"], renorm=a["renormalize"], scoring=a["scoring_func"])
    assert torch.equal(ids.to(torch.int32), t["topk_ids"])
    close(w, t["topk_weights"], m["tol"])
    if t["logits"].dtype == torch.bfloat16 or True:
        from vllm_cpp_b200.ops import cpu_native as N
        ids2, w2 = N.moe_router_topk(t["logits"].float().contiguous(), a["top_k"], renorm=a["renormalize"])
        assert torch.equal(ids2.to(torch.int32), t["topk_ids"])
        close(w2, t["topk_weights"], m["tol"])


def test_moe_block_f32():
    """Router + routed experts + sigmoid-gated shared expert in fp32 against upstream's block."""
    m, t = load("moe_block_f32_small")
    a = m["args"]
    x = t["x"]
    logits = x @ t["gate_w"].t()
    close(logits, t["router_logits"], m["tol"])
    from vllm_cpp_b200.ops.moe import ref_router_topk
    ids, w = ref_router_topk(logits, a["top_k"], renorm=a["renormalize"], scoring=a["scoring_func"])
    assert torch.equal(ids.to(torch.int32), t["topk_ids"])
    I = a["moe_intermediate"]
    routed = torch.zeros_like(x)
    for tok in range(x.shape[0]):
        for j in range(a["top_k"]):
            e = int(ids[tok, j])
            gu = t["w13"][e] @ x[tok]
            routed[tok] += w[tok, j] * (t["w2"][e] @ (torch.nn.functional.silu(gu[:I]) * gu[I:]))
    close(routed, t["routed_out"], {"atol": 1e-4, "rtol": 1e-4})
    S = a["shared_intermediate"]
    sgu = x @ t["w_shared_gate_up"].t()
    shared = (torch.nn.functional.silu(sgu[:, :S]) * sgu[:, S:]) @ t["w_shared_down"].t()
    shared = shared * torch.sigmoid(x @ t["w_shared_gate"].t())
    close(shared, t["shared_out"], {"atol": 1e-4, "rtol": 1e-4})
    close(routed + shared, t["out"], {"atol": 1e-4, "rtol": 1e-4})


# ------------------------------------------------------------------ gated attention block
@pytest.mark.parametrize("case", ["dense_attention_f32_small", "dense_attention_f32_realdims"])
def test_gated_attention(case):
    """Per-head qk RMSNorm (1 + w), partial rotary embedding, causal attention with grouped KV
    heads, sigmoid output gate: the attention half of the hybrid models' full-attention layers."""
    from vllm_cpp_b200.ops import reference as R
    m, t = load(case)
    a = m["args"]
    T, Hq, D = t["q"].shape
    Hkv = a["num_kv_heads"]
    rot = a["rotary_dim"]
    table = R.rope_table(R.rope_inv_freq(rot, a["base"]), int(t["positions"].max()) + 1)
    qkv = torch.cat([t["q"].reshape(T, -1), t["k"].reshape(T, -1), t["v"].reshape(T, -1)], 1)
    q, k, v = R.rope_kv(qkv, t["positions"], table, Hq, Hkv, D, rot_dim=rot, neox=True,
                        q_norm=t["q_norm_weight"], k_norm=t["k_norm_weight"], eps=a["eps"], gemma=True)
    rep = Hq // Hkv
    kf, vf = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = torch.einsum("thd,shd->hts", q.float(), kf) * a["scale"]
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    attn = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vf)
    close(attn, t["attn"], m["tol"])
    close((attn * torch.sigmoid(t["gate"])).reshape(T, -1), t["out"], m["tol"])


def test_gdn_prefill_bf16_against_the_chunked_oracle():
    """bf16 inputs, upstream's chunked kernel as the oracle, one sequence with and one without an
    initial state: the sequential restatement at the recorded bf16 tolerance, and the CPU backend's
    native recurrence on the same vectors."""
    from vllm_cpp_b200.ops.gdn import ref_recurrent
    m, t = load("gdn_prefill_bf16_realdims")
    a = m["args"]
    qsl = t["query_start_loc"].tolist()
    init = a["with_initial_state"]
    outs, states = [], []
    for i in range(len(qsl) - 1):
        b, e = qsl[i], qsl[i + 1]
        s0 = t["state_in"][i].float() if init[i] else torch.zeros_like(t["state_out"][i])
        o, s1 = ref_recurrent(t["q"][b:e], t["k"][b:e], t["v"][b:e], t["g"][b:e].float(), t["beta"][b:e].float(), s0)
        outs.append(o)
        states.append(s1)
    close(torch.cat(outs, 0), t["out"], m["tol"])
    close(torch.stack(states, 0), t["state_out"], m["tol"])
    from vllm_cpp_b200.ops import cpu_native as N
    ssm = torch.stack([t["state_in"][i].float() if init[i] else torch.zeros_like(t["state_out"][i])
                       for i in range(len(init))], 0).contiguous()
    out = N.gdn_recurrent(t["q"].to(torch.bfloat16).contiguous(), t["k"].to(torch.bfloat16).contiguous(),
                          t["v"].to(torch.bfloat16).contiguous(), t["g"].float().contiguous(),
                          t["beta"].float().contiguous(), ssm, qsl, list(range(len(init))), [1] * len(init))
    close(out.float(), t["out"], {"atol": 1e-2, "rtol": 1e-2})
    close(ssm, t["state_out"], {"atol": 1e-2, "rtol": 1e-2})


def test_gdn_packed_decode_gating_and_step():
    """One decode step of the packed kernel's contract: g = -exp(A_log) * softplus(a + dt_bias),
    beta = sigmoid(b), q / k L2-normalised in the kernel, bf16 state in and out."""
    from vllm_cpp_b200.ops.gdn import ref_post_conv, ref_recurrent
    m, t = load("gdn-packed-decode-oracle")
    a = m["args"]
    Hk, Hv, B = a["Hk"], a["Hv"], a["batch"]
    qn, kn, g, beta = ref_post_conv(t["mixed_qkv"], Hk, Hv, t["a"], t["b"], t["A_log"], t["dt_bias"])
    close(g, t["g"], {"atol": 2e-3, "rtol": 2e-3})
    close(beta, t["beta_full_f32"], {"atol": 2e-3, "rtol": 2e-3})
    v = t["mixed_qkv"][:, 2 * Hk * 128:].reshape(B, Hv, 128)
    assert torch.equal(v, t["v"])
    idx = t["state_indices"].tolist()
    for i in range(B):
        o, s1 = ref_recurrent(qn[i: i + 1], kn[i: i + 1], v[i: i + 1], g[i: i + 1], beta[i: i + 1],
                              t["state_in"][idx[i]].float())
        close(o[0], t["out"][i], {"atol": 2e-2, "rtol": 2e-2})
        close(s1, t["state_out"][idx[i]], {"atol": 2e-2, "rtol": 2e-2})


def test_moe_block_bf16_layer_contract():
    """The sparse-MoE block of the hybrid MoE models in bf16 (router, routed experts, gated shared
    expert): this engine's restatement and its CPU kernels against upstream's layer output."""
    from vllm_cpp_b200.ops import cpu_native as N
    from vllm_cpp_b200.ops.moe import ref_moe_block, ref_router_topk
    m, t = load("moe_block_bf16_small")
    a = m["args"]
    x = t["x"]
    logits = x.float() @ t["gate_w"].float().t()
    ids, w = ref_router_topk(logits, a["top_k"], renorm=a["renormalize"], scoring=a["scoring_func"])
    assert torch.equal(ids.to(torch.int32), t["topk_ids"])
    routed = ref_moe_block(x, ids, w, t["w13"], t["w2"])
    S = a["shared_intermediate"]
    sgu = (x.float() @ t["w_shared_gate_up"].float().t()).to(torch.bfloat16).float()
    act = (torch.nn.functional.silu(sgu[:, :S]) * sgu[:, S:]).to(torch.bfloat16).float()
    shared = (act @ t["w_shared_down"].float().t()) * torch.sigmoid(x.float() @ t["w_shared_gate"].float().t())
    close(routed.float() + shared, t["out"], m["tol"])
    native = N.moe_experts(x.contiguous(), ids.to(torch.int32), w.float(), t["w13"].contiguous(), t["w2"].contiguous(),
                           e0=0, act_kind=0)
    close(native.float() + shared, t["out"], m["tol"])


# ------------------------------------------------------------------ tokenizer
def test_tokenizer_against_recorded_encodings():
    """A SentencePiece-style BPE tokenizer file with byte fallback (Metaspace pre-tokenizer that
    does not split, so runs of spaces merge) and the ids / decoded text the HF tokenizers library
    produced for a corpus of edge cases: byte-exact both ways."""
    from vllm_cpp_b200 import _engine as E
    d = G / "tokenizer_mistral"
    if not (d / "tokenizer.json").exists():
        pytest.skip("this set of goldens has no tokenizer file")
    tok = E.Tokenizer.from_hf_json((d / "tokenizer.json").read_text(encoding="utf-8"), "")
    rec = json.loads((d / "encodings.json").read_text(encoding="utf-8"))
    assert tok.bos_id == rec["bos_id"]
    for ent in rec["entries"]:
        assert list(tok.encode(ent["text"], False)) == ent["ids"], ent["text"]
        assert list(tok.encode(ent["text"], True)) == ent["ids_special"], ent["text"]
        assert tok.decode(ent["ids"], False) == ent["decode"], ent["text"]


@pytest.mark.parametrize("case", ["long_rope_yarn_mrope_bf16_interleaved", "long_rope_yarn_mrope_f32_contiguous"])
def test_sectioned_rotary_positions(case):
    """Three position streams (temporal, height, width) over sections of the frequencies, in the
    contiguous and the interleaved layout, on a YaRN table."""
    from vllm_cpp_b200.models.rope import mrope_cos_sin, rope_parameters
    from vllm_cpp_b200.ops import reference as R
    m, t = load(case)
    a = m["args"]
    p = a["rope_parameters"]
    cfg = _rope_cfg(p, a["is_neox_style"])
    D, hq, hkv = a["head_size"], a["num_q_heads"], a["num_kv_heads"]
    rot = cfg.rotary_dim or D
    inv, msc, _ = rope_parameters(cfg, D, a["max_position"])
    want_table = t["cos_sin_cache"].float()
    table = R.rope_table(inv, want_table.shape[0], msc)[:, :rot]
    close(table, want_table, m["tol"])
    cos, sin = mrope_cos_sin(table, t["positions"], p["mrope_section"], bool(p.get("mrope_interleaved")))
    T = t["positions"].shape[-1]
    q = R.apply_rope(t["q_in"].float().reshape(T, hq, D), cos, sin, rot, a["is_neox_style"])
    k = R.apply_rope(t["k_in"].float().reshape(T, hkv, D), cos, sin, rot, a["is_neox_style"])
    close(q.reshape(T, -1), t["q_out"], m["tol"])
    close(k.reshape(T, -1), t["k_out"], m["tol"])
