"""Gated DeltaNet kernels against fp32 PyTorch restatements: conv1d (varlen + state, decode
update), post-conv prep, the tcgen05 chunked scan against the sequential recurrence, packed
decode, gated RMSNorm."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from vllm_cpp_b200 import ops  # noqa: E402
from vllm_cpp_b200.ops import gdn as G  # noqa: E402

DEV = "cuda"


def _rel(a, b):
    from _numerics import rel_err
    return rel_err(a, b, row_tol=0.15, abs_tol=0.1)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("lens,C", [([5, 1, 70, 2, 33], 256), ([300], 1280), ([1, 1, 1], 128)])
def test_conv1d_fwd_varlen_with_state(lens, C):
    torch.manual_seed(0)
    T = sum(lens)
    n = len(lens)
    x_full = (torch.randn(T, C + 64, device=DEV)).to(torch.bfloat16)
    x = x_full[:, 32:32 + C]                         # strided view
    w = (torch.randn(C, 4, device=DEV) * 0.5).to(torch.bfloat16)
    state = torch.randn(n + 2, C, 3, device=DEV).to(torch.bfloat16)
    qsl = [0]
    for l in lens:
        qsl.append(qsl[-1] + l)
    slots = list(range(n, 0, -1))                    # arbitrary slot assignment
    has_init = [(i % 2) for i in range(n)]
    exp_out, exp_state = G.ref_conv1d(x, w, state, qsl, slots, has_init)
    out = torch.zeros(T, C, dtype=torch.bfloat16, device=DEV)
    st = state.clone()
    G.conv1d_fwd(x, w, st, _i32(qsl), _i32(slots), _i32(has_init), out)
    assert _rel(out, exp_out) < 1e-2
    assert torch.equal(st, exp_state)


def test_conv1d_update_matches_fwd():
    torch.manual_seed(1)
    B, C = 7, 384
    w = (torch.randn(C, 4, device=DEV) * 0.5).to(torch.bfloat16)
    state = torch.randn(B, C, 3, device=DEV).to(torch.bfloat16)
    x = torch.randn(B, C, device=DEV).to(torch.bfloat16)
    slots = list(range(B))
    exp_out, exp_state = G.ref_conv1d(x, w, state, list(range(B + 1)), slots, [1] * B)
    out = torch.empty_like(x)
    st = state.clone()
    G.conv1d_update(x, w, st, _i32(slots), out)
    assert _rel(out, exp_out) < 1e-2
    assert torch.equal(st, exp_state)


def _gdn_inputs(T, Hk, Hv, seed=0, g_scale=1.0):
    torch.manual_seed(seed)
    conv_dim = 2 * Hk * 128 + Hv * 128
    xc = (torch.randn(T, conv_dim, device=DEV)).to(torch.bfloat16)
    a = (torch.randn(T, Hv, device=DEV) * g_scale).to(torch.bfloat16)
    b = torch.randn(T, Hv, device=DEV).to(torch.bfloat16)
    A_log = torch.log(torch.rand(Hv, device=DEV) * 4 + 0.5)
    dt_bias = torch.randn(Hv, device=DEV) * 0.5
    return xc, a, b, A_log, dt_bias


def test_post_conv():
    T, Hk, Hv = 37, 2, 6
    xc, a, b, A_log, dt_bias = _gdn_inputs(T, Hk, Hv)
    q = torch.empty(T, Hk, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.empty_like(q)
    g = torch.empty(T, Hv, device=DEV)
    beta = torch.empty(T, Hv, device=DEV)
    G.post_conv(xc, Hk, Hv, a, b, A_log, dt_bias, q, k, g, beta)
    eq, ek, eg, eb = G.ref_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias)
    assert _rel(q, eq) < 1e-2 and _rel(k, ek) < 1e-2
    assert torch.allclose(g, eg, rtol=1e-3, atol=1e-4) and torch.allclose(beta, eb, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("lens,Hk,Hv,with_state", [([64], 1, 1, False), ([128], 1, 2, False),
                                                   ([200, 17, 64, 1, 333], 2, 6, True),
                                                   ([1000], 2, 4, True)])
def test_chunk_scan_matches_recurrence(lens, Hk, Hv, with_state):
    T, n = sum(lens), len(lens)
    xc, a, b, A_log, dt_bias = _gdn_inputs(T, Hk, Hv, seed=3)
    q, k, g, beta = G.ref_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias)
    g, beta = g.contiguous(), beta.contiguous()
    v_col0 = 2 * Hk * 128
    v = xc[:, v_col0:].reshape(T, Hv, 128)
    qsl = [0]
    for l in lens:
        qsl.append(qsl[-1] + l)
    slots = [n - i for i in range(n)]
    has_init = [1 if (with_state and i % 2 == 0) else 0 for i in range(n)]
    state = (torch.randn(n + 2, Hv, 128, 128, device=DEV) * 0.1)
    st = state.clone()
    out = torch.zeros(T, Hv, 128, dtype=torch.bfloat16, device=DEV)
    ws = G.GdnWorkspace(torch.device(DEV), T, n, Hv)
    G.chunk_scan(q, k, xc, g, beta, st, qsl, _i32(slots), _i32(has_init), out, ws, v_col0=v_col0)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    for s in range(n):
        bgn, end = qsl[s], qsl[s + 1]
        s0 = state[slots[s]] if has_init[s] else torch.zeros_like(state[0])
        eo, es = G.ref_recurrent(q[bgn:end], k[bgn:end], v[bgn:end], g[bgn:end], beta[bgn:end], s0)
        assert _rel(out[bgn:end], eo) < 3e-2, f"seq {s} output"
        assert _rel(st[slots[s]], es) < 3e-2, f"seq {s} state"


def test_packed_decode_matches_recurrence():
    B, Hk, Hv = 5, 2, 6
    xc, a, b, A_log, dt_bias = _gdn_inputs(B, Hk, Hv, seed=5)
    q, k, g, beta = G.ref_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias)
    v = xc[:, 2 * Hk * 128:].reshape(B, Hv, 128)
    state = torch.randn(B + 1, Hv, 128, 128, device=DEV) * 0.1
    slots = [B - i for i in range(B)]
    st = state.clone()
    out = torch.empty(B, Hv, 128, dtype=torch.bfloat16, device=DEV)
    G.packed_decode(xc, a, b, A_log, dt_bias, st, _i32(slots), out, Hk, Hv)
    for i in range(B):
        eo, es = G.ref_recurrent(q[i:i + 1], k[i:i + 1], v[i:i + 1], g[i:i + 1], beta[i:i + 1], state[slots[i]])
        assert _rel(out[i], eo[0]) < 2e-2
        assert _rel(st[slots[i]], es) < 1e-2
    assert torch.equal(st[0], state[0])             # untouched slot


def test_rmsnorm_gated():
    torch.manual_seed(2)
    R, D, heads = 50, 128, 3
    x = torch.randn(R, heads * D, device=DEV).to(torch.bfloat16)
    zfull = torch.randn(R, 5 * D, device=DEV).to(torch.bfloat16)
    z = zfull[:, D:(1 + heads) * D]
    w = (torch.rand(D, device=DEV) + 0.5).to(torch.bfloat16)
    out = torch.empty_like(x)
    for gate in ("silu", "sigmoid"):
        G.rmsnorm_gated(x, z, w, out, gate=gate, heads=heads)
        assert _rel(out, G.ref_rmsnorm_gated(x, z, w, gate=gate, heads=heads)) < 1e-2
