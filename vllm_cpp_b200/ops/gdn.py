"""Gated DeltaNet op wrappers (conv1d, post-conv prep, chunked scan, packed decode, gated
RMSNorm) and their fp32 PyTorch restatements (the sequential recurrence is the oracle for the
chunked tensor-core scan)."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr

_declared = False
CHUNK = 64


def _declare():
    global _declared
    if _declared:
        return
    P, I, L, F = _lib.P, _lib.I, _lib.L, _lib.F
    _lib.declare("b200_gdn_conv1d_fwd", [P, L, P, P, P, P, P, P, L, I, I, I, P], I)
    _lib.declare("b200_gdn_conv1d_update", [P, L, P, P, P, P, L, I, I, P], I)
    _lib.declare("b200_gdn_post_conv", [P, L, I, I, I, I, P, P, L, P, P, P, P, P, P, F, P], I)
    _lib.declare("b200_gdn_packed_decode", [P, L, P, P, L, P, P, P, P, P, I, I, I, I, I, F, P], I)
    _lib.declare("b200_rmsnorm_gated", [P, L, P, L, P, P, L, L, I, F, I, I, P], I)
    _lib.declare("b200_gdn_chunk_scan", [P, P, P, L, I, P, P, I, I, I, P, P, I, P, P, P, I, P, P, P, P,
                                         P, P, P, P], I)
    lib()
    _declared = True


def conv1d_fwd(x, w, conv_state, qsl, slots, has_init, out):
    """x/out: bf16 [T, C] (row-strided views allowed); w: bf16 [C, 4]; conv_state: bf16
    [slots, C, 3]; qsl int32 [n_seq + 1]; slots / has_init int32 [n_seq]."""
    _declare()
    T, C = x.shape
    n_seq = qsl.numel() - 1
    check(lib().b200_gdn_conv1d_fwd(ptr(x), x.stride(0), ptr(w), ptr(conv_state), ptr(qsl), ptr(slots),
                                    ptr(has_init), ptr(out), out.stride(0), n_seq, T, C, stream_ptr()),
          "gdn_conv1d_fwd")
    return out


def conv1d_update(x, w, conv_state, slots, out):
    _declare()
    B, C = x.shape
    check(lib().b200_gdn_conv1d_update(ptr(x), x.stride(0), ptr(w), ptr(conv_state), ptr(slots), ptr(out),
                                       out.stride(0), B, C, stream_ptr()), "gdn_conv1d_update")
    return out


def post_conv(xc, Hk, Hv, a, b, A_log, dt_bias, q_out, k_out, g, beta, eps=1e-6):
    """xc: bf16 [T, 2*Hk*128 + Hv*128] conv output; a, b: bf16 [T, Hv] (same row stride)."""
    _declare()
    T = xc.shape[0]
    assert a.stride(0) == b.stride(0)
    check(lib().b200_gdn_post_conv(ptr(xc), xc.stride(0), T, Hk, Hv, 128, ptr(a), ptr(b), a.stride(0),
                                   ptr(A_log), ptr(dt_bias), ptr(q_out), ptr(k_out), ptr(g), ptr(beta),
                                   eps, stream_ptr()), "gdn_post_conv")


def packed_decode(xc, a, b, A_log, dt_bias, state, slots, out, Hk, Hv, eps=1e-6):
    """One token per request: xc bf16 [B, conv_dim] (post-conv), state fp32
    [slots, Hv, 128, 128] updated in place, out bf16 [B, Hv, 128]."""
    _declare()
    B = xc.shape[0]
    check(lib().b200_gdn_packed_decode(ptr(xc), xc.stride(0), ptr(a), ptr(b), a.stride(0), ptr(A_log),
                                       ptr(dt_bias), ptr(state), ptr(slots), ptr(out), B, Hk, Hv, 128,
                                       128, eps, stream_ptr()), "gdn_packed_decode")
    return out


def rmsnorm_gated(x, z, w, out, eps=1e-6, gate="silu", heads=1):
    """out = rmsnorm(x) * w * gate(z) over groups of D = w.numel() columns. x, z, out: bf16
    [T, heads * D] row-strided (each head normalised on its own)."""
    _declare()
    T = x.shape[0]
    D = w.numel()
    assert x.shape[1] == heads * D
    check(lib().b200_rmsnorm_gated(ptr(x), x.stride(0), ptr(z), z.stride(0), ptr(w), ptr(out),
                                   out.stride(0), T * heads, D, eps, 0 if gate == "silu" else 1,
                                   heads, stream_ptr()), "rmsnorm_gated")
    return out


def build_chunk_table(qsl_host) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(chunk_tok0, chunk_len, seq_chunk0) for sequences given by host query_start_loc."""
    tok0, ln, seq0 = [], [], [0]
    for s in range(len(qsl_host) - 1):
        b, e = int(qsl_host[s]), int(qsl_host[s + 1])
        t = b
        while t < e:
            tok0.append(t)
            ln.append(min(CHUNK, e - t))
            t += CHUNK
        seq0.append(len(tok0))
    return (np.asarray(tok0, dtype=np.int32), np.asarray(ln, dtype=np.int32),
            np.asarray(seq0, dtype=np.int32))


class GdnWorkspace:
    """Scratch of the chunked scan for up to ``max_tokens`` tokens in ``max_seqs`` sequences."""

    def __init__(self, device, max_tokens: int, max_seqs: int, Hv: int):
        self.max_chunks = max_tokens // CHUNK + max_seqs + 1
        nt = self.max_chunks
        bf = dict(dtype=torch.bfloat16, device=device)
        self.u = torch.zeros((nt * CHUNK, Hv, 128), **bf)
        self.w = torch.zeros((nt * CHUNK, Hv, 128), **bf)
        self.qs = torch.zeros((nt * CHUNK, Hv, 128), **bf)
        self.p = torch.zeros((nt, Hv, CHUNK, CHUNK), **bf)
        self.gc = torch.zeros((nt, Hv, CHUNK), dtype=torch.float32, device=device)
        self.table = torch.zeros(3 * nt + max_seqs + 8, dtype=torch.int32, device=device)
        self.Hv = Hv


def chunk_scan(q, k, v, g, beta, state, qsl_host, slots, has_init, out, ws: GdnWorkspace, v_col0=0,
               table=None):
    """q, k: bf16 [T, Hk, 128] normalised; v: bf16 2-D row-strided tensor whose columns
    [v_col0 + hv*128, ...) hold the value heads; g, beta: fp32 [T, Hv]; state fp32
    [slots, Hv, 128, 128]; out bf16 [T, Hv, 128]. ``table`` = device (tok0, len, seq0) views
    if the caller staged them already, else they are built from ``qsl_host`` and copied."""
    _declare()
    T, Hk, _ = q.shape
    Hv = g.shape[1]
    n_seq = len(qsl_host) - 1
    if table is None:
        t0, ln, s0 = build_chunk_table(qsl_host)
        NT = len(t0)
        assert NT <= ws.max_chunks
        host = np.concatenate([t0, ln, s0])
        ws.table[: host.size].copy_(torch.from_numpy(host), non_blocking=False)
        d_t0, d_ln, d_s0 = ws.table[:NT], ws.table[NT:2 * NT], ws.table[2 * NT:2 * NT + n_seq + 1]
    else:
        d_t0, d_ln, d_s0 = table
        NT = d_t0.numel()
    v2 = v if v.dim() == 2 else v.reshape(T, -1)
    check(lib().b200_gdn_chunk_scan(ptr(q), ptr(k), ptr(v2), v2.stride(0), v_col0, ptr(g), ptr(beta), T, Hk,
                                    Hv, ptr(d_t0), ptr(d_ln), NT, ptr(d_s0), ptr(slots), ptr(has_init),
                                    n_seq, ptr(state), ptr(ws.u), ptr(ws.w), ptr(ws.qs), ptr(ws.p),
                                    ptr(ws.gc), ptr(out), stream_ptr()), "gdn_chunk_scan")
    return out


# ------------------------------------------------------------------------------ references
def ref_conv1d(x, w, conv_state, qsl, slots, has_init):
    """fp32 restatement; returns (out bf16, new_state bf16 copy)."""
    T, C = x.shape
    xf, wf = x.float(), w.float()
    out = torch.empty(T, C, dtype=torch.float32, device=x.device)
    st = conv_state.clone()
    for s in range(len(qsl) - 1):
        b, e = int(qsl[s]), int(qsl[s + 1])
        if e <= b:
            continue
        slot = int(slots[s])
        init = st[slot].float().t() if int(has_init[s]) else torch.zeros(3, C, device=x.device)  # [3, C]
        seq = torch.cat([init, xf[b:e]], 0)                       # [3 + L, C]
        acc = sum(seq[i:i + (e - b)] * wf[:, i] for i in range(4))
        out[b:e] = torch.nn.functional.silu(acc)
        st[slot] = seq[-3:].t().to(st.dtype)
    return out.to(torch.bfloat16), st


def ref_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias, eps=1e-6):
    T = xc.shape[0]
    x = xc.float()
    q = x[:, : Hk * 128].reshape(T, Hk, 128)
    k = x[:, Hk * 128: 2 * Hk * 128].reshape(T, Hk, 128)
    qn = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + eps)
    kn = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + eps)
    g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float(), threshold=20.0)
    beta = torch.sigmoid(b.float())
    return qn.to(torch.bfloat16), kn.to(torch.bfloat16), g, beta


def ref_recurrent(q, k, v, g, beta, state0):
    """Sequential gated delta rule for ONE sequence. q, k: [L, Hk, Dk]; v: [L, Hv, Dv];
    g, beta: [L, Hv]; state0 fp32 [Hv, Dv, Dk]. Returns (o fp32 [L, Hv, Dv], state)."""
    L, Hk, D = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    S = state0.clone().float()
    qf = q.float().repeat_interleave(rep, 1) * (D ** -0.5)
    kf = k.float().repeat_interleave(rep, 1)
    vf = v.float()
    o = torch.empty(L, Hv, Dv, dtype=torch.float32, device=q.device)
    for t in range(L):
        S = S * torch.exp(g[t]).view(Hv, 1, 1)
        kv = torch.einsum("hvk,hk->hv", S, kf[t])
        vn = (vf[t] - kv) * beta[t].view(Hv, 1)
        S = S + vn.unsqueeze(-1) * kf[t].unsqueeze(1)
        o[t] = torch.einsum("hvk,hk->hv", S, qf[t])
    return o, S


def ref_rmsnorm_gated(x, z, w, eps=1e-6, gate="silu", heads=1):
    T = x.shape[0]
    xf = x.float().reshape(T, heads, -1)
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
    zz = z.float().reshape(T, heads, -1)
    y = y * (torch.nn.functional.silu(zz) if gate == "silu" else torch.sigmoid(zz))
    return y.reshape(T, -1).to(torch.bfloat16)
