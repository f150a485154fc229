"""Mixture-of-experts op wrappers (router top-k, expert sort, grouped GEMM, combine) and their
fp32 PyTorch restatements."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr


class B200MoeScatter(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
                ("peer_recv", ctypes.c_void_p * 8), ("peer_rs_flags", ctypes.c_void_p * 8),
                ("recv_parity_stride", ctypes.c_longlong), ("rs_flag_parity_stride", ctypes.c_int),
                ("op_counter", ctypes.c_void_p)]


_declared = False


def _declare():
    global _declared
    if _declared:
        return
    P, I, F = _lib.P, _lib.I, _lib.F
    _lib.declare("b200_moe_router_topk", [P, I, I, I, I, I, I, P, I, I, F, P, P, P], I)
    _lib.declare("b200_moe_sort", [P, I, I, I, I, P, P, P, P, P, P, I, P], I)
    _lib.declare("b200_moe_gather", [P, I, P, P, I, P, I, I, P], I)
    _lib.declare("b200_moe_grouped_gemm", [P, I, P, I, I, I, P, P, P, P, P, I, P], I)
    _lib.declare("b200_moe_grouped_gemm_gated", [P, I, P, I, I, I, P, P, P, P, P, I, I, P], I)
    _lib.declare("b200_moe_combine", [P, P, P, I, I, I, P, P, P, ctypes.POINTER(B200MoeScatter), P], I)
    _lib.declare("b200_shared_gate", [P, I, P, I, I, P, P], I)
    lib()
    _declared = True


def router_topk(logits: torch.Tensor, k: int, *, renorm: bool = True, scoring: str = "softmax",
                e_bias: torch.Tensor | None = None, n_group: int = 1, topk_group: int = 1,
                routed_scale: float = 1.0):
    """logits: fp32 [T, E] -> (ids int32 [T, k], weights fp32 [T, k])."""
    _declare()
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    check(lib().b200_moe_router_topk(ptr(logits), logits.stride(0), T, E, k, int(renorm),
                                     0 if scoring == "softmax" else 1, ptr(e_bias), n_group,
                                     topk_group, routed_scale, ptr(ids), ptr(w), stream_ptr()),
          "moe_router_topk")
    return ids, w


class MoeWorkspace:
    """Persistent buffers of one MoE layer shape (sized for ``max_tokens``)."""

    def __init__(self, device, max_tokens: int, k: int, num_local_experts: int, hidden: int,
                 inter: int):
        P = max_tokens * k
        E = num_local_experts
        self.max_pairs = P
        self.max_chunks = E + (P + 255) // 256
        i32 = dict(dtype=torch.int32, device=device)
        self.meta = torch.zeros(3 * E + 2, **i32)
        self.sorted_token = torch.zeros(P, **i32)
        self.pair_pos = torch.zeros(P, **i32)
        self.chunk_expert = torch.zeros(self.max_chunks, **i32)
        self.chunk_row0 = torch.zeros(self.max_chunks, **i32)
        self.chunk_n = torch.zeros(self.max_chunks, **i32)
        bf = dict(dtype=torch.bfloat16, device=device)
        self.xs = torch.zeros((P + 256, hidden), **bf)
        self.gu = torch.zeros((P + 256, 2 * inter), **bf)
        self.act = torch.zeros((P + 256, inter), **bf)
        self.y = torch.zeros((P + 256, hidden), **bf)


def moe_sort(topk_ids: torch.Tensor, e0: int, e1: int, ws: MoeWorkspace):
    _declare()
    T, k = topk_ids.shape
    check(lib().b200_moe_sort(ptr(topk_ids), T, k, e0, e1, ptr(ws.meta), ptr(ws.sorted_token),
                              ptr(ws.pair_pos), ptr(ws.chunk_expert), ptr(ws.chunk_row0),
                              ptr(ws.chunk_n), ws.max_chunks, stream_ptr()), "moe_sort")


def moe_gather(x: torch.Tensor, ws: MoeWorkspace, num_local_experts: int, max_rows: int):
    _declare()
    check(lib().b200_moe_gather(ptr(x), x.stride(0), ptr(ws.sorted_token), ptr(ws.meta),
                                num_local_experts, ptr(ws.xs), x.shape[1], max_rows,
                                stream_ptr()), "moe_gather")


def grouped_gemm(xs: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ws: MoeWorkspace,
                 max_rows: int, max_chunks: int | None = None):
    """out[pos] = xs[pos] @ w[expert(pos)]^T ; w: [E, N, K]."""
    _declare()
    E, N, K = w.shape
    check(lib().b200_moe_grouped_gemm(ptr(xs), max_rows, ptr(w), E, N, K, ptr(out),
                                      ptr(ws.chunk_expert), ptr(ws.chunk_row0), ptr(ws.chunk_n),
                                      ptr(ws.meta), max_chunks or ws.max_chunks, stream_ptr()),
          "moe_grouped_gemm")
    return out


def grouped_gemm_gated(xs: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, ws: MoeWorkspace,
                       max_rows: int, max_chunks: int | None = None, kind: int = 0):
    """out[pos] = act(xs[pos] @ w_gate^T) * (xs[pos] @ w_up^T); ``w_gate_up``: [E, 2 I, K] with rows
    [gate | up]. One kernel: both halves accumulate in TMEM and the activation runs in the
    epilogue, so the merged projection is never written."""
    _declare()
    E, N, K = w_gate_up.shape
    check(lib().b200_moe_grouped_gemm_gated(ptr(xs), max_rows, ptr(w_gate_up), E, N, K, ptr(out),
                                            ptr(ws.chunk_expert), ptr(ws.chunk_row0), ptr(ws.chunk_n),
                                            ptr(ws.meta), max_chunks or ws.max_chunks, kind, stream_ptr()),
          "moe_grouped_gemm_gated")
    return out


def combine(y: torch.Tensor, ws: MoeWorkspace, topk_w: torch.Tensor, out: torch.Tensor | None,
            shared: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None,
            scatter: B200MoeScatter | None = None):
    _declare()
    T, k = topk_w.shape
    H = y.shape[1]
    check(lib().b200_moe_combine(ptr(y), ptr(ws.pair_pos), ptr(topk_w), T, k, H, ptr(shared),
                                 ptr(shared_gate), ptr(out),
                                 ctypes.byref(scatter) if scatter is not None else None,
                                 stream_ptr()), "moe_combine")
    return out


def shared_gate(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    _declare()
    T, H = x.shape
    out = torch.empty(T, dtype=torch.float32, device=x.device)
    check(lib().b200_shared_gate(ptr(x), x.stride(0), ptr(w), T, H, ptr(out), stream_ptr()),
          "shared_gate")
    return out


# ------------------------------------------------------------------------------ references
def ref_router_topk(logits, k, renorm=True, scoring="softmax", e_bias=None, n_group=1,
                    topk_group=1, routed_scale=1.0):
    x = logits.float()
    score = torch.softmax(x, -1) if scoring == "softmax" else torch.sigmoid(x)
    sel = score + (e_bias.float() if e_bias is not None else 0.0)
    T, E = x.shape
    if n_group > 1 and topk_group < n_group:
        g = sel.view(T, n_group, E // n_group)
        gs = g.topk(2, dim=-1).values.sum(-1) if e_bias is not None else g.max(-1).values
        keep = torch.zeros_like(gs, dtype=torch.bool)
        keep.scatter_(1, gs.topk(topk_group, dim=-1).indices, True)
        sel = sel.masked_fill(~keep[:, :, None].expand_as(g).reshape(T, E), float("-inf"))
    ids = torch.empty((T, k), dtype=torch.int64, device=x.device)
    s = sel.clone()
    for j in range(k):
        m = s.max(-1, keepdim=True).values
        first = ((s == m).float().cumsum(-1) == 1) & (s == m)
        idx = first.float().argmax(-1)
        ids[:, j] = idx
        s.scatter_(1, idx[:, None], float("-inf"))
    w = score.gather(1, ids)
    if renorm:
        d = w.sum(-1, keepdim=True)
        w = w / torch.where(d > 0, d, torch.ones_like(d))
    return ids.int(), w * routed_scale


def ref_moe_block(x, topk_ids, topk_w, w_gate_up, w_down, e0=0):
    """x [T,H] bf16; w_gate_up [E, 2I, H]; w_down [E, H, I]; returns fp32-accumulated bf16 [T,H]."""
    T, H = x.shape
    E, I2, _ = w_gate_up.shape
    inter = I2 // 2
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    for e in range(E):
        for j in range(topk_ids.shape[1]):
            sel = (topk_ids[:, j].long() == e + e0).nonzero().flatten()
            if sel.numel() == 0:
                continue
            gu = (x[sel].float() @ w_gate_up[e].float().t()).to(torch.bfloat16)
            a = (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(torch.bfloat16)
            y = (a.float() @ w_down[e].float().t()).to(torch.bfloat16)
            out[sel] += topk_w[sel, j, None] * y.float()
    return out.to(torch.bfloat16)
