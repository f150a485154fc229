"""Multi-head latent attention op wrappers (absorbed tcgen05 decode, prefill helpers, batched
small-M GEMM for the per-head W_UK / W_UV products) and fp32 PyTorch restatements."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr

_declared = False
LAT, ROPE, ROW = 512, 64, 576


def _declare():
    global _declared
    if _declared:
        return
    P, I, L, F = _lib.P, _lib.I, _lib.L, _lib.F
    _lib.declare("b200_mla_decode", [P, P, I, P, L, I, I, P, I, P, I, F, I, P, P, P], I)
    _lib.declare("b200_mla_gather_latent", [P, P, I, P, P, I, P, I, I, P], I)
    _lib.declare("b200_mla_assemble_kv", [P, P, P, I, I, I, P], I)
    _lib.declare("b200_mla_pad_q", [P, L, P, I, I, P], I)
    _lib.declare("b200_mla_copy_qpe", [P, L, P, I, I, P], I)
    _lib.declare("b200_gemm_bf16_batched", [P, I, I, P, I, P, I, L, I, I, I, I, P], I)
    lib()
    _declared = True


def gemm_batched(a, a_batch_cols, w, out, out_batch_stride, M, N, K, batch):
    """out[b][m, n] = sum_k a[m, b * a_batch_cols + k] * w[b, n, k]; a, out 2-D row-strided,
    w [batch, N, K] contiguous. M is processed in slabs of 256 rows."""
    _declare()
    for m0 in range(0, M, 256):
        m = min(256, M - m0)
        check(lib().b200_gemm_bf16_batched(ptr(a[m0:]), a.stride(0), a_batch_cols, ptr(w), K, ptr(out[m0:]),
                                           out.stride(0), out_batch_stride, m, N, K, batch, stream_ptr()),
              "gemm_bf16_batched")
    return out


def mla_decode(qabs, cache, block_table, seq_lens, out, scale, block_size, splits=1, tmp=None):
    """qabs bf16 [B, H, 576]; cache bf16 [num_blocks, block_size, 576]; out bf16 [B, H, 512]."""
    _declare()
    B, H, _ = qabs.shape
    tmp_o, tmp_lse = tmp if tmp is not None else (None, None)
    if splits > 1 and tmp_o is None:
        tmp_o = torch.empty((B, H, splits, LAT), dtype=torch.float32, device=qabs.device)
        tmp_lse = torch.empty((B, H, splits), dtype=torch.float32, device=qabs.device)
    check(lib().b200_mla_decode(ptr(qabs), ptr(out), out.stride(0), ptr(cache), cache.shape[0], block_size, H,
                                ptr(block_table), block_table.stride(0), ptr(seq_lens), B, scale, splits,
                                ptr(tmp_o), ptr(tmp_lse), stream_ptr()), "mla_decode")
    return out


def gather_latent(cache, block_table, seq_lens, dense_base, block_size, dense, num_reqs, max_req_blocks):
    _declare()
    check(lib().b200_mla_gather_latent(ptr(cache), ptr(block_table), block_table.stride(0), ptr(seq_lens),
                                       ptr(dense_base), block_size, ptr(dense), num_reqs, max_req_blocks,
                                       stream_ptr()), "mla_gather_latent")


def assemble_kv(kvb, dense, cache, N, H, block_size):
    _declare()
    check(lib().b200_mla_assemble_kv(ptr(kvb), ptr(dense), ptr(cache), N, H, block_size, stream_ptr()),
          "mla_assemble_kv")


def pad_q(q, out, T, H):
    _declare()
    check(lib().b200_mla_pad_q(ptr(q), q.stride(0), ptr(out), T, H, stream_ptr()), "mla_pad_q")


def copy_qpe(q, qabs, T, H):
    _declare()
    check(lib().b200_mla_copy_qpe(ptr(q), q.stride(0), ptr(qabs), T, H, stream_ptr()), "mla_copy_qpe")


# ------------------------------------------------------------------------------ references
def ref_mla_attention(q, cache, block_table, seq_lens, query_start, w_kvb, H, scale, block_size):
    """Non-absorbed restatement over the latent cache. q: [T, H, 192] (rope applied);
    cache: [nb, bs, 576]; w_kvb: [H * 256, 512] (per head [k_nope 128 | v 128]).
    Returns [T, H, 128] fp32."""
    T = q.shape[0]
    out = torch.zeros(T, H, 128, dtype=torch.float32, device=q.device)
    wk = w_kvb.float().view(H, 256, LAT)
    flat = cache.reshape(-1, ROW).float()
    R = seq_lens.numel()
    for r in range(R):
        b, e = int(query_start[r]), int(query_start[r + 1])
        L = int(seq_lens[r])
        if e <= b:
            continue
        pos = torch.arange(L, device=q.device)
        rows = block_table[r][(pos // block_size).long()].long() * block_size + pos % block_size
        lat = flat[rows]                                   # [L, 576]
        kv = torch.einsum("lc,hdc->lhd", lat[:, :LAT], wk).to(torch.bfloat16).float()   # [L, H, 256]
        k = torch.cat([kv[:, :, :128], lat[:, None, LAT:].expand(L, H, ROPE)], -1)      # [L, H, 192]
        v = kv[:, :, 128:]
        qq = q[b:e].float()
        s = torch.einsum("thd,lhd->htl", qq, k) * scale
        qpos = L - (e - b) + torch.arange(e - b, device=q.device)
        mask = pos[None, :] > qpos[:, None]
        s = s.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(s, -1)
        out[b:e] = torch.einsum("htl,lhd->thd", p, v)
    return out


def ref_mla_decode_absorbed(qabs, cache, block_table, seq_lens, scale, block_size):
    B, H, _ = qabs.shape
    flat = cache.reshape(-1, ROW).float()
    out = torch.zeros(B, H, LAT, dtype=torch.float32, device=qabs.device)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        pos = torch.arange(L, device=qabs.device)
        rows = block_table[b][(pos // block_size).long()].long() * block_size + pos % block_size
        lat = flat[rows]
        s = (qabs[b].float() @ lat.t()) * scale
        out[b] = torch.softmax(s, -1) @ lat[:, :LAT]
    return out
