"""Plain PyTorch fp32 restatements of every kernel in ``vllm_cpp_b200.ops``.

They are the oracle for the numerics tests (CPU or GPU tensors) and the arithmetic used by
the CPU model path; nothing here is on the GPU serving path.
"""
from __future__ import annotations

import math

import torch


def gemm(a, w, bias=None, residual=None, out_dtype=torch.bfloat16):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype)


def rmsnorm(x, weight, eps, residual=None, gemma=False):
    """Returns (out, new_residual). bf16 residual add is rounded to the storage dtype first."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float() + (1.0 if gemma else 0.0)
    return (xf * inv * w).to(x.dtype), x


def layernorm(x, weight, bias, eps):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def act_and_mul(x, kind=0):
    inter = x.shape[-1] // 2
    g, u = x[..., :inter].float(), x[..., inter:].float()
    if kind == 0:
        a = g * torch.sigmoid(g)
    elif kind == 1:
        a = torch.nn.functional.gelu(g, approximate="tanh")
    else:
        a = torch.nn.functional.gelu(g)
    return (a * u).to(x.dtype)


def rope_inv_freq(rot_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))


def rope_table(inv_freq, max_pos, mscale=1.0):
    pos = torch.arange(max_pos, dtype=torch.float64, device=inv_freq.device)
    ph = pos[:, None] * inv_freq.to(torch.float64)[None, :]
    return torch.cat([ph.cos() * mscale, ph.sin() * mscale], dim=-1).float()


def apply_rope(x, cos, sin, rot, neox):
    """x: [T, H, D] float; cos/sin: [T, rot/2]."""
    xr, xp = x[..., :rot], x[..., rot:]
    c, s = cos[:, None, :], sin[:, None, :]
    if neox:
        x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
        o = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
    return torch.cat([o, xp], dim=-1)


def rope_kv(qkv, positions, cos_sin, num_q_heads, num_kv_heads, head_dim, rot_dim=None,
            neox=True, q_norm=None, k_norm=None, eps=1e-6, gemma=False):
    """Returns (q, k, v) as [T, H, D] tensors in the input dtype, after optional per-head
    RMSNorm and rotary embedding."""
    T = qkv.shape[0]
    D = head_dim
    rot = rot_dim or D
    q = qkv[:, : num_q_heads * D].reshape(T, num_q_heads, D)
    k = qkv[:, num_q_heads * D: (num_q_heads + num_kv_heads) * D].reshape(T, num_kv_heads, D)
    v = qkv[:, (num_q_heads + num_kv_heads) * D:].reshape(T, num_kv_heads, D)

    def norm(x, w):
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return (xf * inv * (w.float() + (1.0 if gemma else 0.0))).to(x.dtype)

    if q_norm is not None:
        q = norm(q, q_norm)
    if k_norm is not None:
        k = norm(k, k_norm)
    if cos_sin is not None:
        cs = cos_sin[positions]
        cos, sin = cs[:, : rot // 2], cs[:, rot // 2:]
        q = apply_rope(q.float(), cos, sin, rot, neox).to(qkv.dtype)
        k = apply_rope(k.float(), cos, sin, rot, neox).to(qkv.dtype)
    return q, k, v


def write_kv_cache(kv_cache, k, v, slot_mapping, block_size):
    """kv_cache: [num_blocks, 2, block_size, Hkv, D]."""
    for t, slot in enumerate(slot_mapping.tolist()):
        if slot < 0:
            continue
        b, o = divmod(slot, block_size)
        kv_cache[b, 0, o] = k[t]
        kv_cache[b, 1, o] = v[t]


def paged_attention(q, kv_cache, block_table, seq_lens, q_start, num_q_heads, num_kv_heads,
                    head_dim, block_size, scale, softcap=0.0, window=0, causal=True,
                    return_lse=False):
    """Varlen paged attention oracle. q: [T, Hq*D]; query row t of request r sits at position
    ``seq_len_r - q_len_r + (t - q_start_r)`` (bottom-right aligned causal mask)."""
    T = q.shape[0]
    D = head_dim
    G = num_q_heads // num_kv_heads
    out = torch.zeros((T, num_q_heads * D), dtype=torch.float32, device=q.device)
    lse = torch.full((T, num_q_heads), -math.inf, dtype=torch.float32, device=q.device)
    qs = q_start.tolist()
    for r, sl in enumerate(seq_lens.tolist()):
        t0, t1 = qs[r], qs[r + 1]
        ql = t1 - t0
        if ql <= 0 or sl <= 0:
            continue
        nb = (sl + block_size - 1) // block_size
        blocks = block_table[r, :nb].long()
        kk = kv_cache[blocks, 0].reshape(nb * block_size, num_kv_heads, D)[:sl].float()
        vv = kv_cache[blocks, 1].reshape(nb * block_size, num_kv_heads, D)[:sl].float()
        qq = q[t0:t1].reshape(ql, num_q_heads, D).float()
        kk = kk.repeat_interleave(G, dim=1)
        vv = vv.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = (sl - ql) + torch.arange(ql, device=q.device)
        kpos = torch.arange(sl, device=q.device)
        mask = torch.ones((ql, sl), dtype=torch.bool, device=q.device)
        if causal:
            mask &= kpos[None, :] <= qpos[:, None]
        if window > 0:
            mask &= kpos[None, :] > qpos[:, None] - window
        elif window < 0:        # chunked-local attention: a query sees the keys of its own chunk
            mask &= kpos[None, :] >= (qpos[:, None] // -window) * -window
        s = s.masked_fill(~mask[None], -math.inf)
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None])
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        out[t0:t1] = o.reshape(ql, num_q_heads * D)
        lse[t0:t1] = l.t()
    if return_lse:
        return out.to(q.dtype), lse
    return out.to(q.dtype)


def build_prefill_tiles(q_lens, tile=128):
    req, q0 = [], []
    for r, n in enumerate(q_lens):
        for s in range(0, n, tile):
            req.append(r)
            q0.append(s)
    return req, q0


# ------------------------------------------------------------------------------ sampling
def top_k_top_p(logits, top_k, top_p):
    """Sort-based keep-set (the vLLM rule): keep the k largest, then the smallest prefix of
    the descending-probability order whose mass reaches p; ties at the cut are kept."""
    out = logits.clone()
    n, V = logits.shape
    for r in range(n):
        row = out[r]
        k = int(top_k[r]) if top_k is not None else 0
        if 0 < k < V:
            kth = torch.topk(row, k).values[-1]
            row[row < kth] = -math.inf
        p = float(top_p[r]) if top_p is not None else 1.0
        if p < 1.0:
            probs = torch.softmax(row, dim=-1)
            sp, si = torch.sort(probs, descending=True)
            cs = torch.cumsum(sp, dim=-1)
            # first index where cumulative mass >= p
            cut = int(torch.searchsorted(cs, torch.tensor(p * float(cs[-1]), dtype=cs.dtype,
                                                          device=cs.device)))
            cut = min(cut, V - 1)
            thr = row[si[cut]]
            row[row < thr] = -math.inf
    return out


def splitmix64(z: int) -> int:
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def race_sample(probs_row, seed: int, step: int) -> int:
    """Exponential-race draw matching the kernel's counter RNG bit for bit (slow, tests only)."""
    m = (1 << 64) - 1
    best, best_i = -1.0, 0
    pr = probs_row.tolist()
    for i, p in enumerate(pr):
        if p <= 0:
            continue
        z = splitmix64(seed ^ splitmix64((step * 0x100000001B3 + i) & m))
        u = ((z >> 11) + 0.5) / 9007199254740992.0
        e = torch.tensor(-math.log(u), dtype=torch.float64).float().item()
        key = torch.tensor(p, dtype=torch.float32) / torch.tensor(e, dtype=torch.float32)
        key = key.item()
        if key > best:
            best, best_i = key, i
    return best_i
