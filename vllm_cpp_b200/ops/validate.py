"""One validation layer in front of the kernel launchers: every op lists its argument contract as
named rules over the tensors it is given; ``validate(op, **args)`` raises :class:`OpArgumentError`
naming the op, the rule that failed and the offending shapes before anything is launched. The C
launchers keep their own checks (they return -1); this layer is what turns a bad call into a
message a caller can act on, the same for every op.

Reference: the ``Validate*`` helpers of ``include/vt/ops.h`` / ``src/vt/ops.cpp`` (uniform
shape / dtype / layout errors in front of every backend).
"""
from __future__ import annotations

import torch


class OpArgumentError(ValueError):
    def __init__(self, op: str, rule: str, detail: str):
        super().__init__(f"{op}: {rule} ({detail})")
        self.op, self.rule = op, rule


def _desc(**t) -> str:
    parts = []
    for k, v in t.items():
        if isinstance(v, torch.Tensor):
            parts.append(f"{k}={tuple(v.shape)} {str(v.dtype).replace('torch.', '')} stride={tuple(v.stride())}")
        elif v is not None:
            parts.append(f"{k}={v}")
    return ", ".join(parts)


def _rows16(t: torch.Tensor) -> bool:
    """Row-contiguous with 16-byte aligned rows: what a TMA tensor map needs."""
    return t.stride(-1) == 1 and (t.dim() < 2 or (t.stride(-2) * t.element_size()) % 16 == 0) \
        and t.data_ptr() % 16 == 0


BF16 = torch.bfloat16

RULES: dict[str, list] = {
    "gemm": [
        ("a and w are bf16", lambda a, w, **_: a.dtype == BF16 and w.dtype == BF16),
        ("a is [M, K] and w is [N, K] with the same K", lambda a, w, **_: a.dim() == 2 and w.dim() == 2
         and a.shape[1] == w.shape[1]),
        ("rows are contiguous and 16-byte aligned", lambda a, w, **_: _rows16(a) and _rows16(w)),
        ("out is [M, N], bf16 or fp32, row-contiguous", lambda a, w, out=None, **_: out is None or (
            out.shape == (a.shape[0], w.shape[0]) and out.dtype in (BF16, torch.float32) and out.stride(1) == 1)),
        ("bias is bf16 [N]", lambda w, bias=None, **_: bias is None or (bias.dtype == BF16 and bias.numel() == w.shape[0])),
        ("residual is bf16 [M, N]", lambda a, w, residual=None, **_: residual is None or (
            residual.dtype == BF16 and residual.shape == (a.shape[0], w.shape[0]))),
    ],
    "gemm_nvfp4": [
        ("packed operands are uint8 [rows, K/2] with the same K", lambda aq, wq, **_: aq.dtype == torch.uint8
         and wq.dtype == torch.uint8 and aq.dim() == 2 and wq.dim() == 2 and aq.shape[1] == wq.shape[1]),
        ("K is a multiple of 256", lambda aq, **_: (aq.shape[1] * 2) % 256 == 0),
        ("N is a multiple of 8", lambda wq, **_: wq.shape[0] % 8 == 0),
        ("scale chunks cover the padded rows", lambda aq, wq, sfa, sfw, **_: sfa.numel() >= -(-aq.shape[0] // 128) * 128
         * (aq.shape[1] // 8) and sfw.numel() >= -(-wq.shape[0] // 128) * 128 * (wq.shape[1] // 8)),
        ("global scales are fp32 scalars on the device", lambda g_a, g_w, aq, **_: g_a.dtype == torch.float32
         and g_w.dtype == torch.float32 and g_a.device == aq.device and g_w.device == aq.device),
    ],
    "rmsnorm": [
        ("x is [T, H] bf16, row-contiguous", lambda x, **_: x.dim() == 2 and x.dtype == BF16 and x.stride(1) == 1),
        ("weight has H elements", lambda x, weight, **_: weight.numel() == x.shape[1]),
        ("residual is contiguous [T, H]", lambda x, residual=None, **_: residual is None or (
            residual.is_contiguous() and residual.shape == x.shape)),
    ],
    "attn_decode": [
        ("q is [B, Hq * D] bf16, row-contiguous", lambda q, num_q_heads, head_dim, **_: q.dim() == 2
         and q.dtype == BF16 and q.shape[1] == num_q_heads * head_dim and q.stride(1) == 1),
        ("kv_cache is [blocks, 2, block_size, Hkv, D]", lambda kv_cache, num_kv_heads, head_dim, block_size, **_:
         kv_cache.dim() == 5 and tuple(kv_cache.shape[1:]) == (2, block_size, num_kv_heads, head_dim)),
        ("Hq is a multiple of Hkv", lambda num_q_heads, num_kv_heads, **_: num_q_heads % num_kv_heads == 0),
        ("head_dim is 64, 128 or 256", lambda head_dim, **_: head_dim in (64, 128, 256)),
        ("block_table and seq_lens are int32 with B rows", lambda q, block_table, seq_lens, **_:
         block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32 and block_table.shape[0] >= q.shape[0]
         and seq_lens.numel() >= q.shape[0]),
    ],
    "attn_prefill": [
        ("q is [T, Hq * D] bf16, row-contiguous", lambda q, num_q_heads, head_dim, **_: q.dim() == 2
         and q.dtype == BF16 and q.shape[1] == num_q_heads * head_dim and q.stride(1) == 1),
        ("kv_cache is [blocks, 2, block_size, Hkv, D]", lambda kv_cache, num_kv_heads, head_dim, block_size, **_:
         kv_cache.dim() == 5 and tuple(kv_cache.shape[1:]) == (2, block_size, num_kv_heads, head_dim)),
        ("head_dim is 64, 128 or 256", lambda head_dim, **_: head_dim in (64, 128, 256)),
        ("page size divides or is a multiple of 64", lambda block_size, **_: block_size >= 8 and block_size % 8 == 0
         and (64 % block_size == 0 or block_size % 64 == 0)),
        ("tile table entries are int32", lambda tile_req, tile_q0, **_: tile_req.dtype == torch.int32
         and tile_q0.dtype == torch.int32 and tile_req.numel() == tile_q0.numel()),
    ],
    "moe_grouped_gemm": [
        ("w is [E, N, K] bf16", lambda w, **_: w.dim() == 3 and w.dtype == BF16),
        ("xs is [rows, K] bf16 with the weights' K", lambda xs, w, **_: xs.dim() == 2 and xs.dtype == BF16
         and xs.shape[1] == w.shape[2]),
        ("N and K are multiples of 8", lambda w, **_: w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0),
    ],
}


def validate(op: str, **args) -> None:
    """Raises :class:`OpArgumentError` for the first rule of ``op`` the arguments break."""
    for rule, ok in RULES[op]:
        try:
            good = bool(ok(**args))
        except (KeyError, TypeError, IndexError, AttributeError) as e:
            raise OpArgumentError(op, rule, f"could not be evaluated: {e}; {_desc(**args)}") from None
        if not good:
            raise OpArgumentError(op, rule, _desc(**args))
