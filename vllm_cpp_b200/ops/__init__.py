"""Tensor-level entry points of the sm_100a kernel library.

Every function takes CUDA ``torch.Tensor`` arguments, launches on the current stream and
returns without synchronising. There is no eager-PyTorch fallback on this path: a missing
library or a rejected shape raises. Plain fp32 references of the same ops live in
``vllm_cpp_b200.ops.reference`` and are what the numerics tests compare against.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr
from .validate import OpArgumentError, validate  # noqa: F401

ACT_SILU, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
EW_ADD, EW_RELU, EW_MUL_SCALAR, EW_SOFTCAP, EW_SIGMOID_MUL, EW_MUL = 0, 1, 2, 3, 4, 5

_inited_devices: set[int] = set()


def init_device(device: torch.device) -> None:
    """Per-device set-up of the kernel library (stream-K scratch), once, before any capture."""
    if device.type != "cuda":
        return
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _inited_devices:
        return
    with torch.cuda.device(idx):
        check(lib().b200_init_device(), "init_device")
    _inited_devices.add(idx)


_workspaces: dict[tuple[int, str], torch.Tensor] = {}
_retired_workspaces: list[torch.Tensor] = []


def workspace(device: torch.device, nbytes: int, tag: str = "gemm") -> torch.Tensor:
    """Persistent per-device scratch. Never freed: a CUDA graph captured while a smaller buffer was
    current keeps that buffer's address, so a buffer that is outgrown is retired, not released
    (releasing it would hand the captured address to some other tensor)."""
    key = (device.index or 0, tag)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        if w is None:
            init_device(device)
        else:
            _retired_workspaces.append(w)
        w = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = w
    return w


GEMM_WS_BYTES = 64 << 20


def gemm(a: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
         out_dtype: torch.dtype = torch.bfloat16, force_path: int = 0,
         const_w: bool = False) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ w[N,K]^T (+ bias) (+ residual)``; bf16 inputs, fp32 accumulate.
    ``const_w``: ``w`` is a model weight that no kernel in the stream writes, so the GEMM may
    fetch its first tiles while the previous kernel is still running."""
    if not (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.shape[1] == w.shape[1] and a.stride(1) == 1 and w.stride(1) == 1
            and (out is None or (out.stride(1) == 1 and out.shape == (a.shape[0], w.shape[0])))):
        validate("gemm", a=a, w=w, out=out, bias=bias, residual=residual)   # names the broken rule
        raise OpArgumentError("gemm", "argument contract", "see ops.validate.RULES['gemm']")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    ws = workspace(a.device, GEMM_WS_BYTES)
    rc = lib().b200_gemm_bf16(
        ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out.stride(0),
        1 if out.dtype == torch.float32 else 0, ptr(bias), ptr(residual),
        residual.stride(0) if residual is not None else 0, M, N, K, ptr(ws), ws.numel(),
        force_path | (0x100 if const_w else 0), stream_ptr())
    check(rc, f"gemm M={M} N={N} K={K}")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, *,
            residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
            gemma: bool = False) -> torch.Tensor:
    """``out = rmsnorm(x) * w``; with ``residual``: ``residual += x`` first (in place) and the
    norm is taken over the updated residual."""
    if x.dim() != 2 or weight.numel() != x.shape[1] or x.stride(1) != 1:
        validate("rmsnorm", x=x, weight=weight, residual=residual)
    T, H = x.shape
    if out is None:
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    if residual is not None:
        assert residual.is_contiguous()
    check(lib().b200_rmsnorm(ptr(x), x.stride(0), ptr(residual), ptr(weight), ptr(out),
                             out.stride(0), T, H, eps, int(gemma), stream_ptr()), "rmsnorm")
    return out


def layernorm(x, weight, bias, eps, out=None):
    T, H = x.shape
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    check(lib().b200_layernorm(ptr(x), ptr(weight), ptr(bias), ptr(out), T, H, eps, stream_ptr()),
          "layernorm")
    return out


def act_and_mul(x: torch.Tensor, kind: int = ACT_SILU, out: torch.Tensor | None = None,
                interleaved: bool = False):
    """``x = [gate | up]`` along the last dim -> ``act(gate) * up``. ``interleaved``: the columns
    come in blocks of ``[128 gate | 128 up]`` (see :func:`interleave_gate_up`)."""
    T, two_i = x.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=x.dtype, device=x.device)
    flags = kind | (0x100 if interleaved else 0)
    check(lib().b200_act_and_mul(ptr(x), x.stride(0), ptr(out), T, inter, flags, stream_ptr()),
          "act_and_mul")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Weight rows in blocks of ``[128 gate | 128 up]``: every 256-column tile of the merged
    projection then holds both halves of 128 outputs, which lets the GEMM epilogue apply the
    gated activation. Needs the intermediate size to be a multiple of 128."""
    I, H = gate.shape
    assert up.shape == gate.shape and I % 128 == 0
    return torch.stack([gate.reshape(I // 128, 128, H), up.reshape(I // 128, 128, H)], 1).reshape(2 * I, H)


def gemm_gated(a: torch.Tensor, w_il: torch.Tensor, kind: int = ACT_SILU, *,
               out: torch.Tensor | None = None, scratch: torch.Tensor | None = None,
               force_path: int = 0) -> torch.Tensor:
    """``act(a @ w_gate^T) * (a @ w_up^T)`` with ``w_il`` from :func:`interleave_gate_up`.
    Above 128 rows the activation runs in the GEMM epilogue (one kernel, the merged
    projection never reaches memory); below, the small-M GEMM writes the interleaved
    projection to ``scratch`` and the activation kernel reads it."""
    M, K = a.shape
    N = w_il.shape[0]
    assert a.dtype == torch.bfloat16 and w_il.dtype == torch.bfloat16 and N % 256 == 0
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    if M > 128:
        check(lib().b200_gemm_bf16_gated(ptr(a), a.stride(0), ptr(w_il), w_il.stride(0), ptr(out),
                                         out.stride(0), M, N, K, kind, force_path, stream_ptr()),
              f"gemm_gated M={M} N={N} K={K}")
        return out
    if scratch is None:
        scratch = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    gemm(a, w_il, out=scratch, const_w=True)      # w_il is a model weight by construction
    return act_and_mul(scratch, kind, out, interleaved=True)


def silu_and_mul(x, out=None):
    return act_and_mul(x, ACT_SILU, out)


def gelu_tanh_and_mul(x, out=None):
    return act_and_mul(x, ACT_GELU_TANH, out)


def eltwise(a, b, kind, scalar=0.0, out=None):
    a = a.contiguous()
    if b is not None:
        b = b.contiguous()
    if out is None:
        out = torch.empty_like(a)
    check(lib().b200_eltwise(ptr(a), ptr(b), ptr(out), a.numel(), kind, float(scalar),
                             stream_ptr()), "eltwise")
    return out


def add(a, b, out=None):
    return eltwise(a, b, EW_ADD, out=out)


def relu(a, out=None):
    return eltwise(a, None, EW_RELU, out=out)


def mul_scalar(a, s, out=None):
    return eltwise(a, None, EW_MUL_SCALAR, s, out=out)


def softcap(a, cap, out=None):
    return eltwise(a, None, EW_SOFTCAP, cap, out=out)


def sigmoid_mul(a, gate, out=None):
    """``a * sigmoid(gate)`` (attention output gate)."""
    return eltwise(a, gate, EW_SIGMOID_MUL, out=out)


def cast_f32(a):
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    check(lib().b200_cast_bf16_f32(ptr(a.contiguous()), ptr(out), a.numel(), stream_ptr()), "cast")
    return out


def cast_bf16(a):
    out = torch.empty(a.shape, dtype=torch.bfloat16, device=a.device)
    check(lib().b200_cast_f32_bf16(ptr(a.contiguous()), ptr(out), a.numel(), stream_ptr()), "cast")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, *, out=None, vocab_start: int = 0,
              vocab_total: int | None = None, scale: float = 1.0):
    assert ids.dtype == torch.int64
    T = ids.numel()
    rows, H = table.shape
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    check(lib().b200_embedding(ptr(ids), ptr(table), ptr(out), T, H, vocab_start, rows,
                               vocab_total if vocab_total is not None else vocab_start + rows,
                               scale, stream_ptr()), "embedding")
    return out


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out=None):
    assert idx.dtype == torch.int32 and x.is_contiguous()
    n = idx.numel()
    if out is None:
        out = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib().b200_gather_rows(ptr(x), ptr(idx), ptr(out), n, x.shape[0],
                                 x.shape[1] * x.element_size(), stream_ptr()), "gather_rows")
    return out


def rope_table(inv_freq: torch.Tensor, max_pos: int, mscale: float = 1.0) -> torch.Tensor:
    """``[max_pos, 2*half]`` fp32 table ``[cos | sin]`` from fp64 inverse frequencies."""
    inv = inv_freq.to(dtype=torch.float64).contiguous()
    half = inv.numel()
    out = torch.empty((max_pos, 2 * half), dtype=torch.float32, device=inv.device)
    check(lib().b200_rope_table(ptr(inv), ptr(out), max_pos, half, mscale, stream_ptr()),
          "rope_table")
    return out


def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor | None, *,
            num_q_heads: int, num_kv_heads: int, head_dim: int, rot_dim: int | None = None,
            neox: bool = True, q_norm: torch.Tensor | None = None,
            k_norm: torch.Tensor | None = None, eps: float = 1e-6, gemma: bool = False,
            slot_mapping: torch.Tensor | None = None, kv_cache: torch.Tensor | None = None,
            block_size: int = 16, q_out: torch.Tensor | None = None,
            q_head_stride: int | None = None, offsets: tuple[int, int, int] | None = None):
    """Fused per-head qk-RMSNorm + RoPE + KV-cache write over merged ``[T, q|k|v]`` rows.
    q is rotated in place (or into ``q_out``); rotated k and raw v go to ``kv_cache``."""
    T = qkv.shape[0]
    D = head_dim
    if offsets is None:
        offsets = (0, num_q_heads * D, (num_q_heads + num_kv_heads) * D)
    rot = rot_dim if rot_dim is not None else D
    check(lib().b200_rope_kv(
        ptr(qkv), qkv.stride(0), offsets[0], offsets[1], offsets[2],
        q_head_stride if q_head_stride is not None else D, num_q_heads, num_kv_heads, D, rot,
        ptr(positions), ptr(cos_sin), ptr(q_norm), ptr(k_norm), eps, int(gemma), int(neox),
        ptr(slot_mapping), ptr(kv_cache), block_size, ptr(q_out), T, stream_ptr()), "rope_kv")


def reshape_and_cache(k, v, slot_mapping, kv_cache, block_size, num_kv_heads, head_dim):
    T = k.shape[0]
    check(lib().b200_reshape_and_cache(ptr(k), k.stride(0), ptr(v), v.stride(0), ptr(slot_mapping),
                                       ptr(kv_cache), block_size, num_kv_heads, head_dim, T,
                                       stream_ptr()), "reshape_and_cache")


def concat_and_cache_mla(kv_c, k_pe, slot_mapping, cache):
    T = kv_c.shape[0]
    check(lib().b200_concat_and_cache_mla(ptr(kv_c), kv_c.stride(0), ptr(k_pe), k_pe.stride(0),
                                          ptr(slot_mapping), ptr(cache), kv_c.shape[1],
                                          k_pe.shape[1], T, stream_ptr()), "concat_and_cache_mla")


def attn_prefill(q: torch.Tensor, kv_cache: torch.Tensor, *, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, q_start: torch.Tensor, tile_req: torch.Tensor,
                 tile_q0: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                 block_size: int, scale: float, out: torch.Tensor | None = None,
                 lse: torch.Tensor | None = None, softcap: float = 0.0, window: int = 0,
                 causal: bool = True):
    """Varlen paged prefill attention. ``q``: [T, Hq*D] (row stride free); K/V are read from
    the paged cache only. ``tile_req/tile_q0`` list the 128-row query tiles (host built)."""
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, num_q_heads * head_dim), dtype=q.dtype, device=q.device)
    num_blocks = kv_cache.shape[0]
    check(lib().b200_attn_prefill(
        ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(lse), ptr(kv_cache), num_blocks,
        block_size, num_q_heads, num_kv_heads, head_dim, ptr(block_table), block_table.stride(0),
        ptr(seq_lens), ptr(q_start), ptr(tile_req), ptr(tile_q0), tile_req.numel(), T, scale,
        softcap, window, int(causal), stream_ptr()), "attn_prefill")
    return out


def _decode_uses_tc(head_dim: int, group: int, block_size: int) -> bool:
    """Whether the first choice of the attention backend registry, the tcgen05 swapped-operand decode
    kernel (head_dim 128 and 256, GQA groups up to 16, page sizes that tile 128 tokens), serves this
    shape; everything else takes the CUDA-core kernel."""
    from ..models.attention_backends import select
    b = select("decode", "paged", head_dim=head_dim, group=group, block_size=block_size)
    return b is not None and b.name == "tcgen05-decode"


def attn_decode_splits(batch, num_kv_heads, group, head_dim, max_seq_len,
                       block_size: int = 16) -> int:
    if _decode_uses_tc(head_dim, group, block_size):
        # two CTAs fit on an SM (one at head_dim 256): split only while every split still gets a
        # slot in the first wave (a second, ragged wave plus the merge kernel costs more than it gains)
        ctas = max(1, batch * num_kv_heads)
        want = ((2 if head_dim == 128 else 1) * num_sms()) // ctas
        tiles = max(1, -(-max_seq_len // 128))
        return max(1, min(want, max(1, tiles // 2), 32))
    return lib().b200_attn_decode_splits(batch, num_kv_heads, group, head_dim, max_seq_len)


def attn_decode(q: torch.Tensor, kv_cache: torch.Tensor, *, block_table: torch.Tensor,
                seq_lens: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                block_size: int, scale: float, out: torch.Tensor | None = None, splits: int = 0,
                softcap: float = 0.0, window: int = 0, tmp: tuple | None = None,
                force_cuda_core: bool = False):
    """Paged decode attention, one query row per sequence."""
    B = q.shape[0]
    if out is None:
        out = torch.empty((B, num_q_heads * head_dim), dtype=q.dtype, device=q.device)
    use_tc = (not force_cuda_core) and _decode_uses_tc(head_dim, num_q_heads // num_kv_heads,
                                                       block_size)
    if splits <= 0:
        splits = attn_decode_splits(B, num_kv_heads, num_q_heads // num_kv_heads, head_dim,
                                    block_table.shape[1] * block_size,
                                    block_size if use_tc else 0)
    tmp_o = tmp_lse = None
    if splits > 1:
        if tmp is None:
            tmp_o = torch.empty((B, num_q_heads, splits, head_dim), dtype=torch.float32,
                                device=q.device)
            tmp_lse = torch.empty((B, num_q_heads, splits), dtype=torch.float32, device=q.device)
        else:
            tmp_o, tmp_lse = tmp
    if use_tc:
        check(lib().b200_attn_decode_tc(
            ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(kv_cache), kv_cache.shape[0],
            block_size, num_q_heads, num_kv_heads, head_dim, ptr(block_table),
            block_table.stride(0), ptr(seq_lens), B, scale, softcap, window, splits, ptr(tmp_o),
            ptr(tmp_lse), stream_ptr()), "attn_decode_tc")
        return out
    check(lib().b200_attn_decode(
        ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(kv_cache), block_size, num_q_heads,
        num_kv_heads, head_dim, ptr(block_table), block_table.stride(0), ptr(seq_lens), B, scale,
        softcap, window, splits, ptr(tmp_o), ptr(tmp_lse), stream_ptr()), "attn_decode")
    return out


def merge_attn_states(a, lse_a, b, lse_b, out=None, lse_out=None):
    T, H, D = a.shape
    if out is None:
        out = torch.empty_like(a)
    check(lib().b200_merge_attn_states(ptr(a), ptr(lse_a), ptr(b), ptr(lse_b), ptr(out),
                                       ptr(lse_out), T, H, D, stream_ptr()), "merge_attn_states")
    return out


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    n, V = logits.shape
    assert logits.dtype == torch.float32
    if out is None:
        out = torch.empty((n,), dtype=torch.int64, device=logits.device)
    ws = workspace(logits.device, max(n, 1) * 64 * 8 + 1024, "argmax")
    sf = ws[: n * 64 * 4]
    si = ws[n * 64 * 4: n * 64 * 8]
    check(lib().b200_argmax(ptr(logits), logits.stride(0), n, V, ptr(out), ptr(sf), ptr(si),
                            stream_ptr()), "argmax")
    return out


def argmax_candidates(logits: torch.Tensor, v_valid: int, index_base: int, out: torch.Tensor) -> torch.Tensor:
    """Local stage of the vocabulary-parallel argmax: ``out[n, 2]`` int32 = (bits of the best
    value, ``index_base`` + its column) over the first ``v_valid`` columns of this rank's shard."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= 2 * n
    ws = workspace(logits.device, max(n, 1) * 64 * 8 + 1024, "argmax")
    check(lib().b200_argmax_candidates(ptr(logits), logits.stride(0), n, V, v_valid, index_base, ptr(out),
                                       ptr(ws[: n * 64 * 4]), ptr(ws[n * 64 * 4: n * 64 * 8]), stream_ptr()),
          "argmax_candidates")
    return out


def argmax_combine(cand: torch.Tensor, n: int, world: int, vocab: int, out: torch.Tensor) -> torch.Tensor:
    """Final stage: ``cand[world, n, 2]`` (rank-major) -> ``out[n]`` int64 ids; ties go to the
    lowest index, as in :func:`argmax` over the full row."""
    check(lib().b200_argmax_combine(ptr(cand), n, world, vocab, ptr(out), stream_ptr()), "argmax_combine")
    return out


def apply_temperature(logits, temperature):
    n, V = logits.shape
    check(lib().b200_apply_temperature(ptr(logits), logits.stride(0), n, V, ptr(temperature),
                                       stream_ptr()), "apply_temperature")
    return logits


def apply_penalties(logits, rows, toks, out_counts, rep, freq, pres):
    check(lib().b200_apply_penalties(ptr(logits), logits.stride(0), logits.shape[1], ptr(rows),
                                     ptr(toks), ptr(out_counts), rows.numel(), ptr(rep), ptr(freq),
                                     ptr(pres), stream_ptr()), "apply_penalties")
    return logits


def apply_logit_bias(logits, rows, toks, vals):
    check(lib().b200_sparse_edit(ptr(logits), logits.stride(0), logits.shape[1], ptr(rows),
                                 ptr(toks), ptr(vals), rows.numel(), 0, stream_ptr()), "logit_bias")
    return logits


def apply_token_mask(logits, rows, toks):
    check(lib().b200_sparse_edit(ptr(logits), logits.stride(0), logits.shape[1], ptr(rows),
                                 ptr(toks), 0, rows.numel(), 1, stream_ptr()), "token_mask")
    return logits


def apply_bitmask(logits, mask, row_ids=None):
    check(lib().b200_apply_bitmask(ptr(logits), logits.stride(0), logits.shape[1], ptr(mask),
                                   mask.shape[0], ptr(row_ids), stream_ptr()), "apply_bitmask")
    return logits


def apply_min_p(logits, min_p):
    n, V = logits.shape
    check(lib().b200_apply_min_p(ptr(logits), logits.stride(0), n, V, ptr(min_p), stream_ptr()),
          "apply_min_p")
    return logits


def apply_top_k_top_p(logits, top_k, top_p):
    n, V = logits.shape
    check(lib().b200_apply_top_k_top_p(ptr(logits), logits.stride(0), n, V, ptr(top_k), ptr(top_p),
                                       stream_ptr()), "apply_top_k_top_p")
    return logits


def softmax(logits, log: bool = False, out=None):
    n, V = logits.shape
    if out is None:
        out = torch.empty_like(logits)
    check(lib().b200_softmax(ptr(logits), logits.stride(0), ptr(out), out.stride(0), n, V,
                             int(log), stream_ptr()), "softmax")
    return out


def random_sample(probs, seeds, steps, out=None):
    n, V = probs.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int64, device=probs.device)
    check(lib().b200_random_sample(ptr(probs), probs.stride(0), n, V, ptr(seeds), ptr(steps),
                                   ptr(out), stream_ptr()), "random_sample")
    return out


def merge_greedy_random(greedy, rand, temperature, out=None):
    if out is None:
        out = torch.empty_like(greedy)
    check(lib().b200_merge_greedy_random(ptr(greedy), ptr(rand), ptr(temperature), ptr(out),
                                         greedy.numel(), stream_ptr()), "merge_greedy_random")
    return out


def token_rank(logprobs, toks):
    n, V = logprobs.shape
    lp = torch.empty((n,), dtype=torch.float32, device=logprobs.device)
    rk = torch.empty((n,), dtype=torch.int32, device=logprobs.device)
    check(lib().b200_token_rank(ptr(logprobs), logprobs.stride(0), n, V, ptr(toks), ptr(lp),
                                ptr(rk), stream_ptr()), "token_rank")
    return lp, rk


def greedy_reject(target_argmax, draft, cu_draft, max_spec):
    n = cu_draft.numel() - 1
    out = torch.empty((n, max_spec + 1), dtype=torch.int64, device=draft.device)
    check(lib().b200_greedy_reject(ptr(target_argmax), ptr(draft), ptr(cu_draft), n, max_spec,
                                   ptr(out), stream_ptr()), "greedy_reject")
    return out


def read_status() -> int:
    """Status word of the current device (0 = ok). Synchronises; call between steps."""
    return lib().b200_read_status()


def num_sms() -> int:
    return lib().b200_num_sms()
