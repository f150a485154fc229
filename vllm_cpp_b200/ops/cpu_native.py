"""ctypes front end of the native CPU backend (``csrc/cpu`` -> ``_cpu.so``): thread pool with
output-partitioned work and AVX2 / scalar tiers; bf16 storage, fp32 arithmetic.

Reference: ``src/vt/cpu/`` (threadpool, elementwise GEMM micro-kernels, paged attention, ops).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent.parent / "_cpu.so"
        if not path.exists():
            from .. import _build
            _build.build_cpu()
        L = C.CDLL(str(path))
        P, I, L64, F = C.c_void_p, C.c_int, C.c_int64, C.c_float
        L.b200cpu_set_threads.argtypes = [I]
        L.b200cpu_num_threads.restype = I
        L.b200cpu_simd_tier.restype = I
        L.b200cpu_matmul_bt.argtypes = [P, L64, P, L64, P, L64, I, P, P, L64, I, I, I]
        L.b200cpu_rmsnorm.argtypes = [P, L64, P, F, P, L64, P, L64, I, I, I]
        L.b200cpu_act_and_mul.argtypes = [P, L64, P, L64, I, I, I]
        L.b200cpu_embedding.argtypes = [P, P, P, L64, I, I, L64, L64, F]
        L.b200cpu_rope_kv.argtypes = [P, L64, P, P, I, I, I, I, I, I, P, P, F, I, P, P, I]
        L.b200cpu_paged_attention.argtypes = [P, L64, P, P, L64, P, P, I, I, I, I, I, F, F, I, P, L64]
        L.b200cpu_moe_router_topk.argtypes = [P, L64, I, I, I, I, I, P, I, I, F, P, P]
        L.b200cpu_moe_experts.argtypes = [P, L64, P, P, I, I, P, P, I, I, I, I, I, P, L64]
        L.b200cpu_gdn_conv1d.argtypes = [P, L64, P, P, P, P, P, I, I, P, L64]
        L.b200cpu_gdn_post_conv.argtypes = [P, L64, I, I, I, P, L64, P, L64, P, P, F, P, P, P, P]
        L.b200cpu_gdn_recurrent.argtypes = [P, P, P, L64, P, P, P, P, P, P, I, I, I, P]
        L.b200cpu_rmsnorm_gated.argtypes = [P, L64, P, L64, P, F, I, I, I, I, P, L64]
        L.b200cpu_mla_attention.argtypes = [P, L64, P, P, L64, P, P, I, P, I, F, I, P]
        L.b200cpu_matmul_bt_quant.argtypes = [P, L64, P, I, P, L64, I, I, I, I]
        L.b200cpu_quantize_blocks.argtypes = [P, L64, I, P]
        for name in ("b200cpu_moe_router_topk", "b200cpu_moe_experts", "b200cpu_gdn_conv1d",
                     "b200cpu_gdn_post_conv", "b200cpu_gdn_recurrent", "b200cpu_rmsnorm_gated",
                     "b200cpu_mla_attention", "b200cpu_matmul_bt_quant", "b200cpu_quantize_blocks"):
            getattr(L, name).restype = None
        for name in ("b200cpu_matmul_bt", "b200cpu_rmsnorm", "b200cpu_act_and_mul", "b200cpu_embedding",
                     "b200cpu_rope_kv", "b200cpu_paged_attention", "b200cpu_set_threads"):
            getattr(L, name).restype = None
        _LIB = L
    return _LIB


def _p(t):
    return None if t is None else t.data_ptr()


def _bf16(t):
    assert t.dtype == torch.bfloat16 and t.device.type == "cpu" and t.stride(-1) == 1
    return t


def set_num_threads(n: int) -> None:
    lib().b200cpu_set_threads(n)


def num_threads() -> int:
    return lib().b200cpu_num_threads()


def gemm(a, w, bias=None, residual=None, out=None, out_dtype=torch.bfloat16):
    _bf16(a), _bf16(w)
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype)
    assert out.stride(1) == 1
    lib().b200cpu_matmul_bt(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
                            1 if out.dtype == torch.float32 else 0, _p(bias), _p(residual),
                            residual.stride(0) if residual is not None else 0, M, N, K)
    return out


def rmsnorm(x, w, eps, residual=None, out=None, gemma=False):
    _bf16(x)
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    lib().b200cpu_rmsnorm(x.data_ptr(), x.stride(0), w.data_ptr(), float(eps), _p(residual),
                          residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0),
                          T, H, int(gemma))
    return out


def act_and_mul(x, kind=0, out=None):
    _bf16(x)
    T, two_i = x.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=x.dtype)
    lib().b200cpu_act_and_mul(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), T, inter, kind)
    return out


def embedding(ids, table, out=None, vocab_start=0, scale=1.0):
    ids = ids.to(torch.int64).contiguous()
    T, H = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype)
    lib().b200cpu_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), out.stride(0), T, H,
                            vocab_start, table.shape[0], float(scale))
    return out


def rope_kv(qkv, positions, table, *, num_q_heads, num_kv_heads, head_dim, rot_dim, neox, q_norm, k_norm,
            eps, gemma, slot_mapping, kv_cache, block_size):
    _bf16(qkv)
    pos = positions.to(torch.int64).contiguous()
    sm = slot_mapping.to(torch.int64).contiguous() if slot_mapping is not None else None
    tab = table.contiguous() if table is not None else None
    lib().b200cpu_rope_kv(qkv.data_ptr(), qkv.stride(0), pos.data_ptr(), _p(tab), qkv.shape[0], num_q_heads,
                          num_kv_heads, head_dim, rot_dim or head_dim, int(neox), _p(q_norm), _p(k_norm),
                          float(eps), int(gemma), _p(sm), _p(kv_cache), block_size)


def paged_attention(q, kv_cache, block_table, seq_lens, q_start, *, num_q_heads, num_kv_heads, head_dim,
                    block_size, scale, softcap=0.0, window=0, out=None):
    _bf16(q)
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, num_q_heads * head_dim), dtype=q.dtype)
    bt = block_table.to(torch.int32).contiguous()
    sl = seq_lens.to(torch.int32).contiguous()
    qs = q_start.to(torch.int32).contiguous()
    R = sl.numel()
    assert int(qs[R]) <= T
    lib().b200cpu_paged_attention(q.data_ptr(), q.stride(0), kv_cache.data_ptr(), bt.data_ptr(), bt.stride(0),
                                  sl.data_ptr(), qs.data_ptr(), R, num_q_heads, num_kv_heads, head_dim,
                                  block_size, float(scale), float(softcap), int(window), out.data_ptr(),
                                  out.stride(0))
    return out


# ------------------------------------------------------------------------------ mixture of experts
def _i32(t):
    return t.to(torch.int32).contiguous()


def moe_router_topk(logits, k, renorm=True, scoring="softmax", e_bias=None, n_group=1, topk_group=1,
                    routed_scale=1.0):
    """fp32 logits [T, E] -> (ids int32 [T, k], weights fp32 [T, k]); see ``ops.moe.ref_router_topk``."""
    lg = logits.float().contiguous()
    T, E = lg.shape
    ids = torch.empty((T, k), dtype=torch.int32)
    w = torch.empty((T, k), dtype=torch.float32)
    eb = e_bias.float().contiguous() if e_bias is not None else None
    lib().b200cpu_moe_router_topk(lg.data_ptr(), lg.stride(0), T, E, k, int(renorm), 0 if scoring == "softmax" else 1,
                                  _p(eb), n_group, topk_group, float(routed_scale), ids.data_ptr(), w.data_ptr())
    return ids, w


def moe_experts(x, ids, w, w_gate_up, w_down, e0=0, act_kind=0, out=None):
    """Routed-expert block of this rank's experts ``[e0, e0 + E_local)``: bf16 [T, H]."""
    _bf16(x)
    T, H = x.shape
    El, I2, _ = w_gate_up.shape
    ids, w = _i32(ids), w.float().contiguous()
    w_gate_up, w_down = w_gate_up.contiguous(), w_down.contiguous()
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16)
    lib().b200cpu_moe_experts(x.data_ptr(), x.stride(0), ids.data_ptr(), w.data_ptr(), T, ids.shape[1],
                              w_gate_up.data_ptr(), w_down.data_ptr(), e0, El, H, I2 // 2, act_kind,
                              out.data_ptr(), out.stride(0))
    return out


# ------------------------------------------------------------------------------ Gated DeltaNet
def gdn_conv1d(x, w, conv_state, qsl, slots, has_init, out=None):
    """Causal conv (kernel 4) + SiLU over ragged sequences; ``conv_state`` [slots, C, 3] is updated in place."""
    _bf16(x)
    T, C = x.shape
    assert conv_state.is_contiguous() and conv_state.dtype == torch.bfloat16 and w.shape == (C, 4)
    qsl, slots, has_init = _i32(torch.as_tensor(qsl)), _i32(torch.as_tensor(slots)), _i32(torch.as_tensor(has_init))
    if out is None:
        out = torch.empty((T, C), dtype=torch.bfloat16)
    w = w.contiguous()
    lib().b200cpu_gdn_conv1d(x.data_ptr(), x.stride(0), w.data_ptr(), conv_state.data_ptr(), qsl.data_ptr(),
                             slots.data_ptr(), has_init.data_ptr(), slots.numel(), C, out.data_ptr(), out.stride(0))
    return out


def gdn_post_conv(xc, Hk, Hv, a, b, A_log, dt_bias, eps=1e-6):
    """-> (q bf16 [T, Hk, 128], k bf16 [T, Hk, 128], g fp32 [T, Hv], beta fp32 [T, Hv])."""
    _bf16(xc), _bf16(a), _bf16(b)
    T = xc.shape[0]
    q = torch.empty((T, Hk, 128), dtype=torch.bfloat16)
    k = torch.empty((T, Hk, 128), dtype=torch.bfloat16)
    g = torch.empty((T, Hv), dtype=torch.float32)
    beta = torch.empty((T, Hv), dtype=torch.float32)
    al, db = A_log.float().contiguous(), dt_bias.float().contiguous()
    lib().b200cpu_gdn_post_conv(xc.data_ptr(), xc.stride(0), T, Hk, Hv, a.data_ptr(), a.stride(0), b.data_ptr(),
                                b.stride(0), al.data_ptr(), db.data_ptr(), float(eps), q.data_ptr(), k.data_ptr(),
                                g.data_ptr(), beta.data_ptr())
    return q, k, g, beta


def gdn_recurrent(q, k, v, g, beta, state, qsl, slots, has_init):
    """Sequential gated delta rule; ``v`` [T, Hv, 128] may be a strided view; ``state`` fp32
    [slots, Hv, 128, 128] is updated in place. Returns fp32 [T, Hv, 128]."""
    T, Hk, _ = q.shape
    Hv = v.shape[1]
    assert q.is_contiguous() and k.is_contiguous() and v.stride(2) == 1 and v.stride(1) == 128
    assert state.dtype == torch.float32 and state.is_contiguous()
    qsl, slots, has_init = _i32(torch.as_tensor(qsl)), _i32(torch.as_tensor(slots)), _i32(torch.as_tensor(has_init))
    out = torch.empty((T, Hv, 128), dtype=torch.float32)
    g, beta = g.float().contiguous(), beta.float().contiguous()
    lib().b200cpu_gdn_recurrent(q.data_ptr(), k.data_ptr(), v.data_ptr(), v.stride(0), g.data_ptr(), beta.data_ptr(),
                                state.data_ptr(), qsl.data_ptr(), slots.data_ptr(), has_init.data_ptr(),
                                slots.numel(), Hk, Hv, out.data_ptr())
    return out


def rmsnorm_gated(x, z, w, eps=1e-6, gate="silu", heads=1, out=None):
    _bf16(x), _bf16(z)
    T, W = x.shape
    if out is None:
        out = torch.empty((T, W), dtype=torch.bfloat16)
    w = w.to(torch.bfloat16).contiguous()
    lib().b200cpu_rmsnorm_gated(x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0), w.data_ptr(), float(eps), T,
                                heads, W // heads, 0 if gate == "silu" else 1, out.data_ptr(), out.stride(0))
    return out


# ------------------------------------------------------------------------------ multi-head latent attention
def mla_attention(q, cache, block_table, seq_lens, query_start, w_kvb, H, scale, block_size):
    """q bf16 [T, H, 192] (a view with row stride allowed); cache bf16 [nb, bs, 576]; -> fp32 [T, H, 128]."""
    assert q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == 192
    T = q.shape[0]
    bt, sl, qs = _i32(block_table), _i32(seq_lens), _i32(query_start)
    out = torch.zeros((T, H, 128), dtype=torch.float32)
    w_kvb, cache = w_kvb.contiguous(), cache.contiguous()
    lib().b200cpu_mla_attention(q.data_ptr(), q.stride(0), cache.data_ptr(), bt.data_ptr(), bt.stride(0),
                                sl.data_ptr(), qs.data_ptr(), sl.numel(), w_kvb.data_ptr(), H, float(scale),
                                block_size, out.data_ptr())
    return out


# ------------------------------------------------------------------------------ block-quantised weights
Q8_0, Q4_0 = 8, 4
_BLOCK_BYTES = {Q8_0: 34, Q4_0: 18}


def quantize_blocks(w: torch.Tensor, kind: int) -> torch.Tensor:
    """fp32 / bf16 [N, K] -> packed GGUF blocks uint8 [N, K / 32 * block_bytes]."""
    N, K = w.shape
    assert K % 32 == 0
    wf = w.float().contiguous()
    out = torch.empty((N, K // 32 * _BLOCK_BYTES[kind]), dtype=torch.uint8)
    lib().b200cpu_quantize_blocks(wf.data_ptr(), wf.numel(), kind, out.data_ptr())
    return out


def gemm_quant(a, wq, kind: int, out_dtype=torch.bfloat16):
    """``a[M, K] @ dequant(wq)[N, K]^T`` with the weights kept packed: per-block integer dot products
    against int8-quantised activations (reference ``src/vt/cpu/cpu_quant_gemm.cpp``)."""
    _bf16(a)
    M, K = a.shape
    N = wq.shape[0]
    assert wq.dtype == torch.uint8 and wq.is_contiguous() and wq.shape[1] == K // 32 * _BLOCK_BYTES[kind]
    out = torch.empty((M, N), dtype=out_dtype)
    lib().b200cpu_matmul_bt_quant(a.data_ptr(), a.stride(0), wq.data_ptr(), kind, out.data_ptr(), out.stride(0),
                                  1 if out_dtype == torch.float32 else 0, M, N, K)
    return out
