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
