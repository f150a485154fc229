"""Loader for the in-tree sm_100a kernel library (``_kernels.so``).

The library is plain C (raw pointers + stream), so the same entry points serve the Python
wrappers here and the C++ runtime. Loading fails loudly: on a machine with a GPU a missing
library is an error, never a silent fallback to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch  # noqa: F401  (loads libcudart before the kernel library resolves against it)

_PKG = Path(__file__).resolve().parent.parent
# B200_KERNELS_SO: load another build of the library (e.g. one compiled with instrumentation)
_LIB_PATH = Path(os.environ["B200_KERNELS_SO"]) if os.environ.get("B200_KERNELS_SO") else _PKG / "_kernels.so"
_lib = None


class KernelLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            if os.environ.get("VLLM_B200_AUTOBUILD", "1") == "1":
                from .. import _build
                _build.build_kernels()
            if not _LIB_PATH.exists():
                raise KernelLibraryMissing(
                    f"{_LIB_PATH} not found: run `python -m vllm_cpp_b200._build`")
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except (KernelLibraryMissing, OSError):
        return False


P = ctypes.c_void_p
I = ctypes.c_int
L = ctypes.c_int64
F = ctypes.c_float
Z = ctypes.c_size_t

_SIGS = {
    "b200_num_sms": ([], I),
    "b200_init_device": ([], I),
    "b200_read_status": ([], I),
    "b200_status_ptr": ([], P),
    "b200_set_peer_wait_cycles": ([ctypes.c_longlong], ctypes.c_longlong),
    "b200_gemm_bf16": ([P, I, P, I, P, I, I, P, P, I, I, I, I, P, Z, I, P], I),
    "b200_rmsnorm": ([P, I, P, P, P, I, I, I, F, I, P], I),
    "b200_layernorm": ([P, P, P, P, I, I, F, P], I),
    "b200_act_and_mul": ([P, I, P, I, I, I, P], I),
    "b200_gemm_bf16_gated": ([P, I, P, I, P, I, I, I, I, I, I, P], I),
    "b200_eltwise": ([P, P, P, Z, I, F, P], I),
    "b200_cast_bf16_f32": ([P, P, Z, P], I),
    "b200_cast_f32_bf16": ([P, P, Z, P], I),
    "b200_embedding": ([P, P, P, I, I, L, L, L, F, P], I),
    "b200_gather_rows": ([P, P, P, I, I, I, P], I),
    "b200_rope_kv": ([P, I, I, I, I, I, I, I, I, I, P, P, P, P, F, I, I, P, P, I, P, I, P], I),
    "b200_reshape_and_cache": ([P, I, P, I, P, P, I, I, I, I, P], I),
    "b200_concat_and_cache_mla": ([P, I, P, I, P, P, I, I, I, P], I),
    "b200_rope_table": ([P, P, I, I, F, P], I),
    "b200_attn_prefill": ([P, I, P, I, P, P, L, I, I, I, I, P, I, P, P, P, P, I, I, F, F, I, I, P], I),
    "b200_attn_decode_splits": ([I, I, I, I, I], I),
    "b200_attn_decode": ([P, I, P, I, P, I, I, I, I, P, I, P, I, F, F, I, I, P, P, P], I),
    "b200_attn_decode_tc": ([P, I, P, I, P, L, I, I, I, I, P, I, P, I, F, F, I, I, P, P, P], I),
    "b200_merge_attn_states": ([P, P, P, P, P, P, I, I, I, P], I),
    "b200_argmax": ([P, I, I, I, P, P, P, P], I),
    "b200_argmax_candidates": ([P, I, I, I, I, I, P, P, P, P], I),
    "b200_argmax_combine": ([P, I, I, I, P, P], I),
    "b200_apply_temperature": ([P, I, I, I, P, P], I),
    "b200_apply_penalties": ([P, I, I, P, P, P, I, P, P, P, P], I),
    "b200_sparse_edit": ([P, I, I, P, P, P, I, I, P], I),
    "b200_apply_bitmask": ([P, I, I, P, I, P, P], I),
    "b200_apply_min_p": ([P, I, I, I, P, P], I),
    "b200_apply_top_k_top_p": ([P, I, I, I, P, P, P], I),
    "b200_softmax": ([P, I, P, I, I, I, I, P], I),
    "b200_random_sample": ([P, I, I, I, P, P, P, P], I),
    "b200_merge_greedy_random": ([P, P, P, P, I, P], I),
    "b200_token_rank": ([P, I, I, I, P, P, P, P], I),
    "b200_greedy_reject": ([P, P, P, I, I, P, P], I),
    "b200_splice_sampled": ([P, P, P, P, I, P], I),
    "b200_scatter_sampled": ([P, P, P, I, P], I),
    "b200_splitmix64": ([ctypes.c_uint64], ctypes.c_uint64),
}


def _declare(l: ctypes.CDLL) -> None:
    for name, (args, res) in _SIGS.items():
        try:
            fn = getattr(l, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = res


def declare(name: str, args, res=I) -> None:
    """Register the signature of an entry point added by a later kernel file."""
    _SIGS[name] = (args, res)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = args
        fn.restype = res


class KernelError(RuntimeError):
    pass


_CODES = {-1: "rejected shape/alignment", -2: "launch failure", -3: "tensor-map encode failure",
          -4: "size beyond the stated maximum"}


LAUNCHES = [0]  # launcher calls made by this process (each launches >= 1 kernel)

# B200_SYNC_CHECK=1: synchronise the device after every launcher call and name the first one
# after which the device reports an error (asynchronous faults otherwise surface far from
# their cause). A debugging aid: it serialises host and device.
SYNC_CHECK = os.environ.get("B200_SYNC_CHECK", "0") == "1"


def sync_check(what: str) -> None:
    if torch.cuda.is_current_stream_capturing():
        return
    try:
        torch.cuda.synchronize()
    except Exception as e:  # the context is gone: report and leave without running destructors
        import sys
        sys.stderr.write(f"\nB200_SYNC_CHECK: the device reported an error after launcher '{what}': "
                         f"{str(e).splitlines()[0]}\n")
        sys.stderr.flush()
        os._exit(3)


def check(rc: int, what: str) -> None:
    LAUNCHES[0] += 1
    if rc != 0:
        raise KernelError(f"{what}: {_CODES.get(rc, 'error')} (code {rc})")
    if SYNC_CHECK:
        sync_check(what)


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """Handle of the current CUDA stream of the current device. Called once per kernel launch, so
    it goes through the raw C entry point (``torch.cuda.current_stream()`` builds a Stream object
    and resolves the device through several Python layers, ~14 us a call)."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch._C._cuda_getDevice())
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


class _DevPtr:
    def __init__(self, p: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (p, False),
                                         "version": 3, "strides": None}


def device_view(p: int, nbytes: int, device) -> torch.Tensor:
    """uint8 tensor over ``nbytes`` of device memory that the kernel library owns."""
    return torch.as_tensor(_DevPtr(p, nbytes), device=device)


def status_word(device) -> torch.Tensor:
    """int32[1] view of the current device's kernel status word (non-zero after a bounded wait
    inside a kernel ran out; see ``b200_read_status``)."""
    p = lib().b200_status_ptr()
    if not p:
        raise KernelError("the kernel status word could not be allocated")
    return device_view(p, 4, device).view(torch.int32)
