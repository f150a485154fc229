"""ctypes view of the native per-layer launch entry (``csrc/kernels/layer.cu``): one call issues
every kernel of a pre-norm dense decoder block, instead of ~10 Python-level launches."""
from __future__ import annotations

import ctypes as C

from . import _lib as _lib_mod
from ._lib import LAUNCHES, KernelError, lib, stream_ptr

P, I, F = C.c_void_p, C.c_int, C.c_float


class DenseLayerWeights(C.Structure):
    _fields_ = [("ln1", P), ("qkv", P), ("q_norm", P), ("k_norm", P), ("o", P), ("ln2", P), ("gate_up", P),
                ("down", P), ("kv_cache", P),
                ("fp8", I), ("qkv_scale", P), ("o_scale", P), ("gate_up_scale", P), ("down_scale", P)]


class DenseStep(C.Structure):
    _fields_ = [("T", I), ("H", I), ("Hq", I), ("Hkv", I), ("D", I), ("rot", I), ("inter", I), ("block_size", I),
                ("neox", I), ("gemma", I), ("act_kind", I), ("gate_up_interleaved", I),
                ("eps", F), ("scale", F), ("softcap", F), ("window", I), ("num_blocks", C.c_longlong),
                ("positions", P), ("cos_sin", P), ("slot_mapping", P), ("block_table", P), ("max_blocks", I),
                ("seq_lens", P), ("num_decodes", I), ("decode_splits", I), ("decode_tc", I),
                ("decode_tmp_o", P), ("decode_tmp_lse", P),
                ("num_prefills", I), ("num_tiles", I), ("num_prefill_tokens", I),
                ("prefill_q_start", P), ("tile_req", P), ("tile_q0", P),
                ("hidden", P), ("resid", P), ("normed", P), ("qkv_buf", P), ("attn", P), ("gate_up_buf", P),
                ("act", P), ("gemm_ws", P), ("gemm_ws_bytes", C.c_ulonglong), ("first_layer", I),
                ("fp8_act", P), ("fp8_scales", P)]


_declared = False


def dense_layer(weights: DenseLayerWeights, step: DenseStep) -> None:
    global _declared
    L = lib()
    if not _declared:
        L.b200_dense_layer.argtypes = [C.POINTER(DenseLayerWeights), C.POINTER(DenseStep), P]
        L.b200_dense_layer.restype = I
        _declared = True
    rc = L.b200_dense_layer(C.byref(weights), C.byref(step), stream_ptr())
    if rc < 0:
        raise KernelError(f"dense_layer: kernel launcher returned {rc}")
    LAUNCHES[0] += rc
    if _lib_mod.SYNC_CHECK:
        _lib_mod.sync_check(f"dense_layer T={step.T} decodes={step.num_decodes} prefills={step.num_prefills} "
                            f"splits={step.decode_splits}")


class TpLayers(C.Structure):
    """Peer-mapped buffers of the fused tensor-parallel path as ``b200_dense_layers_tp`` takes them."""
    _fields_ = [("world", I), ("rank", I), ("rpr_max", I), ("max_tokens", I),
                ("recv", P * 8), ("rs_flags", P * 8), ("x_full", P * 8), ("ag_flags", P * 8),
                ("op_counter", P), ("done_counter", P), ("residual", P), ("final_norm", P)]


_tp_declared = False


def dense_layers_tp(weights: list, step: DenseStep, tp: TpLayers) -> None:
    """Every block of the fused tensor-parallel forward in one native call."""
    global _tp_declared
    L = lib()
    n = len(weights)
    arr = getattr(dense_layers_tp, "_arr", None)
    if arr is None or arr[0] is not weights:
        packed = (DenseLayerWeights * n)(*weights)
        arr = (weights, packed)
        dense_layers_tp._arr = arr
    if not _tp_declared:
        L.b200_dense_layers_tp.argtypes = [C.POINTER(DenseLayerWeights), I, C.POINTER(DenseStep),
                                           C.POINTER(TpLayers), P]
        L.b200_dense_layers_tp.restype = I
        L.b200_tp_layers_abi.argtypes = [C.POINTER(I)]
        L.b200_tp_layers_abi.restype = None
        abi = (I * 2)()
        L.b200_tp_layers_abi(abi)
        if (abi[0], abi[1]) != (C.sizeof(TpLayers), TpLayers.final_norm.offset):
            raise KernelError("TpLayers layout differs between the binding and the kernel library")
        _tp_declared = True
    rc = L.b200_dense_layers_tp(arr[1], n, C.byref(step), C.byref(tp), stream_ptr())
    if rc < 0:
        raise KernelError(f"dense_layers_tp: kernel launcher returned {rc}")
    LAUNCHES[0] += rc
