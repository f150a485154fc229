"""Quantised GEMM wrappers (fp8 e4m3, NVFP4 weights x bf16 activations) and the activation /
weight quantisation producers, with fp32 PyTorch restatements of the formats."""
from __future__ import annotations

import torch

from . import _lib, workspace
from ._lib import check, lib, ptr, stream_ptr

_declared = False
FP4_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _declare():
    global _declared
    if _declared:
        return
    P, I, L, F, Z = _lib.P, _lib.I, _lib.L, _lib.F, _lib.Z
    _lib.declare("b200_gemm_fp8", [P, I, P, I, P, I, P, P, I, P, I, I, I, P], I)
    _lib.declare("b200_nvfp4_dequant", [P, P, P, P, L, I, P], I)
    _lib.declare("b200_gemm_w4a16", [P, I, P, P, P, P, I, P, I, I, I, P, Z, P], I)
    _lib.declare("b200_gemm_nvfp4", [P, P, P, P, P, P, P, I, P, I, I, I, I, P, Z, P], I)
    _lib.declare("b200_nvfp4_sf_to_chunks", [P, L, I, I, P, P], I)
    _lib.declare("b200_quant_fp8", [P, L, P, F, I, P, P, L, L, I, P], I)
    _lib.declare("b200_quant_fp8_dynamic", [P, L, P, P, L, L, I, P], I)
    _lib.declare("b200_quant_fp8_rowwise", [P, L, P, P, F, I, I, I, P, L, P, I, I, P], I)
    _lib.declare("b200_quant_nvfp4", [P, L, P, P, P, L, I, I, I, P], I)
    _lib.declare("b200_quant_nvfp4_gated", [P, L, P, L, P, P, P, L, I, I, P], I)
    _lib.declare("b200_rmsnorm_quant_nvfp4", [P, L, P, P, F, I, P, P, P, P, L, I, I, P], I)
    lib()
    _declared = True


def gemm_fp8(a8, w8, a_scale, w_scale, out=None, bias=None):
    """a8 [M, K], w8 [N, K] float8_e4m3fn; a_scale fp32 [1] (per tensor) or [M] (per token, M > 1);
    w_scale fp32 [1] or [N]."""
    _declare()
    M, K = a8.shape
    N = w8.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    assert a_scale.numel() in (1, M) and w_scale.numel() in (1, N)
    flags = int(w_scale.numel() > 1) | (2 if a_scale.numel() == M else 0)     # M == 1: either reading is the same
    check(lib().b200_gemm_fp8(ptr(a8), a8.stride(0), ptr(w8), w8.stride(0), ptr(out), out.stride(0),
                              ptr(a_scale), ptr(w_scale), flags, ptr(bias), M, N, K,
                              stream_ptr()), "gemm_fp8")
    return out


def nvfp4_dequant(packed, sf, gscale, out=None):
    _declare()
    N, kh = packed.shape
    if out is None:
        out = torch.empty((N, kh * 2), dtype=torch.bfloat16, device=packed.device)
    check(lib().b200_nvfp4_dequant(ptr(packed), ptr(sf), ptr(gscale), ptr(out), N, kh * 2, stream_ptr()),
          "nvfp4_dequant")
    return out


def gemm_w4a16(a, packed, sf, gscale, out=None, bias=None, scratch=None):
    """a bf16 [M, K]; packed uint8 [N, K/2]; sf e4m3 bytes [N, K/16]; gscale fp32 [1] (multiplier).
    M <= 128 runs the fused expand-in-shared-memory kernel; larger M expands the matrix into
    ``scratch`` (bf16 [N, K]) once and runs the bf16 GEMM."""
    _declare()
    from . import gemm
    M, K = a.shape
    N = packed.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if M <= 128:
        ws = workspace(a.device, 64 << 20, "w4")
        check(lib().b200_gemm_w4a16(ptr(a), a.stride(0), ptr(packed), ptr(sf), ptr(gscale), ptr(out),
                                    out.stride(0), ptr(bias), M, N, K, ptr(ws), ws.numel(), stream_ptr()),
              "gemm_w4a16")
        return out
    if scratch is None:
        scratch = torch.empty((N, K), dtype=torch.bfloat16, device=a.device)
    nvfp4_dequant(packed, sf, gscale, scratch)
    return gemm(a, scratch[:N], bias=bias, out=out)


def quant_fp8(x, scale, out=None, norm_weight=None, eps=1e-6, gemma=False):
    """fp8(x / scale), optionally after RMSNorm. Returns a float8_e4m3fn tensor."""
    _declare()
    T, H = x.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    check(lib().b200_quant_fp8(ptr(x), x.stride(0), ptr(norm_weight), eps, int(gemma), ptr(scale), ptr(out),
                               out.stride(0), T, H, stream_ptr()), "quant_fp8")
    return out


def quant_fp8_rowwise(x, out=None, scales=None, norm_weight=None, eps=1e-6, gemma=False, residual=None,
                      act_kind=None, interleaved=False):
    """Per-token dynamic fp8: every row gets the scale max|row| / 448. The producer of the row can
    run in the same kernel: RMSNorm (``norm_weight``; with ``residual`` the sum is written back to
    it first), or ``act(gate) * up`` over ``[gate | up]`` rows (``act_kind``). Returns
    (float8_e4m3fn [T, K], scales fp32 [T])."""
    _declare()
    T = x.shape[0]
    mode = 1 if norm_weight is not None else (2 if act_kind is not None else 0)
    K = x.shape[1] // 2 if mode == 2 else x.shape[1]
    if out is None:
        out = torch.empty((T, K), dtype=torch.float8_e4m3fn, device=x.device)
    if scales is None:
        scales = torch.empty(T, dtype=torch.float32, device=x.device)
    flags = (int(act_kind) | (0x100 if interleaved else 0)) if mode == 2 else 0
    check(lib().b200_quant_fp8_rowwise(ptr(x), x.stride(0), ptr(residual), ptr(norm_weight), eps, int(gemma), mode,
                                       flags, ptr(out), out.stride(0), ptr(scales), T, K, stream_ptr()),
          "quant_fp8_rowwise")
    return out, scales


def quant_fp8_dynamic(x, out=None):
    """Per-tensor dynamic fp8: scale = max|x| / 448 taken on the device (no host read). Returns
    (float8_e4m3fn [T, H], scale fp32 [1]); the scale lives in a per-device scratch word, valid
    until the next call on that device (the GEMM that follows on the stream reads it)."""
    _declare()
    T, H = x.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    scratch = workspace(x.device, 8, "fp8_dyn_scale").view(torch.float32)
    check(lib().b200_quant_fp8_dynamic(ptr(x), x.stride(0), ptr(scratch), ptr(out), out.stride(0), T, H,
                                       stream_ptr()), "quant_fp8_dynamic")
    return out, scratch[1:2]


def quant_nvfp4(x, gscale, K=None, silu_mul=False, swizzle=False, out=None):
    """Returns (packed uint8 [T, K/2], block scales uint8). gscale fp32 [1]. ``out``: a
    (packed, scales) pair to write into (scale rows past T are left as they are: they only
    ever meet zero-filled activation rows)."""
    _declare()
    T = x.shape[0]
    K = K or (x.shape[1] // 2 if silu_mul else x.shape[1])
    n_sf = ((T + 127) // 128) * 128 * (K // 16) if swizzle else T * (K // 16)
    if out is not None:
        packed, sf = out
        assert packed.shape == (T, K // 2) and sf.numel() >= n_sf
    else:
        packed = torch.empty((T, K // 2), dtype=torch.uint8, device=x.device)
        sf = torch.zeros(n_sf, dtype=torch.uint8, device=x.device)
    check(lib().b200_quant_nvfp4(ptr(x), x.stride(0), ptr(gscale), ptr(packed), ptr(sf), T, K,
                                 int(silu_mul), int(swizzle), stream_ptr()), "quant_nvfp4")
    return packed, (sf if swizzle else sf.view(T, K // 16))


def _nvfp4_out(T, K, swizzle, device, out):
    n_sf = ((T + 127) // 128) * 128 * (K // 16) if swizzle else T * (K // 16)
    if out is not None:
        packed, sf = out
        assert packed.shape == (T, K // 2) and sf.numel() >= n_sf
        return packed, sf
    return (torch.empty((T, K // 2), dtype=torch.uint8, device=device),
            torch.zeros(n_sf, dtype=torch.uint8, device=device))


def quant_nvfp4_gated(x, gate, gscale, swizzle=False, out=None):
    """``x * sigmoid(gate)`` -> NVFP4 (the gated attention output in front of o_proj); reference
    producer ``src/vt/cuda/cuda_matmul_nvfp4.cu:1826``."""
    _declare()
    T, K = x.shape
    packed, sf = _nvfp4_out(T, K, swizzle, x.device, out)
    check(lib().b200_quant_nvfp4_gated(ptr(x), x.stride(0), ptr(gate), gate.stride(0), ptr(gscale), ptr(packed),
                                       ptr(sf), T, K, int(swizzle), stream_ptr()), "quant_nvfp4_gated")
    return packed, (sf if swizzle else sf[: T * (K // 16)].view(T, K // 16))


def rmsnorm_quant_nvfp4(x, weight, eps, gscale, residual=None, gemma=False, swizzle=False, out=None,
                        normed=None):
    """(``residual += x``;) RMSNorm -> NVFP4 in one kernel; ``normed`` optionally receives the bf16
    normalised rows too. Reference producer ``src/vt/cuda/cuda_matmul_nvfp4.cu:1667``."""
    _declare()
    T, K = x.shape
    packed, sf = _nvfp4_out(T, K, swizzle, x.device, out)
    if residual is not None:
        assert residual.is_contiguous() and residual.shape == (T, K)
    check(lib().b200_rmsnorm_quant_nvfp4(ptr(x), x.stride(0), ptr(residual), ptr(weight), float(eps), int(gemma),
                                         ptr(gscale), ptr(packed), ptr(sf), ptr(normed), T, K, int(swizzle),
                                         stream_ptr()), "rmsnorm_quant_nvfp4")
    return packed, (sf if swizzle else sf[: T * (K // 16)].view(T, K // 16))


def nvfp4_sf_chunks(sf: torch.Tensor, pad_rows: int = 256) -> torch.Tensor:
    """Row-major e4m3 block scales ``[rows, K/16]`` -> the 128 x 4 chunk layout the block-scaled MMA
    reads (rows padded with zero scales to a multiple of ``pad_rows``); done once per weight."""
    _declare()
    rows, kb = sf.shape
    padded = (rows + pad_rows - 1) // pad_rows * pad_rows
    out = torch.empty(padded * kb, dtype=torch.uint8, device=sf.device)
    check(lib().b200_nvfp4_sf_to_chunks(ptr(sf.contiguous()), rows, kb * 16, pad_rows, ptr(out), stream_ptr()),
          "nvfp4_sf_to_chunks")
    return out


# (rows bucket, N, K) -> weight rows per CTA; filled by the heuristic or, with B200_NVFP4_AUTOTUNE=1, by
# timing both tile widths once per shape (outside stream capture)
_NVFP4_PLANS: dict[tuple[int, int, int], int] = {}
_PLAN_FILE_READ = [False]


def _plan_file() -> str:
    import os
    return os.environ.get("B200_NVFP4_PLAN_FILE", "")


def load_nvfp4_plans(path: str | None = None) -> int:
    """Reads plans saved by an earlier process (JSON ``{"M,N,K": tile}``); plans already in memory
    win. Returns the number read. A missing or unreadable file is no plans, not an error: the cache
    is an optimisation (reference: ``nvfp4_persistent_cache.cpp``, the tactic cache that survives
    restarts so that serving does not re-tune)."""
    import json
    import os
    path = path or _plan_file()
    if not path or not os.path.exists(path):
        return 0
    try:
        with open(path) as f:
            raw = json.load(f)
    except (OSError, ValueError):
        return 0
    n = 0
    for k, v in raw.items():
        try:
            key = tuple(int(x) for x in k.split(","))
        except ValueError:
            continue
        if len(key) == 3 and v in (128, 256) and key not in _NVFP4_PLANS:
            _NVFP4_PLANS[key] = int(v)
            n += 1
    return n


def save_nvfp4_plans(path: str | None = None) -> None:
    """Writes the plan table (atomically: a temporary file, then a rename)."""
    import json
    import os
    path = path or _plan_file()
    if not path:
        return
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump({",".join(map(str, k)): v for k, v in sorted(_NVFP4_PLANS.items())}, f, indent=0)
    os.replace(tmp, path)


def _m_bucket(M: int) -> int:
    for b in (16, 64, 128, 512, 2048):
        if M <= b:
            return b
    return 8192


def nvfp4_plan(M: int, N: int, K: int, run=None) -> int:
    """Tile width (128 or 256 weight rows per CTA) of the W4A4 GEMM for a shape, cached per
    (rows bucket, N, K). Heuristic: 256-row tiles unless they leave more than a third of the SMs
    without a tile at decode sizes, where two 128-row tiles per 256 rows spread better (measured:
    34816 x 5120 at 64 rows 37 us with 256 against 44 us with 128; 5120 x 17408 36.9 against 34.6).
    ``run(n_tile)``: when given and B200_NVFP4_AUTOTUNE=1, both widths are timed once with CUDA
    events and the faster one is kept (reference: the per-shape tactic cache of
    ``src/vt/cuda/nvfp4_cutlass_tactic_impl.cuh``)."""
    import os
    if not _PLAN_FILE_READ[0]:
        _PLAN_FILE_READ[0] = True
        load_nvfp4_plans()
    key = (_m_bucket(M), N, K)
    plan = _NVFP4_PLANS.get(key)
    if plan is not None:
        return plan
    from . import num_sms
    tiles256 = -(-N // 256) * -(-M // 128)
    plan = 128 if (M <= 128 and tiles256 * 3 < num_sms() * 2 and N >= 256) else 256
    if run is not None and os.environ.get("B200_NVFP4_AUTOTUNE", "0") == "1" \
            and not torch.cuda.is_current_stream_capturing():
        best = None
        for nt in (256, 128):
            for _ in range(2):
                run(nt)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                run(nt)
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1)
            if best is None or t < best[0]:
                best = (t, nt)
        plan = best[1]
        _NVFP4_PLANS[key] = plan
        save_nvfp4_plans()            # timed plans are worth keeping across restarts (B200_NVFP4_PLAN_FILE)
    _NVFP4_PLANS[key] = plan
    return plan


def gemm_nvfp4(aq, sfa, g_a, wq, sfw, g_w, out=None, bias=None, n_tile: int = 0):
    """W4A4: ``aq`` uint8 [M, K/2] and ``sfa`` from :func:`quant_nvfp4` (``swizzle=True``, global scale
    ``g_a``); ``wq`` uint8 [N, K/2], ``sfw`` from :func:`nvfp4_sf_chunks`, ``g_w`` the weight's fp32
    multiplier. Both products run on ``tcgen05.mma.kind::mxf4nvf4`` with the scales in tensor memory.
    ``n_tile`` 0: the cached plan of the shape (:func:`nvfp4_plan`)."""
    _declare()
    if aq.dim() != 2 or wq.dim() != 2 or aq.shape[1] != wq.shape[1] or (aq.shape[1] * 2) % 256 or wq.shape[0] % 8:
        from .validate import validate
        validate("gemm_nvfp4", aq=aq, wq=wq, sfa=sfa, sfw=sfw, g_a=g_a, g_w=g_w)
    M, kh = aq.shape
    N = wq.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    ws = workspace(aq.device, 64 << 20, "w4")

    def run(nt):
        check(lib().b200_gemm_nvfp4(ptr(aq), ptr(sfa), ptr(g_a), ptr(wq), ptr(sfw), ptr(g_w), ptr(out), out.stride(0),
                                    ptr(bias), M, N, kh * 2, nt, ptr(ws), ws.numel(), stream_ptr()),
              f"gemm_nvfp4 M={M} N={N} K={kh * 2}")

    run(n_tile or nvfp4_plan(M, N, kh * 2, run))
    return out


# ------------------------------------------------------------------------------ references
def ref_quant_nvfp4_weights(w: torch.Tensor):
    """Quantise an fp32/bf16 [N, K] matrix to NVFP4: (packed, e4m3 scale bytes, global scale
    multiplier fp32 [1]) such that w ~= e2m1 * e4m3_scale * global."""
    wf = w.float()
    N, K = wf.shape
    amax = wf.abs().max().clamp_min(1e-12)
    g = (amax / (448.0 * 6.0)).reshape(1)                   # multiplier
    blocks = wf.reshape(N, K // 16, 16)
    bmax = blocks.abs().amax(-1)
    s8 = (bmax / 6.0 / g).to(torch.float8_e4m3fn)
    sdec = s8.float() * g
    q = blocks / sdec.clamp_min(1e-30).unsqueeze(-1)
    vals = torch.tensor(FP4_VALUES, device=w.device)
    idx = (q.abs().unsqueeze(-1) - vals).abs().argmin(-1)
    code = (idx | ((q < 0).long() << 3)).reshape(N, K).to(torch.uint8)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return packed, s8.view(torch.uint8).contiguous(), g.to(torch.float32)


def ref_quant_nvfp4_activations(x: torch.Tensor, gscale: torch.Tensor):
    """The activation quantiser restated in PyTorch: per 16 values the scale is
    e4m3(amax * gscale / 6) and the codes are e2m1(x * gscale / scale), nearest with ties to the
    even code. Returns (packed uint8 [T, K/2], scale bytes uint8 [T, K/16])."""
    xf = x.float()
    T, K = xf.shape
    gs = gscale.float().reshape(())
    blocks = xf.reshape(T, K // 16, 16)
    s8 = (blocks.abs().amax(-1) * gs / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    sdec = s8.float()
    mul = torch.where(sdec > 0, gs / sdec.clamp_min(1e-30), torch.zeros_like(sdec)).unsqueeze(-1)
    q = blocks * mul
    a = q.abs()
    code = ((a > 0.25).long() + (a >= 0.75).long() + (a > 1.25).long() + (a >= 1.75).long() +
            (a > 2.5).long() + (a >= 3.5).long() + (a > 5.0).long())
    code = (code | ((q < 0).long() << 3)).reshape(T, K).to(torch.uint8)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return packed, s8.view(torch.uint8).contiguous()


def ref_dequant_nvfp4(packed, sf_bytes, g):
    N, kh = packed.shape
    vals = torch.tensor(FP4_VALUES + [-v for v in FP4_VALUES], device=packed.device)
    p = packed.long()
    v = torch.stack([vals[p & 15], vals[p >> 4]], -1).reshape(N, kh * 2)
    s = sf_bytes.view(torch.float8_e4m3fn).float() * g.float()
    return (v.reshape(N, -1, 16) * s.reshape(N, -1, 1)).reshape(N, kh * 2)
