"""Op back ends the model code is written against.

``GpuBackend`` launches the sm_100a kernels (no eager fallback). ``CpuBackend`` evaluates the
same ops with the fp32 PyTorch restatements; it is the oracle the GPU path is compared with
(token-exact greedy gates) and the execution path of the CPU benchmark configuration.
"""
from __future__ import annotations

import os

import torch

from ..ops import reference as ref


class QuantWeight:
    """NVFP4 weight of a linear layer: E2M1 pairs, one E4M3 scale per 16 values, fp32 tensor
    scale (multiplier). ``shape`` mimics the dense [N, K] weight it replaces."""

    def __init__(self, packed, sf, gscale, input_gscale=None):
        self.packed, self.sf, self.gscale = packed, sf, gscale
        self.shape = (packed.shape[0], packed.shape[1] * 2)
        self.device = packed.device
        self._scratch = None
        self._sf_chunks = None
        # W4A4: global scale of the activation quantiser (448 * 6 / expected amax); checkpoints
        # calibrated for W4A4 carry it, otherwise a fixed scale that keeps block maxima between
        # 0.05 and 10^4 representable
        self.input_gscale = input_gscale

    def sf_chunks(self):
        """Block scales in the 128 x 4 chunk layout of the block-scaled MMA (built once)."""
        if self._sf_chunks is None:
            from ..ops.quant import nvfp4_sf_chunks
            self._sf_chunks = nvfp4_sf_chunks(self.sf, 256)
        return self._sf_chunks

    def act_gscale(self):
        if self.input_gscale is None:
            self.input_gscale = torch.full((1,), 4.0, dtype=torch.float32, device=self.device)
        return self.input_gscale

    def numel(self):
        return self.packed.numel() + self.sf.numel()

    def element_size(self):
        return 1

    def data_ptr(self):
        return self.packed.data_ptr()

    def dequant(self):
        from ..ops.quant import ref_dequant_nvfp4
        return ref_dequant_nvfp4(self.packed, self.sf, self.gscale).to(torch.bfloat16)

    @staticmethod
    def from_dense(w: torch.Tensor) -> "QuantWeight":
        from ..ops.quant import ref_quant_nvfp4_weights
        packed, sf, g = ref_quant_nvfp4_weights(w)
        return QuantWeight(packed, sf, g)


class Fp8Weight:
    """fp8-e4m3 weight of a linear layer with one fp32 scale per output channel (or per tensor),
    and optionally the checkpoint's static activation scale; without one the activations are
    quantised per call with their own maximum (W8A8 on the fp8 tensor cores either way).
    Reference: the FP8 W8A8 linear method of the 35B-A3B configuration
    (src/vt/cuda/cuda_matmul_fp8_cutlass.cu, QuantFp8StaticKernel + per-tensor scaled-mm)."""

    def __init__(self, w8, w_scale, input_scale=None):
        self.w8, self.w_scale, self.input_scale = w8, w_scale.float().contiguous(), input_scale
        self.shape = tuple(w8.shape)
        self.device = w8.device

    def numel(self):
        return self.w8.numel()

    def element_size(self):
        return 1

    def data_ptr(self):
        return self.w8.data_ptr()

    def dequant(self):
        s = self.w_scale.reshape(-1, 1) if self.w_scale.numel() > 1 else self.w_scale
        return (self.w8.float() * s).to(torch.bfloat16)

    @staticmethod
    def _grid_scales(wf: torch.Tensor, amax: torch.Tensor, scale: torch.Tensor):
        """Rows that were decoded from e4m3 (value = code x scale, rounded to bf16) get a scale that
        puts every element back on the e4m3 grid, so re-encoding returns the checkpoint's codes (times
        a power of two) instead of rounding a second time. The row maximum is some code m x 2^e with
        m in 8..15 times the unknown scale: each m is tried, and the one under which the whole row
        lands on the grid is kept. Rows of other origin (bf16 checkpoints) match no m and keep
        max / 448."""
        found = torch.zeros_like(amax, dtype=torch.bool)
        for m in (14, 15, 13, 12, 11, 10, 9, 8):         # 14 x 2^5 = 448: the plain choice comes first
            cand = (amax / (m * (32.0 if m <= 14 else 16.0))).clamp_min(1e-30)
            q = wf / cand[:, None]
            r = q.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
            ok = ((q - r).abs() <= q.abs() * 2.0 ** -6 + 2.0 ** -12).all(1) & ~found & (amax > 0)
            scale = torch.where(ok, cand, scale)
            found |= ok
        return scale, found

    @staticmethod
    def from_dense(w: torch.Tensor, per_channel: bool = True) -> "Fp8Weight":
        wf = w.float()
        amax = wf.abs().amax(1) if per_channel else wf.abs().max().reshape(1)
        scale = (amax / 448.0).clamp_min(1e-12)
        if per_channel and wf.shape[1] >= 64:
            # weights expanded from an fp8 checkpoint: recover its grid (a sample of rows tells
            # whether the search is worth running over the whole matrix)
            n = min(16, wf.shape[0])
            if bool(Fp8Weight._grid_scales(wf[:n], amax[:n], scale[:n])[1].any()):
                scale = Fp8Weight._grid_scales(wf, amax, scale)[0]
        w8 = (wf / (scale[:, None] if per_channel else scale)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        return Fp8Weight(w8.contiguous(), scale)


def fp8_quant_activations(a: torch.Tensor, input_scale=None):
    """The activation side of W8A8 restated in PyTorch (the CPU oracle of the fp8 path): the
    checkpoint's static per-tensor scale when it gives one, else one scale per token,
    max|row| / 448. Returns (e4m3 values, scale broadcastable over [T, N])."""
    af = a.float()
    if input_scale is not None:
        s = input_scale.float().reshape(())
    else:
        s = (af.abs().amax(-1, keepdim=True) / 448.0).clamp_min(1e-12 / 448.0)
    return (af * (1.0 / s)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn), s


class BlockQuantWeight:
    """A linear-layer weight kept in GGUF blocks of 32 values (Q8_0: fp16 scale + int8; Q4_0: fp16
    scale + nibbles) for the CPU backend's packed GEMM. Re-encoding a tensor that was decoded from
    the same format is lossless (the block maximum maps back to the same scale)."""

    def __init__(self, packed: torch.Tensor, kind: int, shape):
        self.packed, self.kind, self.shape = packed, kind, tuple(shape)
        self.device = packed.device

    @staticmethod
    def from_dense(w: torch.Tensor, fmt: str) -> "BlockQuantWeight":
        from ..ops import cpu_native as N
        kind = {"q8_0": N.Q8_0, "q4_0": N.Q4_0}[fmt]
        return BlockQuantWeight(N.quantize_blocks(w.float().cpu(), kind), kind, w.shape)

    def numel(self):
        return self.packed.numel()

    def element_size(self):
        return 1

    def data_ptr(self):
        return self.packed.data_ptr()

    def dequant(self) -> torch.Tensor:
        import numpy as np
        from ..loader.gguf import dequantize
        from ..ops import cpu_native as N
        t = {N.Q8_0: 8, N.Q4_0: 2}[self.kind]
        return torch.from_numpy(dequantize(self.packed.numpy().reshape(-1), t, self.shape)
                                .astype(np.float32)).to(torch.bfloat16)


_SHARED_SCRATCH: dict = {}


class FusedLinearMixin:
    """Producer + linear pairs the model code asks for by meaning. The default runs the two ops one
    after the other; the GPU back end overrides them where the linear layer takes quantised
    activations, so that the producer writes them directly (no bf16 round trip through HBM and one
    launch less). Reference: the quantise-once producers of the NVFP4 dense dispatch
    (src/vllm/model_executor/models/qwen3_5.cpp:1752-2055)."""

    def norm_gemm(self, hidden, ln_w, eps, w, out, *, residual=None, gemma=False, normed=None,
                  need_normed=False, bias=None):
        """out = RMSNorm(hidden (+ residual, updated in place)) @ w^T. ``normed``: a buffer for the
        normalised rows; they are only guaranteed to be written when ``need_normed`` (a fused
        path skips them otherwise). Returns (out, normalised rows or None)."""
        x = self.rmsnorm(hidden, ln_w, eps, residual=residual, out=normed, gemma=gemma)
        return self.gemm(x, w, bias=bias, out=out), x

    def act_gemm(self, gate_up, kind, w, out, *, act=None, interleaved=False):
        """out = (act(gate) * up) @ w^T for ``gate_up`` rows ``[gate | up]``."""
        a = self.act_and_mul(gate_up, kind, out=act, interleaved=interleaved)
        return self.gemm(a, w, out=out)

    def sigmoid_gate_gemm(self, x, gate, w, out):
        """out = (x * sigmoid(gate)) @ w^T (the output gate of gated attention)."""
        return self.gemm(self.sigmoid_mul(x, gate), w, out=out)


class CpuBackend(FusedLinearMixin):
    name = "cpu"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)

    def gemm(self, a, w, bias=None, residual=None, out=None, out_dtype=torch.bfloat16):
        if isinstance(w, Fp8Weight):
            # both operands in e4m3, products summed in fp32, scales applied to the sum
            a8, s = fp8_quant_activations(a, w.input_scale)
            ws = w.w_scale.reshape(1, -1) if w.w_scale.numel() > 1 else w.w_scale
            y = (a8.float() @ w.w8.float().t()) * s * ws
            if bias is not None:
                y = y + bias.float()
            y = y.to(torch.bfloat16)
            if residual is not None:
                y = (y.float() + residual.float()).to(torch.bfloat16)
            y = y.to(out_dtype)
        else:
            if isinstance(w, (QuantWeight, BlockQuantWeight)):
                w = w.dequant()
            y = ref.gemm(a, w, bias, residual, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def rmsnorm(self, x, w, eps, residual=None, out=None, gemma=False):
        y, newr = ref.rmsnorm(x, w, eps, residual, gemma)
        if residual is not None:
            residual.copy_(newr)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def layernorm(self, x, w, b, eps):
        return ref.layernorm(x, w, b, eps)

    def act_and_mul(self, x, kind=0, out=None, interleaved=False):
        assert not interleaved, "the interleaved gate / up layout is GPU-only"
        return ref.act_and_mul(x, kind)

    def embedding(self, ids, table, out=None, vocab_start=0, vocab_total=None, scale=1.0):
        local = ids - vocab_start
        ok = (local >= 0) & (local < table.shape[0])
        y = table[local.clamp(0, table.shape[0] - 1)]
        y = torch.where(ok[:, None], y, torch.zeros_like(y))
        if scale != 1.0:
            y = (y.float() * scale).to(table.dtype)
        return y

    def gather_rows(self, x, idx, out=None):
        return x[idx.long()]

    def rope_table(self, inv_freq, max_pos, mscale=1.0):
        return ref.rope_table(inv_freq.to(self.device), max_pos, mscale)

    def rope_kv(self, qkv, positions, table, *, num_q_heads, num_kv_heads, head_dim, rot_dim,
                neox, q_norm, k_norm, eps, gemma, slot_mapping, kv_cache, block_size,
                q_head_stride=None, offsets=None):
        q, k, v = ref.rope_kv(qkv, positions, table, num_q_heads, num_kv_heads, head_dim, rot_dim,
                              neox, q_norm, k_norm, eps, gemma)
        T = qkv.shape[0]
        qkv[:, : num_q_heads * head_dim] = q.reshape(T, -1).clone()
        if kv_cache is not None:
            ref.write_kv_cache(kv_cache, k, v, slot_mapping, block_size)

    def attention(self, q, kv_cache, ctx, group, *, num_q_heads, num_kv_heads, head_dim,
                  block_size, scale, out=None, softcap=0.0, window=0):
        y = ref.paged_attention(q, kv_cache, ctx.block_table[group], ctx.seq_lens,
                                ctx.query_start, num_q_heads, num_kv_heads, head_dim, block_size,
                                scale, softcap, window)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def add(self, a, b):
        return (a.float() + b.float()).to(a.dtype)

    def mul_scalar(self, a, s):
        return (a.float() * s).to(a.dtype)

    def softcap(self, a, cap):
        return (cap * torch.tanh(a.float() / cap)).to(a.dtype)

    def sigmoid_mul(self, a, g):
        return (a.float() * torch.sigmoid(g.float())).to(a.dtype)

    def argmax(self, logits):
        return logits.argmax(-1)


class CpuNativeBackend(CpuBackend):
    """The CPU execution path proper: the C++ thread-pool backend (``csrc/cpu``) for the ops of
    a decoder forward pass; anything it does not cover falls through to the oracle."""
    name = "cpu-native"

    def __init__(self, device="cpu"):
        super().__init__(device)
        from ..ops import cpu_native
        self.n = cpu_native
        cpu_native.lib()
        # The heavy ops run on the native pool; what is left to PyTorch here is small (index ops,
        # the sampler). Its OpenMP workers keep spinning for a while after every op and take cores
        # from the pool (a 0.6B decode step: 71 ms with them, 49 ms without), so PyTorch gets one
        # thread once a native back end exists. B200_TORCH_THREADS=n keeps n (0: leave it alone).
        n = os.environ.get("B200_TORCH_THREADS", "1")
        if n.isdigit() and int(n) > 0:
            torch.set_num_threads(int(n))

    def gemm(self, a, w, bias=None, residual=None, out=None, out_dtype=torch.bfloat16):
        if isinstance(w, BlockQuantWeight) and a.dtype == torch.bfloat16 and a.stride(-1) == 1 \
                and w.shape[1] % 32 == 0:
            # weights stay packed: int8 block dot products against per-block quantised activations
            y = self.n.gemm_quant(a, w.packed, w.kind, out_dtype=torch.float32)
            if bias is not None:
                y = y + bias.float()
            if residual is not None:
                y = y + residual.float()
            y = y.to(out.dtype if out is not None else out_dtype)
            if out is not None:
                out.copy_(y)
                return out
            return y
        if isinstance(w, (QuantWeight, BlockQuantWeight, Fp8Weight)) or a.dtype != torch.bfloat16 \
                or a.stride(-1) != 1:
            return super().gemm(a, w, bias, residual, out, out_dtype)
        return self.n.gemm(a, w, bias, residual, out, out.dtype if out is not None else out_dtype)

    def rmsnorm(self, x, w, eps, residual=None, out=None, gemma=False):
        if x.dtype != torch.bfloat16 or (out is not None and out.data_ptr() == x.data_ptr()):
            return super().rmsnorm(x, w, eps, residual, out, gemma)
        return self.n.rmsnorm(x, w, eps, residual, out, gemma)

    def act_and_mul(self, x, kind=0, out=None, interleaved=False):
        assert not interleaved
        if x.dtype != torch.bfloat16:
            return super().act_and_mul(x, kind, out)
        return self.n.act_and_mul(x, kind, out)

    def embedding(self, ids, table, out=None, vocab_start=0, vocab_total=None, scale=1.0):
        if table.dtype != torch.bfloat16:
            return super().embedding(ids, table, out, vocab_start, vocab_total, scale)
        return self.n.embedding(ids, table, out, vocab_start, scale)

    def rope_kv(self, qkv, positions, table, *, num_q_heads, num_kv_heads, head_dim, rot_dim,
                neox, q_norm, k_norm, eps, gemma, slot_mapping, kv_cache, block_size,
                q_head_stride=None, offsets=None):
        if qkv.dtype != torch.bfloat16 or q_head_stride is not None or offsets is not None:
            return super().rope_kv(qkv, positions, table, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                                   head_dim=head_dim, rot_dim=rot_dim, neox=neox, q_norm=q_norm, k_norm=k_norm,
                                   eps=eps, gemma=gemma, slot_mapping=slot_mapping, kv_cache=kv_cache,
                                   block_size=block_size)
        self.n.rope_kv(qkv, positions, table, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                       head_dim=head_dim, rot_dim=rot_dim, neox=neox, q_norm=q_norm, k_norm=k_norm, eps=eps,
                       gemma=gemma, slot_mapping=slot_mapping, kv_cache=kv_cache, block_size=block_size)

    def attention(self, q, kv_cache, ctx, group, *, num_q_heads, num_kv_heads, head_dim,
                  block_size, scale, out=None, softcap=0.0, window=0):
        if q.dtype != torch.bfloat16 or q.stride(-1) != 1:
            return super().attention(q, kv_cache, ctx, group, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                                     head_dim=head_dim, block_size=block_size, scale=scale, out=out,
                                     softcap=softcap, window=window)
        return self.n.paged_attention(q, kv_cache, ctx.block_table[group], ctx.seq_lens, ctx.query_start,
                                      num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                                      block_size=block_size, scale=scale, softcap=softcap, window=window,
                                      out=out)


class GpuBackend(FusedLinearMixin):
    name = "cuda"

    def __init__(self, device="cuda"):
        from .. import ops
        self.ops = ops
        self.device = torch.device(device)
        ops.lib()  # fail loudly here if the kernel library is missing
        # NVFP4 weights: "bf16" keeps activations in bf16 (W4A16), "nvfp4" quantises them per call
        # and runs W4A4 on kind::mxf4nvf4 (what NVFP4 checkpoints are calibrated for)
        self.w4a4 = os.environ.get("B200_NVFP4_ACTIVATIONS", "bf16") == "nvfp4"

    # ---- producers that write quantised activations directly -----------------------------------
    def _w4a4_ok(self, w, K):
        return isinstance(w, QuantWeight) and self.w4a4 and K % 256 == 0 and w.shape[0] % 8 == 0

    def norm_gemm(self, hidden, ln_w, eps, w, out, *, residual=None, gemma=False, normed=None,
                  need_normed=False, bias=None):
        from ..ops import quant as Q
        T, K = hidden.shape
        if T > 0 and hidden.stride(-1) == 1 and os.environ.get("B200_FUSED_PRODUCERS", "1") == "1":
            if self._w4a4_ok(w, K):
                g_a = w.act_gscale()
                keep = normed if need_normed else None
                ap, sfa = Q.rmsnorm_quant_nvfp4(hidden, ln_w, eps, g_a, residual=residual, gemma=gemma, swizzle=True,
                                                out=self._w4a4_buffers(T, K), normed=keep)
                y = Q.gemm_nvfp4(ap, sfa, g_a, w.packed, w.sf_chunks(), w.gscale, out=out, bias=bias)
                return y, keep
            if isinstance(w, Fp8Weight) and w.input_scale is None and not need_normed:
                a8, scales = self._fp8_buffer(T, K), self._fp8_row_scales(T)
                Q.quant_fp8_rowwise(hidden, out=a8, scales=scales, norm_weight=ln_w, eps=eps, gemma=gemma,
                                    residual=residual)
                return Q.gemm_fp8(a8, w.w8, scales, w.w_scale, out=out, bias=bias), None
        return super().norm_gemm(hidden, ln_w, eps, w, out, residual=residual, gemma=gemma, normed=normed,
                                 need_normed=need_normed, bias=bias)

    def act_gemm(self, gate_up, kind, w, out, *, act=None, interleaved=False):
        from ..ops import quant as Q
        T, K = gate_up.shape[0], gate_up.shape[1] // 2
        if T > 0 and gate_up.stride(-1) == 1 and os.environ.get("B200_FUSED_PRODUCERS", "1") == "1":
            if self._w4a4_ok(w, K) and kind == 0 and not interleaved:
                g_a = w.act_gscale()
                ap, sfa = Q.quant_nvfp4(gate_up, g_a, silu_mul=True, swizzle=True, out=self._w4a4_buffers(T, K))
                return Q.gemm_nvfp4(ap, sfa, g_a, w.packed, w.sf_chunks(), w.gscale, out=out)
            if isinstance(w, Fp8Weight) and w.input_scale is None and (not interleaved or K % 128 == 0):
                a8, scales = self._fp8_buffer(T, K), self._fp8_row_scales(T)
                Q.quant_fp8_rowwise(gate_up, out=a8, scales=scales, act_kind=kind, interleaved=interleaved)
                return Q.gemm_fp8(a8, w.w8, scales, w.w_scale, out=out)
        return super().act_gemm(gate_up, kind, w, out, act=act, interleaved=interleaved)

    def sigmoid_gate_gemm(self, x, gate, w, out):
        from ..ops import quant as Q
        T, K = x.shape
        if T > 0 and self._w4a4_ok(w, K) and x.stride(-1) == 1 and gate.stride(-1) == 1 \
                and os.environ.get("B200_FUSED_PRODUCERS", "1") == "1":
            g_a = w.act_gscale()
            ap, sfa = Q.quant_nvfp4_gated(x, gate, g_a, swizzle=True, out=self._w4a4_buffers(T, K))
            return Q.gemm_nvfp4(ap, sfa, g_a, w.packed, w.sf_chunks(), w.gscale, out=out)
        return super().sigmoid_gate_gemm(x, gate, w, out)

    def _fp8_row_scales(self, T: int):
        from .. import ops
        return ops.workspace(self.device, T * 4, "fp8_row_scales").view(torch.float32)[:T]

    def _fp8_buffer(self, T: int, K: int):
        """Persistent scratch of the fp8 activation quantiser."""
        from .. import ops
        return ops.workspace(self.device, T * K, "fp8_act")[: T * K].view(torch.float8_e4m3fn).view(T, K)

    def _w4a4_buffers(self, T: int, K: int):
        """Persistent (packed activations, scale chunks) scratch of the activation quantiser."""
        from .. import ops
        rows = (T + 127) // 128 * 128
        pk = ops.workspace(self.device, rows * (K // 2), "w4a4_act")
        sf = ops.workspace(self.device, rows * (K // 16), "w4a4_sf")
        return pk[: T * (K // 2)].view(T, K // 2), sf[: rows * (K // 16)]

    def gemm(self, a, w, bias=None, residual=None, out=None, out_dtype=torch.bfloat16):
        """``w`` is always a model weight here (never written by a kernel of the step), which
        lets the GEMM start fetching it before the previous kernel has finished."""
        if isinstance(w, Fp8Weight):
            from ..ops import quant as Q
            N, K = w.shape
            if a.stride(-1) != 1:
                a = a.contiguous()
            a8 = self._fp8_buffer(a.shape[0], K)
            if w.input_scale is not None:
                Q.quant_fp8(a, w.input_scale, out=a8)
                a_scale = w.input_scale
            else:
                scales = self._fp8_row_scales(a.shape[0])
                Q.quant_fp8_rowwise(a, out=a8, scales=scales)
                a_scale = scales
            y = Q.gemm_fp8(a8, w.w8, a_scale, w.w_scale, out=out, bias=bias)
            if residual is not None:
                y = self.ops.add(y, residual) if out is None else out.copy_(self.ops.add(y, residual))
            return y
        if isinstance(w, QuantWeight):
            from ..ops import quant as Q
            N, K = w.shape
            if self.w4a4 and K % 256 == 0 and N % 8 == 0 and a.stride(-1) == 1:
                # activations quantised to NVFP4 on the fly, both operands on the block-scaled MMA
                g_a = w.act_gscale()
                ap, sfa = Q.quant_nvfp4(a, g_a, swizzle=True, out=self._w4a4_buffers(a.shape[0], K))
                y = Q.gemm_nvfp4(ap, sfa, g_a, w.packed, w.sf_chunks(), w.gscale, out=out, bias=bias)
                if residual is not None:
                    y = self.ops.add(y, residual) if out is None else out.copy_(self.ops.add(y, residual))
                return y
            scratch = None
            if a.shape[0] > 128:
                # one expansion buffer per device, shared by every layer (stream ordered)
                key = (a.device, N * K)
                scratch = _SHARED_SCRATCH.get(key)
                if scratch is None:
                    scratch = torch.empty((N, K), dtype=torch.bfloat16, device=a.device)
                    _SHARED_SCRATCH[key] = scratch
            y = Q.gemm_w4a16(a, w.packed, w.sf, w.gscale, out=out, bias=bias, scratch=scratch)
            if residual is not None:
                y = self.ops.add(y, residual) if out is None else out.copy_(self.ops.add(y, residual))
            return y
        return self.ops.gemm(a, w, bias=bias, residual=residual, out=out, out_dtype=out_dtype, const_w=True)

    def rmsnorm(self, x, w, eps, residual=None, out=None, gemma=False):
        return self.ops.rmsnorm(x, w, eps, residual=residual, out=out, gemma=gemma)

    def layernorm(self, x, w, b, eps):
        return self.ops.layernorm(x, w, b, eps)

    def act_and_mul(self, x, kind=0, out=None, interleaved=False):
        return self.ops.act_and_mul(x, kind, out, interleaved=interleaved)

    def gemm_gated(self, a, w, kind=0, out=None, scratch=None):
        """act(a W_gate^T) * (a W_up^T) for an interleaved gate / up weight."""
        if isinstance(w, (QuantWeight, Fp8Weight)):
            y = self.gemm(a, w, out=scratch)
            return self.ops.act_and_mul(y, kind, out, interleaved=True)
        return self.ops.gemm_gated(a, w, kind, out=out, scratch=scratch)

    def embedding(self, ids, table, out=None, vocab_start=0, vocab_total=None, scale=1.0):
        return self.ops.embedding(ids, table, out=out, vocab_start=vocab_start,
                                  vocab_total=vocab_total, scale=scale)

    def gather_rows(self, x, idx, out=None):
        return self.ops.gather_rows(x, idx, out)

    def rope_table(self, inv_freq, max_pos, mscale=1.0):
        return self.ops.rope_table(inv_freq.to(self.device), max_pos, mscale)

    def rope_kv(self, qkv, positions, table, *, num_q_heads, num_kv_heads, head_dim, rot_dim,
                neox, q_norm, k_norm, eps, gemma, slot_mapping, kv_cache, block_size,
                q_head_stride=None, offsets=None):
        self.ops.rope_kv(qkv, positions, table, num_q_heads=num_q_heads,
                         num_kv_heads=num_kv_heads, head_dim=head_dim, rot_dim=rot_dim, neox=neox,
                         q_norm=q_norm, k_norm=k_norm, eps=eps, gemma=gemma,
                         slot_mapping=slot_mapping, kv_cache=kv_cache, block_size=block_size,
                         q_head_stride=q_head_stride, offsets=offsets)

    def attention(self, q, kv_cache, ctx, group, *, num_q_heads, num_kv_heads, head_dim,
                  block_size, scale, out=None, softcap=0.0, window=0):
        """Decode rows first (one token per request), then the prefill rows."""
        T = q.shape[0]
        if out is None:
            out = torch.empty((T, num_q_heads * head_dim), dtype=q.dtype, device=q.device)
        nd = ctx.num_decodes
        bt = ctx.block_table[group]
        if nd > 0:
            self.ops.attn_decode(q[:nd], kv_cache, block_table=bt[:nd], seq_lens=ctx.seq_lens[:nd],
                                 num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                                 head_dim=head_dim, block_size=block_size, scale=scale,
                                 out=out[:nd], splits=ctx.decode_splits, softcap=softcap,
                                 window=window, tmp=ctx.extra.get("decode_tmp"))
        if ctx.num_prefills > 0:
            self.ops.attn_prefill(q[nd:], kv_cache, block_table=bt[nd:], seq_lens=ctx.seq_lens[nd:],
                                  q_start=ctx.prefill_q_start, tile_req=ctx.tile_req[:ctx.num_tiles],
                                  tile_q0=ctx.tile_q0[:ctx.num_tiles], num_q_heads=num_q_heads,
                                  num_kv_heads=num_kv_heads, head_dim=head_dim,
                                  block_size=block_size, scale=scale, out=out[nd:],
                                  softcap=softcap, window=window)
        return out

    def add(self, a, b):
        return self.ops.add(a, b)

    def mul_scalar(self, a, s):
        return self.ops.mul_scalar(a, s)

    def softcap(self, a, cap):
        return self.ops.softcap(a, cap)

    def sigmoid_mul(self, a, g):
        return self.ops.sigmoid_mul(a, g)

    def argmax(self, logits):
        return self.ops.argmax(logits)


def make_backend(device) -> "CpuBackend | GpuBackend":
    device = torch.device(device)
    return GpuBackend(device) if device.type == "cuda" else CpuBackend(device)
