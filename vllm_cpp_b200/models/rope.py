"""Rotary-embedding family: inverse frequencies + magnitude scale per variant, computed once
on the host in fp64; the cos/sin table itself is built on the device by ``ops.rope_table``
(or ``reference.rope_table`` on CPU) and every layer reads it by position.

Variants and their reference restatements: base (``layers/rotary_embedding/base.cpp``),
Llama-3 banded scaling (``llama3_rope.cpp:34-62``), YaRN and the DeepSeek variant with
mscale (``yarn_scaling_rope.cpp``; softmax scale correction ``mla_attention.cpp:136-139``),
linear / dynamic-NTK (``dynamic_ntk_scaling_rope.cpp``, ``dynamic_ntk_alpha_rope.cpp``),
Phi-3 LongRoPE short/long factors (``phi3_long_rope_scaled_rope.cpp``), MRoPE sections
(``mrope.cpp``; text-only requests use identical t/h/w positions, so it reduces to base).
"""
from __future__ import annotations

import math

import torch

from ..config import RopeConfig


def _base_inv_freq(rot: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))


def yarn_get_mscale(scale: float, mscale: float = 1.0) -> float:
    if scale <= 1.0:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


def _yarn_find_correction_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_correction_range(low_rot, high_rot, dim, base, max_pos, truncate=True):
    low = _yarn_find_correction_dim(low_rot, dim, base, max_pos)
    high = _yarn_find_correction_dim(high_rot, dim, base, max_pos)
    if truncate:
        low, high = math.floor(low), math.ceil(high)
    return max(low, 0), min(high, dim - 1)


def _yarn_linear_ramp(lo, hi, n):
    if lo == hi:
        hi += 0.001
    r = (torch.arange(n, dtype=torch.float64) - lo) / (hi - lo)
    return r.clamp(0, 1)


def rope_parameters(cfg: RopeConfig, head_dim: int, max_position: int):
    """Returns ``(inv_freq fp64 [rot/2], table_mscale, table_len)``."""
    rot = cfg.rotary_dim or head_dim
    inv = _base_inv_freq(rot, cfg.theta)
    mscale = 1.0
    table_len = max_position
    t = cfg.scaling_type
    if t in (None, "default", "mrope"):
        pass
    elif t == "linear":
        inv = inv / cfg.factor
    elif t == "llama3":
        low_wl = cfg.original_max_position / cfg.low_freq_factor
        high_wl = cfg.original_max_position / cfg.high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (cfg.original_max_position / wl - cfg.low_freq_factor) / (
            cfg.high_freq_factor - cfg.low_freq_factor)
        scaled = torch.where(wl > low_wl, inv / cfg.factor, inv)
        mid = (1 - smooth) * inv / cfg.factor + smooth * inv
        is_mid = (wl >= high_wl) & (wl <= low_wl)
        inv = torch.where(is_mid, mid, scaled)
    elif t in ("yarn", "deepseek_yarn"):
        extrap = inv
        interp = inv / cfg.factor
        # upstream's multimodal (sectioned) rotary class takes the correction range over the whole
        # head width, its plain YaRN class over the rotated width; they only differ with partial rotation
        lo, hi = _yarn_correction_range(cfg.beta_fast, cfg.beta_slow, head_dim if cfg.mrope_section else rot,
                                        cfg.theta, cfg.original_max_position, cfg.truncate)
        mask = (1 - _yarn_linear_ramp(lo, hi, rot // 2)) * cfg.extrapolation_factor
        inv = interp * (1 - mask) + extrap * mask
        if not cfg.apply_yarn_scaling:
            mscale = cfg.attn_factor
        elif t == "deepseek_yarn":
            mscale = (yarn_get_mscale(cfg.factor, cfg.mscale) /
                      yarn_get_mscale(cfg.factor, cfg.mscale_all_dim)) * cfg.attn_factor
        else:
            mscale = yarn_get_mscale(cfg.factor) * cfg.attn_factor
        table_len = max(table_len, int(cfg.original_max_position * cfg.factor))
    elif t == "dynamic":
        if cfg.alpha is not None:
            base = cfg.theta * cfg.alpha ** (rot / (rot - 2))
        else:
            max_len = cfg.original_max_position * cfg.factor
            base = cfg.theta * ((cfg.factor * max_len / cfg.original_max_position) -
                                (cfg.factor - 1)) ** (rot / (rot - 2))
        inv = _base_inv_freq(rot, base)
    elif t in ("longrope", "su"):
        # The long factors apply once the context exceeds the original window; the engine
        # sizes the table for max_position, so pick by that.
        use_long = max_position > cfg.original_max_position
        f = cfg.long_factor if use_long else cfg.short_factor
        if f is not None:
            inv = inv / torch.tensor(f, dtype=torch.float64)
        # the magnitude correction follows the checkpoint's declared window, whatever length this
        # engine was sized for (and applies to the short factors too)
        scale = (cfg.config_max_position or max_position) / cfg.original_max_position
        mscale = 1.0 if scale <= 1.0 else math.sqrt(
            1 + math.log(scale) / math.log(cfg.original_max_position))
        given = cfg.long_mscale if use_long else cfg.short_mscale
        if given is not None:
            mscale = float(given)
    else:
        raise ValueError(f"unknown rope scaling type {t}")
    return inv, float(mscale), int(table_len)


def softmax_scale(cfg: RopeConfig, qk_head_dim: int) -> float:
    """Attention softmax scale; DeepSeek-YaRN multiplies by mscale_all_dim squared."""
    s = qk_head_dim ** -0.5
    if cfg.scaling_type == "deepseek_yarn" and cfg.mscale_all_dim:
        m = yarn_get_mscale(cfg.factor, cfg.mscale_all_dim)
        s = s * m * m
    return s


def mrope_positions(positions: torch.Tensor) -> torch.Tensor:
    """Text-only MRoPE: the three position streams coincide."""
    return positions.unsqueeze(0).expand(3, -1)


def mrope_cos_sin(table: torch.Tensor, positions: torch.Tensor, sections, interleaved: bool = False):
    """cos / sin rows [T, rot/2] for sectioned rotary positions. ``table`` [max_pos, rot] holds
    [cos | sin] per position; ``positions`` is [T] (text: one stream) or [3, T] (temporal, height,
    width); ``sections`` gives how many of the rot/2 frequencies follow each stream. Contiguous
    layout: the first ``sections[0]`` frequencies take the temporal position, the next the
    height, the rest the width. Interleaved layout: frequency i takes stream i % 3 while that
    stream still has frequencies left (i < 3 * sections[stream]), else the temporal one.
    Reference: src/vllm/model_executor/layers/rotary_embedding/mrope.cpp."""
    half = table.shape[1] // 2
    if positions.dim() == 1:
        rows = table[positions]
        return rows[:, :half], rows[:, half:]
    assert positions.shape[0] == 3 and sum(sections) == half
    per = table[positions]                                   # [3, T, rot]
    stream = torch.zeros(half, dtype=torch.long)
    if interleaved:
        for i in range(half):
            st = i % 3
            stream[i] = st if (st > 0 and i < 3 * sections[st]) else 0
    else:
        stream = torch.repeat_interleave(torch.arange(3), torch.tensor(list(sections)))
    idx = stream.to(table.device)
    f = torch.arange(half, device=table.device)
    cos = per[idx, :, f].t()                                 # [T, half]
    sin = per[idx, :, half + f].t()
    return cos, sin
