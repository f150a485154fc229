"""Attention backend registry: which kernel serves which (phase, layout, head size) and in which
order they are tried. One table instead of conditions spread over the call sites; the dispatchers
in ``ops`` and the model backends ask it, ``describe()`` prints what a model will run on.

Reference: the attention backend selector and its priority list
(``src/vllm/v1/attention/selector.cpp``, ``include/vllm/v1/attention/backends/registry.h``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional


@dataclass(frozen=True)
class AttentionBackend:
    name: str
    phase: str                      # "decode" | "prefill"
    kind: str                       # "paged" (full / sliding / chunked-local GQA), "mla", "gdn"
    priority: int                   # lower is tried first
    kernel: str                     # the launcher behind it
    supports: Callable[..., bool]

    def __repr__(self):
        return f"<{self.name}: {self.phase} {self.kind} -> {self.kernel}>"


def _pages_tile(block_size: int, tile: int) -> bool:
    if block_size < 8 or block_size % 8:
        return False
    return (tile % block_size == 0) if block_size <= tile else (block_size % tile == 0)


REGISTRY: list[AttentionBackend] = [
    AttentionBackend("tcgen05-decode", "decode", "paged", 0, "b200_attn_decode_tc",
                     lambda head_dim, group, block_size, **_: head_dim in (128, 256) and group <= 16
                     and _pages_tile(block_size, 128)),
    AttentionBackend("cuda-core-decode", "decode", "paged", 1, "b200_attn_decode",
                     lambda head_dim, **_: head_dim in (64, 128, 256)),
    AttentionBackend("tcgen05-prefill", "prefill", "paged", 0, "b200_attn_prefill",
                     lambda head_dim, block_size, **_: head_dim in (64, 128, 256) and _pages_tile(block_size, 64)),
    AttentionBackend("mla-absorbed-decode", "decode", "mla", 0, "b200_mla_decode",
                     lambda num_heads, block_size, **_: 1 <= num_heads <= 16 and _pages_tile(block_size, 128)),
    AttentionBackend("mla-expanded-prefill", "prefill", "mla", 0, "b200_attn_prefill (head_dim 256 over expanded K/V)",
                     lambda **_: True),
    AttentionBackend("gdn-packed-decode", "decode", "gdn", 0, "b200_gdn_packed_decode",
                     lambda head_dim=128, **_: head_dim == 128),
    AttentionBackend("gdn-chunk-scan", "prefill", "gdn", 0, "b200_gdn_chunk_scan",
                     lambda head_dim=128, **_: head_dim == 128),
]


def candidates(phase: str, kind: str = "paged") -> list[AttentionBackend]:
    return sorted((b for b in REGISTRY if b.phase == phase and b.kind == kind), key=lambda b: b.priority)


def select(phase: str, kind: str = "paged", *, exclude: tuple = (), **features) -> Optional[AttentionBackend]:
    """First backend of the priority list whose ``supports`` accepts the features
    (head_dim, group, block_size, num_heads ...); None when nothing does."""
    for b in candidates(phase, kind):
        if b.name in exclude:
            continue
        try:
            if b.supports(**features):
                return b
        except TypeError:
            continue
    return None


def describe(cfg, block_size: int) -> dict:
    """Backends a model configuration resolves to, per layer kind and phase."""
    out = {}
    if getattr(cfg, "kv_lora_rank", 0):
        out["mla"] = {p: getattr(select(p, "mla", num_heads=cfg.num_heads, block_size=block_size), "name", None)
                      for p in ("decode", "prefill")}
    else:
        group = max(1, cfg.num_heads // max(1, cfg.num_kv_heads))
        out["paged"] = {p: getattr(select(p, "paged", head_dim=cfg.head_dim, group=group, block_size=block_size),
                                   "name", None) for p in ("decode", "prefill")}
    if getattr(cfg, "layer_types", None) and "linear_attention" in cfg.layer_types:
        out["gdn"] = {p: getattr(select(p, "gdn"), "name", None) for p in ("decode", "prefill")}
    return out
