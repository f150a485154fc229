"""Shared model plumbing: the per-step context handed to ``forward`` and helpers for
weight creation / sharding.

Reference: ``include/vllm/model_executor/models/model_registry.h:100-116`` (ModelForwardInput)
and ``dense_attn_block.h:242-307`` (once-per-step device inputs).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class StepContext:
    """Device-resident inputs of one engine step (views into the packed step buffer)."""
    num_tokens: int
    num_reqs: int
    num_decodes: int            # requests; decode requests come first, one token each
    num_prefills: int
    num_prefill_tokens: int
    num_tiles: int
    num_logits: int
    input_ids: torch.Tensor     # int64 [T]
    positions: torch.Tensor     # int64 [T]
    slot_mapping: list          # per KV group: int64 [T]
    query_start: torch.Tensor   # int32 [R+1]
    seq_lens: torch.Tensor      # int32 [R]
    block_table: list           # per KV group: int32 [R, max_blocks]
    logits_indices: torch.Tensor  # int32 [num_logits]
    tile_req: torch.Tensor      # int32 [num_tiles]
    tile_q0: torch.Tensor
    prefill_q_start: torch.Tensor  # int32 [P+1]
    state_slots: torch.Tensor   # int32 [R]
    decode_splits: int = 1
    max_seq_len: int = 0
    max_query_len: int = 0
    decode_only_full_logits: bool = False   # decode-only batch: logits for every row
    extra: dict = field(default_factory=dict)


def normal_(shape, std, device, dtype, gen) -> torch.Tensor:
    """Random-init weight drawn on the CPU generator (identical across ranks/devices for a
    given seed) and moved to ``device``."""
    w = torch.empty(shape, dtype=torch.float32)
    w.normal_(0.0, std, generator=gen)
    return w.to(dtype).to(device)


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n].contiguous()


class BufferPool:
    """Persistent activation buffers keyed by name; grown on demand, never shrunk. A buffer that
    is outgrown is kept alive (a CUDA graph captured earlier still holds its address)."""

    def __init__(self, device):
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []
        if torch.device(device).type == "cuda":
            from .. import ops
            ops.init_device(torch.device(device))

    def get(self, name: str, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        b = self._bufs.get(name)
        if b is None or b.shape[0] < rows or b.shape[1] != cols or b.dtype != dtype:
            cap = rows if b is None else max(rows, b.shape[0])
            if b is not None:
                self._retired.append(b)
            b = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._bufs[name] = b
        return b[:rows]

    def reserve(self, name: str, rows: int, cols: int, dtype=torch.bfloat16) -> None:
        self.get(name, rows, cols, dtype)
