"""NVTX ranges for the forward pass (per step, per layer, per block of a layer), switched on
with ``B200_NVTX=1`` so that an external profiler can attribute kernels to layers. Off by
default: ``range()`` then returns one shared no-op context manager."""
from __future__ import annotations

import contextlib
import os

ENABLED = os.environ.get("B200_NVTX", "0") == "1"
_NULL = contextlib.nullcontext()


def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    if not ENABLED:
        return _NULL
    import torch
    return torch.cuda.nvtx.range(name)
