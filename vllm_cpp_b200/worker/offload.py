"""Worker half of KV offloading: owns the pinned host pool and executes the copy plan the
scheduler-side connector builds each step (stores of finished requests' blocks first, then
loads into freshly allocated blocks), one strided copy per layer and direction.

Configuration (``EngineArgs.kv_transfer_config``):
``{"kv_connector": "OffloadingConnector", "cpu_blocks": 1024, "policy": "lru" | "arc",
"fs_dir": "/path" (optional disk tier), "fs_max_bytes": 0}``.

Reference: ``include/vllm/v1/kv_offload/kv_block_transfer.h``, ``include/vllm/config/kv_transfer.h``.
"""
from __future__ import annotations

import torch

from .. import _engine as E


class KVOffloadWorker:
    def __init__(self, kv_caches: list, block_size: int, config: dict, model_id: str = "model"):
        name = config.get("kv_connector", "OffloadingConnector")
        if name not in ("OffloadingConnector", "CPUOffloadingConnector"):
            raise ValueError(f"unknown kv_connector {name!r}")
        self.kv_caches = list(kv_caches)           # per layer: [num_blocks, ...]
        self.block_size = block_size
        self.layer_bytes = [c[0].numel() * c.element_size() for c in self.kv_caches]
        self.block_bytes = sum(self.layer_bytes)
        self.slots = int(config.get("cpu_blocks", 256))
        dev = self.kv_caches[0].device
        self.host = torch.zeros((self.slots, self.block_bytes), dtype=torch.uint8,
                                pin_memory=dev.type == "cuda")
        self._views = []
        off = 0
        for c, nb in zip(self.kv_caches, self.layer_bytes):
            self._views.append(self.host[:, off:off + nb])
            off += nb
        fs_dir = config.get("fs_dir")
        ident = E.CacheIdentity(model_id, block_size, self.block_bytes, str(self.kv_caches[0].dtype)) \
            if fs_dir else None
        self.tiers = E.TieringManager(self.slots, config.get("policy", "lru"), self.host.data_ptr(),
                                      self.block_bytes, fs_dir, ident, int(config.get("fs_max_bytes", 0)))
        self.connector = E.OffloadConnector(self.tiers, block_size)
        self.loaded_blocks = 0
        self.stored_blocks = 0

    def _copy(self, transfers, to_host: bool) -> None:
        if not transfers:
            return
        slots = torch.tensor([t.cpu_slot for t in transfers], dtype=torch.long)
        blocks = torch.tensor([t.gpu_block for t in transfers], dtype=torch.long)
        dev = self.kv_caches[0].device
        for cache, view in zip(self.kv_caches, self._views):
            flat = cache.view(cache.shape[0], -1).view(torch.uint8)
            if to_host:
                view[slots] = flat[blocks.to(dev)].cpu()
            else:
                flat[blocks.to(dev)] = view[slots].to(dev, non_blocking=True)

    def run_step_plan(self) -> None:
        """Called by the runner before the forward pass of a step."""
        meta = self.connector.take_meta()
        if meta is None or (not meta.loads and not meta.stores):
            return
        self._copy(meta.stores, True)
        self._copy(meta.loads, False)
        if self.kv_caches[0].device.type == "cuda":
            torch.cuda.current_stream().synchronize() if meta.stores else None
        self.stored_blocks += len(meta.stores)
        self.loaded_blocks += len(meta.loads)
        self.connector.transfers_done(meta)
