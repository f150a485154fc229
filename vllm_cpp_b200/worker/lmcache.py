"""KV chunks of a request <-> an LMCache remote server (``lm://host:port``).

``LMCacheStore`` turns the paged KV cache of the attention layers into LMCache chunks: the
prompt is cut into chunks of ``chunk_size`` tokens, each keyed by the rolling BLAKE3 hash of
everything up to and including it (so a key identifies a whole prefix), and each chunk's KV is
sent in the ``KV_2LTD`` layout ``[2, layers, tokens, kv_heads * head_dim]``. ``lookup`` counts how
many leading tokens the server already holds, ``load`` writes them back into freshly allocated
blocks. The wire format, hashing and key strings live in C++ (``csrc/engine/offload/lmcache.*``).

Reference: ``src/vllm/v1/kv_offload/lmcache/lmcache_connector.cpp``,
``chunked_token_database.cpp``.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import _engine as E

lm = E.lmcache

_DTYPES = {torch.bfloat16: lm.Dtype.BFLOAT16, torch.float16: lm.Dtype.FLOAT16, torch.float32: lm.Dtype.FLOAT32}


def parse_url(url: str) -> tuple[str, int]:
    """``lm://host:port`` -> (host, port)."""
    if not url.startswith("lm://"):
        raise ValueError(f"not an LMCache url: {url!r}")
    host, _, port = url[5:].rpartition(":")
    if not host or not port.isdigit():
        raise ValueError(f"LMCache url needs host:port: {url!r}")
    return host, int(port)


class LMCacheStore:
    def __init__(self, url: str, model_name: str, kv_caches: Sequence[torch.Tensor], block_size: int,
                 chunk_size: int = 256, world_size: int = 1, worker_id: int = 0, connect: bool = True,
                 hash_algo: str = "blake3"):
        """``kv_caches``: one ``[num_blocks, 2, block_size, Hkv, D]`` tensor per attention layer."""
        host, port = parse_url(url)
        self.client = lm.RemoteClient(host, port)
        if connect:
            self.client.connect()
        # "blake3": LMCache's own rolling chunk hash; "vllm": the sha256_cbor chain a vLLM +
        # LMCache peer keys on (ChunkedTokenDatabase), so that both sides hit each other's chunks
        if hash_algo not in ("blake3", "vllm"):
            raise ValueError(f"unknown LMCache hash_algo {hash_algo!r}")
        self.hash_algo = hash_algo
        self.hasher = lm.TokenHasher(chunk_size)
        self.model_name, self.world_size, self.worker_id = model_name, world_size, worker_id
        self.kv_caches = list(kv_caches)
        self.block_size, self.chunk_size = block_size, chunk_size
        c = self.kv_caches[0]
        self.hidden = c.shape[3] * c.shape[4]
        self.dtype = _DTYPES[c.dtype]
        self.elem = c.element_size()
        self.stats = {"put_chunks": 0, "hit_chunks": 0, "miss_chunks": 0}

    # ------------------------------------------------------------------ keys
    def chunk_keys(self, token_ids: Sequence[int]) -> list[str]:
        toks = [int(t) & 0xFFFFFFFF for t in token_ids]
        if self.hash_algo == "vllm":
            hashes = [h for _, _, h in lm.vllm_chunk_hashes(toks, self.chunk_size)]
        else:
            hashes = [lm.TokenHasher.fold(d) for d in self.hasher.chunk_hashes(toks)]
        return [lm.CacheKey(self.model_name, self.world_size, self.worker_id, h, self.dtype).to_string()
                for h in hashes]

    # ------------------------------------------------------------------ paged cache <-> planes
    def _slots(self, block_ids: Sequence[int], start: int, end: int) -> torch.Tensor:
        pos = torch.arange(start, end)
        blocks = torch.tensor(list(block_ids), dtype=torch.int64)
        return blocks[pos // self.block_size] * self.block_size + pos % self.block_size

    def _gather(self, block_ids, start, end):
        slots = self._slots(block_ids, start, end)
        k_planes, v_planes = [], []
        for cache in self.kv_caches:
            nb, _, bs, h, d = cache.shape
            flat = cache.view(nb, 2, bs, h * d)
            idx = slots.to(cache.device)
            k = flat[:, 0].reshape(nb * bs, h * d)[idx].cpu().contiguous()
            v = flat[:, 1].reshape(nb * bs, h * d)[idx].cpu().contiguous()
            k_planes.append(bytes(k.view(torch.uint8).numpy().tobytes()))
            v_planes.append(bytes(v.view(torch.uint8).numpy().tobytes()))
        return k_planes, v_planes

    def _scatter(self, block_ids, start, end, k_planes, v_planes):
        slots = self._slots(block_ids, start, end)
        for cache, kb, vb in zip(self.kv_caches, k_planes, v_planes):
            nb, _, bs, h, d = cache.shape
            k = torch.frombuffer(bytearray(kb), dtype=torch.uint8).view(cache.dtype).view(end - start, h, d)
            v = torch.frombuffer(bytearray(vb), dtype=torch.uint8).view(cache.dtype).view(end - start, h, d)
            idx = slots.to(cache.device)
            b, o = idx // bs, idx % bs
            cache[b, 0, o] = k.to(cache.device)
            cache[b, 1, o] = v.to(cache.device)

    # ------------------------------------------------------------------ store / lookup / load
    def store(self, token_ids: Sequence[int], block_ids: Sequence[int], skip_chunks: int = 0) -> int:
        """Sends every complete chunk of the request (after the first ``skip_chunks``); returns
        the number of chunks sent."""
        keys = self.chunk_keys(token_ids)
        L, C = len(self.kv_caches), self.chunk_size
        sent = 0
        for i, key in enumerate(keys):
            if i < skip_chunks or self.client.exist(key):
                continue
            k, v = self._gather(block_ids, i * C, (i + 1) * C)
            payload = lm.pack_kv2ltd(L, C, self.hidden, self.elem, k, v)
            self.client.put(key, payload, lm.MemFormat.KV_2LTD, self.dtype, [2, L, C, self.hidden])
            sent += 1
        self.stats["put_chunks"] += sent
        return sent

    def lookup(self, token_ids: Sequence[int]) -> int:
        """Number of leading tokens whose KV the server holds (a multiple of the chunk size)."""
        n = 0
        for key in self.chunk_keys(token_ids):
            if not self.client.exist(key):
                break
            n += self.chunk_size
        return n

    def load(self, token_ids: Sequence[int], block_ids: Sequence[int], num_tokens: int) -> int:
        """Fetches the first ``num_tokens`` tokens' KV into the request's blocks; returns how many
        tokens were actually loaded (a chunk that has vanished ends the prefix)."""
        keys = self.chunk_keys(token_ids)[: num_tokens // self.chunk_size]
        L, C = len(self.kv_caches), self.chunk_size
        done = 0
        for i, key in enumerate(keys):
            got = self.client.get(key)
            if got is None:
                self.stats["miss_chunks"] += 1
                break
            data, fmt, dtype, shape = got
            if fmt != lm.MemFormat.KV_2LTD or dtype != self.dtype or list(shape) != [2, L, C, self.hidden]:
                raise ValueError(f"LMCache chunk {key} has layout {fmt} {dtype} {shape}, expected "
                                 f"KV_2LTD {self.dtype} {[2, L, C, self.hidden]}")
            k, v = lm.unpack_kv2ltd(L, C, self.hidden, self.elem, data)
            self._scatter(block_ids, i * C, (i + 1) * C, k, v)
            self.stats["hit_chunks"] += 1
            done += C
        return done


class LMCacheConnector(E.KVConnectorHook):
    """Scheduler-side KV connector over an :class:`LMCacheStore` (synchronous loads).

    At admission the scheduler asks how many tokens beyond its own prefix-cache hit the server
    holds; after the blocks are allocated the load is queued and ``run_step_plan`` (called by the
    runner before the forward pass) fills them; a finished request's complete chunks are stored.
    Configuration: ``EngineArgs.kv_transfer_config = {"kv_connector": "LMCacheConnector",
    "url": "lm://host:port", "chunk_size": 256, "hash_algo": "blake3" | "vllm",
    "model_name": ...}``; the chunk size must be a multiple of the KV block size.

    Reference: ``src/vllm/v1/kv_offload/lmcache/lmcache_connector.cpp``.
    """

    def __init__(self, store: LMCacheStore):
        super().__init__()
        if store.chunk_size % store.block_size:
            raise ValueError("LMCache chunk_size must be a multiple of the KV block size")
        self.store = store
        self._loads: list = []
        self._lookups: dict[str, int] = {}
        self.loaded_tokens = 0
        self.stored_chunks = 0

    @property
    def connector(self):          # same attribute the offload worker exposes to the engine
        return self

    # ---- scheduler hooks (plain data in, see the C++ trampoline)
    def get_num_new_matched_tokens(self, req_id, token_ids, num_computed):
        # at least one token of the request must still be computed locally
        have = self.store.lookup(token_ids[: len(token_ids) - 1])
        self._lookups[req_id] = have
        return (max(0, have - num_computed), False)

    def update_state_after_alloc(self, req_id, token_ids, block_ids, num_external_tokens):
        have = self._lookups.pop(req_id, 0)
        if num_external_tokens > 0 and have > 0:
            self._loads.append((list(token_ids), list(block_ids[0]), have))

    def build_connector_meta(self):
        return None

    def request_finished(self, req_id, token_ids, block_ids, num_computed_tokens):
        # KV exists for the computed tokens only (the last sampled token has none yet)
        n = min(int(num_computed_tokens), len(token_ids))
        if n >= self.store.chunk_size:
            self.stored_chunks += self.store.store(list(token_ids[:n]), list(block_ids[0]))
        return False

    # ---- worker hook
    def run_step_plan(self) -> None:
        loads, self._loads = self._loads, []
        for token_ids, blocks, n in loads:
            self.loaded_tokens += self.store.load(token_ids, blocks, n)
