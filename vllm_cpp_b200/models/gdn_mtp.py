"""Multi-token-prediction draft head of the Qwen3.5 / 3.6 / Qwen3-Next hybrids, wired as a drafter.

The head continues from the trunk: for a position p it takes the trunk's final hidden state at p
and the embedding of the token at p + 1, normalises each (Gemma-style 1 + w), concatenates them,
projects back to the hidden width (``mtp.fc``), runs ``mtp.layers`` (full-attention decoder blocks
of the trunk's kind, with their own KV cache) and ``mtp.norm``, and reads the trunk's ``lm_head``:
the result predicts the token at p + 2. Embedding and lm_head are the trunk's tensors.

The decoder blocks are an instance of the trunk's own model class over a configuration that has
only those layers, so every kernel, the paged KV cache and chunked prefill behave as in the trunk;
the head only replaces the input rows (``inputs_embeds``) and owns the three extra tensors.

As a drafter (``SpeculativeConfig(method="mtp", num_speculative_tokens=k)``): after the trunk's
step the head runs over the same rows with the token ids shifted by one (the last accepted row of a
request gets the token the trunk just chose), which both fills the head's KV cache for every
position the trunk has passed and yields one draft per request for the next step. Drafts two to k
come from decode-only passes of the head over its own hidden state (one row per request, at the
look-ahead positions the scheduler reserved). Rows past the accepted prefix of a verification, and
those look-ahead rows, write cache entries that the next pass over those positions overwrites.

Reference: src/vllm/model_executor/models/qwen3_5_mtp.cpp (weights and forward of the head; the
reference does not connect it to its engine loop).
"""
from __future__ import annotations

import copy
import dataclasses

import torch


class Qwen35MTP:
    def __init__(self, target, num_layers: int = 1):
        cfg = copy.copy(target.cfg)
        cfg.num_layers = num_layers
        cfg.layer_types = ["full_attention"] * num_layers
        cfg.quant = None                               # the head's tensors are bf16 in the checkpoints
        self.target = target
        self.inner = type(target)(cfg, device=target.device, parallel=target.par, comm=target.comm,
                                  max_position=getattr(target, "max_position", None))
        self.inner.be = target.be
        self.H = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        self.w: dict[str, torch.Tensor] = {}
        self.next_ids = None

    # ------------------------------------------------------------------ weights
    def _share(self) -> None:
        self.inner.w["embed"] = self.target.w["embed"]
        self.inner.w["lm_head"] = self.target.w["lm_head"]

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        self.inner.init_random(seed + 7919)
        self._share()
        g = torch.Generator().manual_seed(seed + 104729)
        dev, dt = self.target.device, self.target.dtype
        self.w = {"fc": torch.empty(self.H, 2 * self.H).normal_(0, std, generator=g).to(dt).to(dev),
                  "pre_fc_norm_embedding": torch.zeros(self.H, dtype=dt, device=dev),
                  "pre_fc_norm_hidden": torch.zeros(self.H, dtype=dt, device=dev)}

    def load_weights(self, named) -> None:
        """``mtp.*`` tensors of a checkpoint: the three input-stage tensors stay here, the decoder
        blocks and the final norm go to the inner model under the trunk's names."""
        dev, dt = self.target.device, self.target.dtype
        inner = []
        for name, t in named:
            if name.startswith("model.mtp."):
                name = name[len("model."):]
            if not name.startswith("mtp."):
                continue
            rest = name[len("mtp."):]
            key = rest[:-len(".weight")] if rest.endswith(".weight") else rest
            if key in ("fc", "pre_fc_norm_embedding", "pre_fc_norm_hidden"):
                self.w[key] = t.to(dt).contiguous().to(dev)
            elif rest == "norm.weight":
                inner.append(("model.norm.weight", t))
            elif rest.startswith("layers."):
                inner.append(("model." + rest, t))
        missing = {"fc", "pre_fc_norm_embedding", "pre_fc_norm_hidden"} - set(self.w)
        if missing or not inner:
            raise ValueError(f"checkpoint has no multi-token-prediction head (missing {sorted(missing) or 'mtp.layers'})")
        self._share()               # the inner loader ties lm_head to the embedding it finds
        self.inner.load_weights(iter(inner))
        self._share()

    # ------------------------------------------------------------------ caches
    def alloc(self, num_blocks: int, block_size: int, max_tokens: int, max_reqs: int) -> None:
        self.inner.alloc_kv_cache(num_blocks, block_size)
        self.inner.reserve_buffers(max_tokens, max_reqs)
        dev = self.target.device
        self.next_ids = torch.zeros(max_tokens, dtype=torch.int64, device=dev)
        self.rows = torch.zeros(max_reqs, dtype=torch.int32, device=dev)
        # step inputs of the decode-only passes that extend a draft chain (one row per request)
        max_blocks = (self.inner.max_position + block_size - 1) // block_size + 1
        self.d_pos = torch.zeros(max_reqs, dtype=torch.int64, device=dev)
        self.d_slots = torch.zeros(max_reqs, dtype=torch.int64, device=dev)
        self.d_seq = torch.zeros(max_reqs, dtype=torch.int32, device=dev)
        self.d_qs = torch.zeros(max_reqs + 1, dtype=torch.int32, device=dev)
        self.d_bt = None
        self._max_reqs = max_reqs

    def bind_block_table(self, max_blocks: int) -> None:
        self.d_bt = torch.zeros((self._max_reqs, max_blocks), dtype=torch.int32, device=self.target.device)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, next_ids: torch.Tensor, hidden: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """ctx: the trunk's step. next_ids int64 [T]: the token after each row's token; hidden
        [T, H]: the trunk's final hidden state per row; rows int32 [n]: rows whose prediction is
        wanted. Returns fp32 logits [n, vocab]."""
        t, be, T = self.target, self.target.be, ctx.num_tokens
        emb = be.embedding(next_ids[:T], t.w["embed"], vocab_start=t.vocab_start, vocab_total=t.cfg.vocab_size)
        if t.tp > 1:
            t.comm.all_reduce(emb)
        e = be.rmsnorm(emb, self.w["pre_fc_norm_embedding"], self.eps, gemma=True)
        h = be.rmsnorm(hidden[:T], self.w["pre_fc_norm_hidden"], self.eps, gemma=True)
        x = be.gemm(torch.cat([e, h], dim=1), self.w["fc"])
        extra = dict(ctx.extra)
        extra["inputs_embeds"] = x
        extra.pop("greedy_out", None)
        ctx2 = dataclasses.replace(ctx, logits_indices=rows, num_logits=int(rows.numel()),
                                   decode_only_full_logits=False, extra=extra)
        return self.inner.forward(ctx2)
