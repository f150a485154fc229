"""A second, smaller language model as the drafter of speculative decoding
(``SpeculativeConfig(method="draft_model", draft_model=<directory>, num_speculative_tokens=k)``).

The draft model is an ordinary model of any registered family with the target's vocabulary. It
keeps a paged KV cache of its own over the same block numbers as the target's, so the scheduler's
block tables and look-ahead slots serve both. Per engine step it runs

* once over the rows of the step the target just ran (same token ids, positions and slots), which
  fills its cache for every position the target has passed -- prompt chunks included; the logits of
  this pass are not needed; and
* ``k`` decode-only passes, one row per request that wants drafts: the token the target just chose
  at the position after the request's last kept row, then the draft model's own argmax at the
  following positions. The cache entries these passes write (and those of rejected drafts in the
  first pass) are replaced when the target reaches those positions.

Drafts are verified by the target with the greedy rejection rule, so the emitted tokens are the
target's own whatever the draft model proposes; a draft model that equals the target has every
draft accepted.

Reference: include/vllm/config/speculative.h names the method ("draft_model") and its look-ahead
arithmetic; the reference has no proposer for it.
"""
from __future__ import annotations

import dataclasses

import torch


class DraftModel:
    def __init__(self, model, target):
        if model.cfg.vocab_size != target.cfg.vocab_size:
            raise ValueError(f"draft model vocabulary {model.cfg.vocab_size} differs from the target's "
                             f"{target.cfg.vocab_size}")
        if hasattr(model, "snapshot_state"):
            raise ValueError("a draft model with recurrent state is not supported (its state would "
                             "have to be rolled back with every rejected draft)")
        self.model = model
        self.target = target
        self.rows = None

    def alloc(self, num_blocks: int, block_size: int, max_tokens: int, max_reqs: int, max_blocks: int) -> None:
        m = self.model
        if len(m.kv_cache_groups(block_size)) != 1:
            raise ValueError("the draft model must have one kind of attention layer (one KV cache group)")
        m.alloc_kv_cache(num_blocks, block_size)
        m.reserve_buffers(max_tokens, max_reqs)
        dev = m.device
        self.next_ids = torch.zeros(max_tokens, dtype=torch.int64, device=dev)
        self.rows = torch.zeros(max_reqs, dtype=torch.int32, device=dev)
        self.d_pos = torch.zeros(max_reqs, dtype=torch.int64, device=dev)
        self.d_slots = torch.zeros(max_reqs, dtype=torch.int64, device=dev)
        self.d_seq = torch.zeros(max_reqs, dtype=torch.int32, device=dev)
        self.d_qs = torch.zeros(max_reqs + 1, dtype=torch.int32, device=dev)
        self.d_bt = torch.zeros((max_reqs, max_blocks), dtype=torch.int32, device=dev)

    @staticmethod
    def _own_extra(ctx) -> dict:
        # the target's step may carry buffers the target writes (its argmax ids); the drafter's
        # passes must not touch them
        extra = dict(ctx.extra)
        extra.pop("greedy_out", None)
        extra.pop("inputs_embeds", None)
        return extra

    def fill(self, ctx) -> None:
        """The draft model over the target's step: writes its KV cache; one logits row, unused."""
        self.rows[:1].zero_()
        ctx2 = dataclasses.replace(ctx, logits_indices=self.rows[:1], num_logits=1,
                                   decode_only_full_logits=False, extra=self._own_extra(ctx))
        self.model.forward(ctx2)

    def decode(self, ctx) -> torch.Tensor:
        """One decode-only pass; fp32 logits [n, vocab]."""
        return self.model.forward(ctx)
