"""Speculative decoding building blocks: configuration (look-ahead arithmetic per method), the
greedy rejection sampler (accept a draft token iff it equals the target's argmax, stop at the
first mismatch, always emit one more token: the replacement or the bonus), an n-gram proposer,
the Qwen3.5/3.6 multi-token-prediction draft head and a separate draft model (models/draft.py).
The scheduler reserves look-ahead slots and rolls rejected tokens back; the loop is switched on
with ``EngineArgs(speculative_config=...)`` or the server's ``--speculative-config`` (methods
ngram, mtp and draft_model; the reference stops short of a user-facing switch).

Reference: ``include/vllm/config/speculative.h``, ``include/vllm/v1/spec_decode/
rejection_sampler.h:1-128``, ``src/vllm/model_executor/models/qwen3_5_mtp.cpp``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SpeculativeConfig:
    method: str = "mtp"                  # mtp | eagle | eagle3 | draft_model | ngram | dflash
    num_speculative_tokens: int = 1
    draft_model: Optional[str] = None    # checkpoint directory (or .gguf file) of the draft model
    draft_model_config: Optional[object] = None   # a ModelConfig instead: random weights from draft_seed
    draft_seed: Optional[int] = None
    prompt_lookup_min: int = 2
    prompt_lookup_max: int = 4
    parallel_drafting: bool = False      # dflash: all draft positions from one forward

    def __post_init__(self):
        if self.method not in ("mtp", "eagle", "eagle3", "draft_model", "ngram", "dflash"):
            raise ValueError(f"unknown speculative method {self.method!r}")
        if self.num_speculative_tokens < 1:
            raise ValueError("num_speculative_tokens must be at least 1")
        if self.method == "draft_model" and not self.draft_model and self.draft_model_config is None:
            raise ValueError("draft_model speculation needs a draft model")

    @property
    def num_lookahead_slots(self) -> int:
        """KV slots the scheduler must hold beyond the tokens it schedules."""
        return self.num_speculative_tokens

    @property
    def max_tokens_per_step(self) -> int:
        """Tokens one request can gain per step: every draft accepted plus the bonus token."""
        return self.num_speculative_tokens + 1

    def draft_forward_passes(self) -> int:
        return 1 if (self.parallel_drafting or self.method in ("dflash", "ngram")) else self.num_speculative_tokens

    def uses_draft_kv(self) -> bool:
        return self.method in ("eagle", "eagle3", "draft_model", "mtp")


def greedy_rejection_sample(target_argmax: torch.Tensor, draft: torch.Tensor, cu_draft: torch.Tensor,
                            max_spec: int) -> torch.Tensor:
    """target_argmax int64 [sum(n_draft) + n]: the target's greedy token at every draft position
    followed, per request, by the bonus position; draft int64 [sum(n_draft)]; cu_draft int32
    [n + 1]. Returns int64 [n, max_spec + 1] padded with -1."""
    n = cu_draft.numel() - 1
    if target_argmax.is_cuda:
        from .ops import _lib
        from .ops._lib import check, lib, ptr, stream_ptr
        P, I = _lib.P, _lib.I
        _lib.declare("b200_greedy_reject", [P, P, P, I, I, P, P], I)
        out = torch.empty((n, max_spec + 1), dtype=torch.int64, device=target_argmax.device)
        check(lib().b200_greedy_reject(ptr(target_argmax), ptr(draft), ptr(cu_draft), n, max_spec, ptr(out),
                                       stream_ptr()), "greedy_reject")
        return out
    out = torch.full((n, max_spec + 1), -1, dtype=torch.int64)
    cu = cu_draft.tolist()
    for r in range(n):
        d0, nd = cu[r], cu[r + 1] - cu[r]
        t0 = d0 + r
        i = 0
        while i < nd:
            tg = int(target_argmax[t0 + i])
            out[r, i] = tg
            if tg != int(draft[d0 + i]):
                break
            i += 1
        else:
            out[r, nd] = int(target_argmax[t0 + nd])
    return out


class NgramProposer:
    """Prompt-lookup drafting: find the longest recent n-gram (between ``min_n`` and ``max_n``
    tokens) that occurred earlier in the sequence and propose what followed it."""

    def __init__(self, cfg: SpeculativeConfig):
        self.k = cfg.num_speculative_tokens
        self.min_n, self.max_n = cfg.prompt_lookup_min, cfg.prompt_lookup_max

    def propose(self, token_ids: list[int]) -> list[int]:
        n_tok = len(token_ids)
        for n in range(min(self.max_n, n_tok - 1), self.min_n - 1, -1):
            tail = token_ids[n_tok - n:]
            for start in range(n_tok - n - 1, -1, -1):
                if token_ids[start:start + n] == tail:
                    follow = token_ids[start + n:start + n + self.k]
                    if follow:
                        return follow
        return []


class MtpDraftHead:
    """Qwen3.5/3.6 multi-token-prediction head: the embedding of the token just sampled and the
    trunk's last hidden state are normalised separately, concatenated and projected back to
    the hidden width (``fc``), pass through one decoder block of the trunk's kind and share
    the trunk's ``lm_head``."""

    def __init__(self, hidden: int, eps: float = 1e-6, device="cpu", dtype=torch.bfloat16):
        self.H, self.eps, self.device, self.dtype = hidden, eps, torch.device(device), dtype
        self.w: dict[str, torch.Tensor] = {}

    def init_random(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        H = self.H
        self.w = {"pre_fc_norm_embedding": torch.zeros(H), "pre_fc_norm_hidden": torch.zeros(H),
                  "fc": torch.empty(H, 2 * H).normal_(0, std, generator=g), "norm": torch.zeros(H)}
        self.w = {k: v.to(self.dtype).to(self.device) for k, v in self.w.items()}

    def load_weights(self, named):
        for name, t in named:
            key = name.split("mtp.")[-1].replace(".weight", "")
            if key in ("pre_fc_norm_embedding", "pre_fc_norm_hidden", "fc", "norm"):
                self.w[key] = t.to(self.dtype).to(self.device)

    @staticmethod
    def _norm(x, w, eps):
        xf = x.float()
        return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(x.dtype)

    def forward(self, token_embedding: torch.Tensor, hidden: torch.Tensor, block=None) -> torch.Tensor:
        """-> draft hidden state [T, H] (feed it to the shared lm_head). ``block`` is the
        decoder block callable of the trunk; None skips it (pure projection)."""
        e = self._norm(token_embedding, self.w["pre_fc_norm_embedding"], self.eps)
        h = self._norm(hidden, self.w["pre_fc_norm_hidden"], self.eps)
        x = (torch.cat([e, h], -1).float() @ self.w["fc"].float().t()).to(self.dtype)
        if block is not None:
            x = block(x)
        return self._norm(x, self.w["norm"], self.eps)
