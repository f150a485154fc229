"""Host sampler: the same pipeline order as the device one, on CPU tensors. It is the oracle
for the sampler kernels and the sampler of the CPU execution path.

Order (reference ``src/vllm/v1/sample/sampler.cpp``): grammar bitmask -> logit bias / banned
tokens (min_tokens stop ids, bad words) -> penalties -> greedy argmax snapshot ->
temperature -> min_p -> top-k / top-p -> softmax -> seeded exponential-race draw -> per-row
greedy / random merge.
"""
from __future__ import annotations

import math

import torch

from ..ops import reference as ref

EPS = 1e-5


def sample(runner, info, logits: torch.Tensor, edits: dict) -> torch.Tensor:
    """``edits``: the host-side sampler inputs of the step as plain lists (grammar bitmask rows,
    logit bias, banned tokens, penalty counts; see ``ModelRunner._host_sampler_edits``)."""
    n = info.num_logits
    logits = logits[:n].float().clone()
    rows = [i for i, p in enumerate(info.produces_token) if p]
    v = runner.views

    # logits row -> batch row (a request that verifies drafts owns several rows)
    row_req = v["sample_rows"][: info.num_logits].long()

    def per_row(name):
        return v[name][: info.num_reqs][row_req]

    if edits.get("grammar"):
        row_ids, bitmask, words = edits["grammar"]
        mask = torch.tensor(bitmask, dtype=torch.int32).view(-1, words)
        V = logits.shape[1]
        bits = ((mask[:, :, None] >> torch.arange(32)) & 1).reshape(mask.shape[0], -1)[:, :V].bool()
        for mi, row in enumerate(row_ids):
            if row >= 0:
                logits[row][~bits[mi]] = -math.inf
    if edits.get("bias"):
        for r, t, x in zip(*edits["bias"]):
            logits[r, t] += x
    if edits.get("ban"):
        for r, t in zip(*edits["ban"]):
            logits[r, t] = -math.inf
    if edits.get("penalties"):
        pr, pt, pc = edits["penalties"]
        rep, freq, pres = per_row("rep_pen"), per_row("freq_pen"), per_row("pres_pen")
        for r, t, c in zip(pr, pt, pc):
            x = logits[r, t]
            x = x / rep[r] if x > 0 else x * rep[r]
            x = x - freq[r] * c - (pres[r] if c > 0 else 0.0)
            logits[r, t] = x
    greedy = logits.argmax(-1)
    if info.all_greedy:
        return greedy
    temp = per_row("temperature")
    for r in range(n):
        if temp[r] >= EPS:
            logits[r] /= temp[r]
    min_p = per_row("min_p")
    for r in range(n):
        if min_p[r] > 0:
            pr_ = torch.softmax(logits[r], -1)
            logits[r][pr_ < min_p[r] * pr_.max()] = -math.inf
    logits = ref.top_k_top_p(logits, per_row("top_k").tolist(), per_row("top_p").tolist())
    probs = torch.softmax(logits, -1)
    seeds, steps = per_row("seeds"), per_row("steps")
    out = greedy.clone()
    for r in range(n):
        if temp[r] >= EPS:
            out[r] = ref.race_sample(probs[r], int(seeds[r]) & ((1 << 64) - 1), int(steps[r]))
    return out
