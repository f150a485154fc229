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


def sample(runner, info, logits: torch.Tensor, grammar) -> torch.Tensor:
    n = info.num_logits
    logits = logits[:n].float().clone()
    rows = [i for i, p in enumerate(info.produces_token) if p]
    v = runner.views

    # logits row -> batch row (a request that verifies drafts owns several rows)
    row_req = v["sample_rows"][: info.num_logits].long()

    def per_row(name):
        return v[name][: info.num_reqs][row_req]

    if grammar is not None and grammar.structured_output_request_ids:
        rid = {info.req_ids[j]: info.logits_row0[j] for j in rows}
        words = grammar.words_per_row
        mask = torch.tensor(grammar.bitmask, dtype=torch.int32).view(-1, words)
        V = logits.shape[1]
        bits = ((mask[:, :, None] >> torch.arange(32)) & 1).reshape(mask.shape[0], -1)[:, :V].bool()
        for mi, r in enumerate(grammar.structured_output_request_ids):
            if r in rid:
                logits[rid[r]][~bits[mi]] = -math.inf
    br, btk, bv, nr, nt = runner.batch.logit_edits(info, runner._eos)
    for r, t, x in zip(br, btk, bv):
        logits[r, t] += x
    for r, t in zip(nr, nt):
        logits[r, t] = -math.inf
    if info.any_penalties:
        pr, pt, pc = runner.batch.penalty_entries(info)
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
