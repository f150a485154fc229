"""Speculative decoding with a separate draft model: the emitted tokens are the target's own
whatever the draft model proposes, and a draft model that equals the target has every draft
accepted (which checks the draft model's cache fill, positions and look-ahead slots)."""
import dataclasses

import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams
from vllm_cpp_b200.spec_decode import SpeculativeConfig


def _prompts(cfg, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 5, 33, 120)]


def _run(cfg, prompts, spec, budget=256, n=14, seed=0):
    llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=160, max_model_len=512,
                         max_num_seqs=4, max_num_batched_tokens=budget, speculative_config=spec, seed=seed))
    sp = SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)
    # Besides the tokens: the draft model's logits of every chain step, and the target's logits of the
    # rows that verify those drafts one step later (row i of a verifying step predicts the same
    # position as chain step i of the drafting pass before).
    llm.draft_rounds, llm.target_rounds = {}, {}
    if llm.runner.drafter is not None:
        propose, decode, build = llm.runner._propose_draft_model, llm.runner.drafter.decode, llm.runner._build_output
        cur = []

        def decode_rec(ctx):
            lg = decode(ctx)
            cur.append(lg[: ctx.num_tokens].float().clone())
            return lg

        def propose_rec(info, toks_):
            cur.clear()
            before = set(llm.runner._drafts)
            propose(info, toks_)
            rids = [r for r in llm.runner._drafts if r not in before and llm.runner._drafts[r]]
            for j, rid in enumerate(rids):
                llm.draft_rounds.setdefault(rid, []).append(torch.stack([c[j] for c in cur]))

        def build_rec(info, ids_host):
            row = 0
            for r, p in enumerate(info.produces_token):
                if p:
                    k = info.num_draft[r]
                    if k:
                        llm.target_rounds.setdefault(info.req_ids[r], []).append(
                            llm.runner._logits[row: row + k].float().clone())
                    row += k + 1
            return build(info, ids_host)
        llm.runner.drafter.decode = decode_rec
        llm.runner._propose_draft_model = propose_rec
        llm.runner._build_output = build_rec
    # the gap between the two largest logits of every row that emitted a token: where it is within
    # bf16 noise, a step of another shape (k + 1 query rows instead of one) may pick the other token
    gaps: dict = {}
    inner = llm.runner._build_output

    def gap_rec(info, ids_host):
        lg = llm.runner._logits
        out = inner(info, ids_host)
        row = 0
        for r, p in enumerate(info.produces_token):
            if p:
                kept = len(out.sampled_token_ids[r])
                top = lg[row: row + kept].float().topk(2, -1).values
                gaps.setdefault(info.req_ids[r], []).extend((top[:, 0] - top[:, 1]).tolist())
                row += info.num_draft[r] + 1
        return out
    llm.runner._build_output = gap_rec
    outs = llm.generate(prompts, sp)
    toks = [o.outputs[0].token_ids for o in outs]
    llm.gaps = [gaps[o.request_id] for o in outs]
    return toks, llm


def _assert_same_tokens(toks, base, base_gaps, tie=0.12):
    """Equal token for token; a request may part ways only at a token the baseline chose by less
    than ``tie`` (after which its context differs and nothing more is compared)."""
    compared = 0
    for t, b, g in zip(toks, base, base_gaps):
        assert len(t) == len(b)
        for i, (x, y) in enumerate(zip(t, b)):
            if x != y:
                assert g[i] < tie, f"token {i}: {x} != {y} with a logit gap of {g[i]:.3f}"
                break
            compared += 1
    assert compared >= 0.6 * sum(len(b) for b in base)


@pytest.mark.parametrize("k", [1, 3])
def test_a_draft_model_equal_to_the_target_has_every_draft_accepted(k):
    cfg = synthetic_config("tiny-dense")
    prompts = _prompts(cfg)
    base, ref = _run(cfg, prompts, None)
    spec = SpeculativeConfig(method="draft_model", num_speculative_tokens=k,
                             draft_model_config=dataclasses.replace(cfg), draft_seed=0)
    # a small token budget: prompts arrive in chunks, which the draft model's cache must follow
    toks, llm = _run(cfg, prompts, spec, budget=48)
    _assert_same_tokens(toks, base, ref.gaps)
    st = llm.runner.spec_stats
    assert st["drafted"] > 0 and st["accepted"] == st["drafted"]
    # the draft model saw the same context as the target at every drafted position
    assert len(set(sum(base, []))) > 8, "the tokens are too uniform for this test to mean anything"
    checked = 0
    for rid, rounds in llm.target_rounds.items():
        for d, t in zip(llm.draft_rounds[rid], rounds):
            n = min(len(d), len(t))
            torch.testing.assert_close(d[:n], t[:n], atol=0.06, rtol=0.05)
            checked += n
    assert checked >= st["drafted"] // 2


def test_a_different_draft_model_keeps_the_targets_tokens():
    cfg = synthetic_config("tiny-dense")
    prompts = _prompts(cfg, seed=5)
    base, ref = _run(cfg, prompts, None)
    small = dataclasses.replace(cfg, num_layers=1)
    spec = SpeculativeConfig(method="draft_model", num_speculative_tokens=2, draft_model_config=small, draft_seed=11)
    toks, llm = _run(cfg, prompts, spec)
    _assert_same_tokens(toks, base, ref.gaps)
    st = llm.runner.spec_stats
    assert st["drafted"] > 0 and st["accepted"] < st["drafted"]      # an unrelated model is often wrong


def test_a_dense_draft_model_for_a_hybrid_target():
    cfg = synthetic_config("tiny-gdn")
    prompts = [p[:40] for p in _prompts(cfg, seed=7)]
    base, ref = _run(cfg, prompts, None)
    small = dataclasses.replace(synthetic_config("tiny-dense"), vocab_size=cfg.vocab_size)
    spec = SpeculativeConfig(method="draft_model", num_speculative_tokens=2, draft_model_config=small, draft_seed=2)
    toks, llm = _run(cfg, prompts, spec)
    _assert_same_tokens(toks, base, ref.gaps)
    assert llm.runner.spec_stats["drafted"] > 0


def test_vocabulary_and_state_checks():
    cfg = synthetic_config("tiny-dense")
    other = dataclasses.replace(cfg, vocab_size=cfg.vocab_size + 8)
    with pytest.raises(ValueError, match="vocabulary"):
        _run(cfg, _prompts(cfg), SpeculativeConfig(method="draft_model", draft_model_config=other), n=2)
    with pytest.raises(ValueError, match="recurrent state"):
        g = dataclasses.replace(synthetic_config("tiny-gdn"), vocab_size=cfg.vocab_size)
        _run(cfg, _prompts(cfg), SpeculativeConfig(method="draft_model", draft_model_config=g), n=2)
    with pytest.raises(ValueError, match="needs a draft model"):
        SpeculativeConfig(method="draft_model")
