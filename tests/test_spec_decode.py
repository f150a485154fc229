"""Speculative-decoding pieces and the platform seam."""
import pytest
import torch

from vllm_cpp_b200.platforms import CpuPlatform, current_platform
from vllm_cpp_b200.spec_decode import MtpDraftHead, NgramProposer, SpeculativeConfig, greedy_rejection_sample


def _case(device):
    # request 0: drafts [5, 6, 7], target argmax [5, 6, 9, 1]  -> 5, 6, 9 (mismatch at the third)
    # request 1: drafts [3, 4],    target argmax [3, 4, 8]     -> 3, 4, 8 (all accepted + bonus)
    # request 2: no drafts,        target argmax [2]           -> 2
    ta = torch.tensor([5, 6, 9, 1, 3, 4, 8, 2], dtype=torch.int64, device=device)
    dr = torch.tensor([5, 6, 7, 3, 4], dtype=torch.int64, device=device)
    cu = torch.tensor([0, 3, 5, 5], dtype=torch.int32, device=device)
    want = [[5, 6, 9, -1], [3, 4, 8, -1], [2, -1, -1, -1]]
    return ta, dr, cu, want


def test_greedy_rejection_cpu():
    ta, dr, cu, want = _case("cpu")
    assert greedy_rejection_sample(ta, dr, cu, 3).tolist() == want


@pytest.mark.gpu
def test_greedy_rejection_gpu():
    ta, dr, cu, want = _case("cuda")
    assert greedy_rejection_sample(ta, dr, cu, 3).tolist() == want


def test_config_proposer_and_mtp_head():
    c = SpeculativeConfig("mtp", 3)
    assert (c.num_lookahead_slots, c.max_tokens_per_step, c.draft_forward_passes()) == (3, 4, 3)
    assert SpeculativeConfig("dflash", 4).draft_forward_passes() == 1
    with pytest.raises(ValueError):
        SpeculativeConfig("draft_model", 2)
    with pytest.raises(ValueError):
        SpeculativeConfig("magic", 2)
    p = NgramProposer(SpeculativeConfig("ngram", 3, prompt_lookup_min=2, prompt_lookup_max=3))
    assert p.propose([1, 2, 3, 4, 5, 9, 2, 3, 4]) == [5, 9, 2]
    assert p.propose([1, 2, 3]) == []
    head = MtpDraftHead(64)
    head.init_random(0)
    out = head.forward(torch.randn(5, 64).to(torch.bfloat16), torch.randn(5, 64).to(torch.bfloat16))
    assert out.shape == (5, 64) and torch.isfinite(out.float()).all()


def test_platform_seam():
    p = current_platform("cpu")
    assert isinstance(p, CpuPlatform) and not p.supports_fp8() and p.residency_policy() == "unified"
    with pytest.raises(RuntimeError):
        current_platform("vulkan").device_capability()


@pytest.mark.gpu
def test_cuda_platform():
    p = current_platform("cuda")
    assert p.supports_nvfp4() and p.supports_fp8() and p.attention_backends()[0] == "tcgen05_paged"


def _gen(spec, prompts, max_tokens=24, device="cpu"):
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-dense")
    llm = LLM(EngineArgs(model_config=cfg, device=device, block_size=16, max_model_len=256,
                         max_num_seqs=8, max_num_batched_tokens=128, num_blocks=128,
                         speculative_config=spec, seed=0))
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
    return [o.outputs[0].token_ids for o in outs], llm


def test_ngram_speculation_end_to_end_matches_plain_greedy():
    """Prompt-lookup drafts go through the scheduler, are verified in one forward pass and the
    output equals plain greedy decoding token for token."""
    import torch
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, 512, (12,), generator=g).tolist()
    prompts = [base * 4, torch.randint(0, 512, (40,), generator=g).tolist(), (base[:5] * 9)[:44]]
    plain, _ = _gen(None, prompts)
    spec, llm = _gen(SpeculativeConfig(method="ngram", num_speculative_tokens=3), prompts)
    assert spec == plain
    st = llm.runner.spec_stats
    assert st["drafted"] > 0          # repeated prompts always have a matching n-gram
    assert 0 <= st["accepted"] <= st["drafted"]


def test_speculation_accepts_correct_drafts_and_saves_steps():
    """With an oracle proposer (drafts = the tokens plain greedy decoding produces) every draft
    is accepted: same output, about a quarter of the decode steps at k = 3. A proposer that is
    always wrong costs nothing but the wasted rows."""
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 512, (30,), generator=g).tolist()
    plain, _ = _gen(None, [prompt], max_tokens=32)
    truth = prompt + plain[0]

    class Proxy:
        def __init__(self, inner, wrong):
            self._inner, self._wrong = inner, wrong

        def __getattr__(self, name):
            return getattr(self._inner, name)

        def propose_ngram(self, rid, lo, hi, k):
            n = self._inner.num_tokens(rid)      # prompt + tokens sampled so far
            nxt = truth[n:n + k]
            return [(t + 1) % 512 for t in nxt] if self._wrong else nxt

    for wrong in (False, True):
        cfg = synthetic_config("tiny-dense")
        llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, max_model_len=256,
                             max_num_seqs=8, max_num_batched_tokens=128, num_blocks=128, seed=0,
                             speculative_config=SpeculativeConfig(method="ngram", num_speculative_tokens=3)))
        got: dict = {}
        llm.runner.batch = Proxy(llm.runner.batch, wrong)
        rid = llm.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True))
        steps = 0
        done = False
        while not done and steps < 100:
            for st in llm.step():
                got[st.request_id] = list(st.outputs[0].token_ids)
                done = done or st.finished
            steps += 1
        assert got[rid] == plain[0]
        s = llm.runner.spec_stats
        if wrong:
            assert s["accepted"] == 0 and steps >= 32
        else:
            assert s["accepted"] == s["drafted"] > 0 and steps <= 12
