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
