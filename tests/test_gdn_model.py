"""The Qwen3.5/3.6-style hybrid model (Gated DeltaNet + gated attention) through the engine.
CPU: chunked prefill + decode must reproduce an unchunked run (state carried across steps).
GPU: greedy tokens agree with the CPU oracle."""
import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams


def _prompts(cfg, lens, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def _run(dev, cfg, prompts, budget, max_tokens=6):
    llm = LLM(EngineArgs(model_config=cfg, device=dev, block_size=16, num_blocks=128, max_model_len=512,
                         max_num_seqs=4, max_num_batched_tokens=budget))
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    return [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]


@pytest.mark.parametrize("shape", ["tiny-gdn", "tiny-gdn-moe"])
def test_hybrid_cpu_chunked_prefill_matches_unchunked(shape):
    cfg = synthetic_config(shape)
    prompts = _prompts(cfg, (70, 5, 33))
    whole = _run("cpu", cfg, prompts, 256)
    chunked = _run("cpu", cfg, prompts, 32)      # prompts split over several steps
    assert whole == chunked
    alone = [_run("cpu", cfg, [p], 256)[0] for p in prompts]
    assert whole == alone                         # batching does not mix request states


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["tiny-gdn", "tiny-gdn-moe"])
def test_hybrid_gpu_vs_cpu(shape):
    from vllm_cpp_b200 import ops
    cfg = synthetic_config(shape)
    prompts = _prompts(cfg, (150, 9, 70))
    cpu = _run("cpu", cfg, prompts, 256, 8)
    for budget in (256, 64):
        gpu = _run("cuda", cfg, prompts, budget, 8)
        assert ops.read_status() == 0
        assert [a[0] for a in gpu] == [a[0] for a in cpu]
        hit = sum(sum(1 for p, q in zip(a, b) if p == q) for a, b in zip(gpu, cpu))
        assert hit / sum(len(a) for a in gpu) > 0.7


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["tiny-gdn", "tiny-gdn-moe"])
def test_hybrid_graph_replay_gives_the_eager_tokens(shape):
    """Decode through captured graphs (three requests padded to four rows, graphs captured lazily at
    the first decode step) against the same steps launched eagerly: pad rows carry no state slot and
    the capture's warm-up runs touch no live request, so the recurrent state advances exactly once
    per token and the tokens are the same, run after run."""
    from vllm_cpp_b200 import ops
    cfg = synthetic_config(shape)
    prompts = _prompts(cfg, (40, 7, 300), seed=9)

    def run(graphs):
        llm = LLM(EngineArgs(model_config=cfg, device="cuda", block_size=16, num_blocks=128, max_model_len=512,
                             max_num_seqs=4, max_num_batched_tokens=256, enable_cuda_graphs=graphs))
        sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
        return [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]

    eager = run(False)
    for _ in range(3):
        assert run(True) == eager
    assert ops.read_status() == 0
