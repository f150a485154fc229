"""Tensor / expert parallel sharding and failure detection with host-mock ranks (threads of
one process, no GPU): every rank runs its own engine on its weight shard; collectives go
through ``FakeComm``."""
import threading

import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, ParallelConfig, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams
from vllm_cpp_b200.parallel.comm import FakeComm


def _prompts(cfg):
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 9, 70)]


def _run_world(cfg, world, prompts, n=6):
    w = FakeComm.make_world(world)
    results, errors = [None] * world, [None] * world

    def rank_main(r):
        try:
            par = ParallelConfig(tensor_parallel_size=world, rank=r, fused_collectives=False)
            llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                                 max_num_seqs=4, max_num_batched_tokens=128, parallel=par),
                      comm=FakeComm(w, r, timeout=60.0))
            sp = SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)
            results[r] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        except Exception as e:  # surfaced in the main thread
            errors[r] = e
            w.barrier.abort()

    ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=300)
    for e in errors:
        if e is not None:
            raise e
    return results


@pytest.mark.parametrize("name,world", [("tiny-dense", 2), ("tiny-qwen3", 2), ("tiny-moe", 2), ("tiny-dense", 4),
                                        ("tiny-mla", 2), ("tiny-gdn", 2), ("tiny-gdn+nvfp4", 2)])
def test_sharded_ranks_agree_with_single_rank(name, world):
    name, _, quant = name.partition("+")
    cfg = synthetic_config(name)
    if quant:
        cfg.quant = quant                               # every rank quantises its own shard
    if name == "tiny-gdn":
        cfg.num_heads, cfg.num_kv_heads = 4, 1          # the kv head is replicated on both ranks
    prompts = _prompts(cfg)
    base = _run_world(cfg, 1, prompts)[0]
    ranks = _run_world(cfg, world, prompts)
    assert all(r == ranks[0] for r in ranks)            # every rank samples the same tokens
    hit = sum(sum(1 for p, q in zip(a, b) if p == q) for a, b in zip(ranks[0], base))
    assert [a[0] for a in ranks[0]] == [a[0] for a in base]
    assert hit / sum(len(a) for a in base) > 0.8        # summation order differs, nothing else


def test_missing_rank_is_detected_not_waited_for_forever():
    w = FakeComm.make_world(2)
    c0 = FakeComm(w, 0, timeout=0.5)
    t = torch.ones(4)
    with pytest.raises(RuntimeError, match="failed to join"):
        c0.all_reduce(t)                                # rank 1 never shows up
    # the world is marked failed: later collectives fail fast on every rank
    assert w.failed
    c1 = FakeComm(w, 1, timeout=0.5)
    with pytest.raises(RuntimeError):
        c1.all_gather(t)


def test_rank_that_raises_unblocks_its_peers():
    w = FakeComm.make_world(2)
    seen = {}

    def good():
        try:
            FakeComm(w, 0, timeout=30.0).all_reduce(torch.ones(2))
        except RuntimeError as e:
            seen["err"] = str(e)

    def bad():
        try:
            raise ValueError("simulated crash before the collective")
        except ValueError:
            w.barrier.abort()                           # what the rank wrapper does on any error

    ts = [threading.Thread(target=good), threading.Thread(target=bad)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=10)
    assert "failed to join" in seen.get("err", "")


def _run_driver_worker(cfg, world, submit, sampling=None):
    """One scheduler on rank 0, ``world - 1`` worker ranks that only run published steps.
    ``submit(llm)`` drives rank 0 and returns its result."""
    w = FakeComm.make_world(world)
    out, errors = {}, [None] * world
    llms = [None] * world

    def rank_main(r):
        try:
            par = ParallelConfig(tensor_parallel_size=world, rank=r, fused_collectives=False, driver_worker=True)
            llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                                 max_num_seqs=4, max_num_batched_tokens=128, parallel=par),
                      comm=FakeComm(w, r, timeout=60.0))
            llms[r] = llm
            if r == 0:
                out["result"] = submit(llm)
                llm.shutdown()
            else:
                llm.serve_as_worker()
        except Exception as e:
            errors[r] = e
            w.barrier.abort()

    ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=300)
    return out.get("result"), errors, llms


def test_one_scheduler_many_workers_matches_single_rank():
    """Only rank 0 is given requests (and an abort); the worker ranks follow through the step
    channel and the tokens equal those of a single-rank engine."""
    cfg = synthetic_config("tiny-qwen3")
    prompts = _prompts(cfg)
    base = _run_world(cfg, 1, prompts)[0]

    def submit(llm):
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        doomed = llm.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
        llm.step()
        llm.abort_request(doomed)                    # an abort reaches nobody but the scheduler
        # a sampled (seeded) and a penalised request go through the sampler-input message
        extra = SamplingParams(temperature=0.8, top_p=0.9, seed=5, max_tokens=4, repetition_penalty=1.3)
        return ([o.outputs[0].token_ids for o in llm.generate(prompts, sp)],
                [o.outputs[0].token_ids for o in llm.generate(prompts[:1], extra)])

    (greedy, sampled), errors, llms = _run_driver_worker(cfg, 2, submit)
    assert errors == [None, None]
    hit = sum(sum(1 for p, q in zip(a, b) if p == q) for a, b in zip(greedy, base))
    assert [a[0] for a in greedy] == [a[0] for a in base] and hit / sum(len(a) for a in base) > 0.8
    assert len(sampled[0]) == 4
    with pytest.raises(RuntimeError, match="owns no scheduler"):
        llms[1].add_request(prompts[0], SamplingParams(max_tokens=1))


def test_worker_that_raises_unblocks_the_scheduling_rank():
    cfg = synthetic_config("tiny-dense")
    prompts = _prompts(cfg)

    def submit(llm):
        sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
        return llm.generate(prompts, sp)

    w = FakeComm.make_world(2)
    errors = [None, None]

    def driver():
        try:
            par = ParallelConfig(tensor_parallel_size=2, rank=0, fused_collectives=False, driver_worker=True)
            llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                                 max_num_seqs=4, max_num_batched_tokens=128, parallel=par),
                      comm=FakeComm(w, 0, timeout=20.0))
            submit(llm)
        except Exception as e:
            errors[0] = e

    def worker():
        try:
            par = ParallelConfig(tensor_parallel_size=2, rank=1, fused_collectives=False, driver_worker=True)
            llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                                 max_num_seqs=4, max_num_batched_tokens=128, parallel=par),
                      comm=FakeComm(w, 1, timeout=20.0))
            calls = {"n": 0}
            real = llm.runner._launch_step

            def failing(info, pad, plain):
                calls["n"] += 1
                if calls["n"] == 3:
                    raise RuntimeError("injected worker failure")
                return real(info, pad, plain)

            llm.runner._launch_step = failing
            llm.serve_as_worker()
        except Exception as e:
            errors[1] = e

    ts = [threading.Thread(target=driver), threading.Thread(target=worker)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in ts)                 # nobody waits for ever
    assert "injected" in str(errors[1]) and errors[0] is not None
