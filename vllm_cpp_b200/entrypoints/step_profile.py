"""Per-kernel device time of engine steps: ``python -m vllm_cpp_b200.entrypoints.step_profile``.

Builds an engine on a random-init model of a named shape (optionally cut to a few layers), drives
it through the public API (``LLM.add_request`` / ``LLM.step``) to steady state, and prints the CUDA
kernels of a few steps sorted by time (``torch.profiler``: CUPTI activity records, which also see
inside replayed CUDA graphs). Under ``torch.distributed.run`` it profiles rank 0 of a
tensor-parallel engine; kernels that wait on other ranks cannot be replayed, so this, not a replay
profiler, is how the multi-GPU step is broken down. ``B200_PDL=0`` in the environment keeps kernel
durations from overlapping (programmatic dependent launch starts a kernel while its predecessor
drains).

Reference: the per-op timing tables of ``docs/BENCHMARKS.md`` (VT_TRACE runs).
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("vllm_cpp_b200 step profile")
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N layers (0 = all)")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--decode-only", action="store_true",
                    help="prefill every request first and profile pure decode steps")
    ap.add_argument("--unfused", action="store_true", help="tensor parallel over GEMM + NCCL")
    ap.add_argument("--rows", type=int, default=28)
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..config import EngineArgs, ParallelConfig, synthetic_config
    from ..engine import LLM, SamplingParams
    cfg = synthetic_config(a.model)
    if a.layers:
        cfg.num_layers = a.layers
        if cfg.layer_types:
            cfg.layer_types = cfg.layer_types[: a.layers]
    C, IN, OUT = a.concurrency, a.input_len, a.output_len
    block = 32
    max_len = IN + OUT + block
    par = ParallelConfig(tensor_parallel_size=world, rank=rank, local_rank=local,
                         fused_collectives=not a.unfused,
                         enable_expert_parallel=bool(cfg.num_experts) and world > 1)
    llm = LLM(EngineArgs(model_config=cfg, device="cuda", block_size=block, max_model_len=max_len,
                         max_num_seqs=C, max_num_batched_tokens=8192,
                         num_blocks=C * ((max_len + block - 1) // block + 1) + 64,
                         enable_prefix_caching=True, parallel=par))
    gen = torch.Generator().manual_seed(1)

    def submit(n):
        llm.add_request(torch.randint(0, cfg.vocab_size, (IN,), generator=gen).tolist(),
                        SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))

    def step():
        for st in llm.step():
            if st.finished and not a.decode_only:
                submit(OUT)

    if a.decode_only:
        for _ in range(C):
            submit(OUT)
        n = 0
        while n < 4000:
            step()
            n += 1
            info = llm.runner._info
            if info is not None and info.num_prefills == 0 and n > 3:
                break
    else:
        # staggered lengths, so that finishes (and the prefills that replace them) spread evenly
        for i in range(C):
            submit(1 + (i * OUT) // C)
        first, n = set(llm._states.keys()), 0
        while first & set(llm._states.keys()) and n < 400:
            step()
            n += 1
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"{a.model}: {cfg.num_layers} layers, world {world}, "
              f"{'decode-only' if a.decode_only else 'steady-state'} steps, batch {C}, input {IN}: "
              f"{(time.perf_counter() - t0) * 1e3 / 5:.3f} ms per step (wall, 5 steps)", flush=True)
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            step()
        torch.cuda.synchronize()
    if rank == 0:
        print(f"kernels of {a.steps} steps:")
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=a.rows, max_name_column_width=70))
        print("kernel status word:", llm.runner.ops.read_status())
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)        # graphs holding NCCL kernels make an orderly teardown slow; nothing is left to flush


if __name__ == "__main__":
    raise SystemExit(main())
