"""CPU benchmark configuration: a Qwen3-0.6B-shaped dense decoder in bf16 on the native CPU
backend, 4 prompts of 128 uniform-random ids, 64 greedy tokens each, block size 16, one process.

    python -m vllm_cpp_b200.entrypoints.bench_cpu [--backend native|torch] [--threads N] [--layers L]

Prints one JSON line with prefill and decode token rates and the wall time of the run.
Reference: the CPU rows of docs/BENCHMARKS.md (prefill / decode tok/s of the CPU backend).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="native", choices=["native", "torch"])
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (quick runs)")
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--input-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=64)
    args = ap.parse_args(argv)
    from ..config import EngineArgs, synthetic_config
    from ..engine import LLM, SamplingParams
    if args.threads > 0:
        torch.set_num_threads(args.threads)
        if args.backend == "native":
            from ..ops import cpu_native
            cpu_native.set_num_threads(args.threads)
    cfg = synthetic_config("qwen3-0.6b")
    if args.layers > 0:
        cfg.num_layers = args.layers
    max_len = args.input_len + args.output_len + 16
    llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, max_model_len=max_len,
                         max_num_seqs=args.prompts, max_num_batched_tokens=args.prompts * args.input_len,
                         num_blocks=args.prompts * ((max_len + 15) // 16 + 1) + 8, cpu_backend=args.backend,
                         seed=0))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (args.input_len,), generator=g).tolist()
               for _ in range(args.prompts)]
    for p in prompts:
        llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True))
    t0 = time.perf_counter()
    llm.step()                                   # the whole prefill fits one step
    t_prefill = time.perf_counter() - t0
    steps = 0
    t1 = time.perf_counter()
    while llm._states:
        llm.step()
        steps += 1
    t_decode = time.perf_counter() - t1
    n_in = args.prompts * args.input_len
    n_out = args.prompts * (args.output_len - 1)
    print(json.dumps({
        "config": "Qwen3-0.6B-shaped bf16, CPU, %d x %d -> %d, block 16" % (args.prompts, args.input_len,
                                                                        args.output_len),
        "backend": llm.model.be.name, "layers": cfg.num_layers,
        "threads": (__import__("vllm_cpp_b200.ops.cpu_native", fromlist=["x"]).num_threads()
                    if args.backend == "native" else torch.get_num_threads()),
        "prefill_tok_s": round(n_in / t_prefill, 1), "decode_tok_s": round(n_out / t_decode, 1),
        "decode_steps": steps, "wall_s": round(t_prefill + t_decode, 2)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
