"""CPU benchmark configuration: a Qwen3-0.6B-shaped dense decoder in bf16 on the native CPU
backend, 4 prompts of 128 uniform-random ids, 64 greedy tokens each, block size 16, one process.

    python -m vllm_cpp_b200.entrypoints.bench_cpu [--backend native|torch] [--threads N] [--layers L]
    python -m vllm_cpp_b200.entrypoints.bench_cpu --impl reference --reference-bin <vllm-bench>

The second form times the same workload on the reference project's own CPU build (its stock
bench tool, CMake option VLLM_CPP_CUDA=OFF) with a random-init checkpoint of the same shape
written by ``baseline/ref_assets.py``; the stock tool fixes the block size at 32.

Prints one JSON line with prefill and decode token rates and the wall time of the run.
Reference: the CPU rows of docs/BENCHMARKS.md (prefill / decode tok/s of the CPU backend).
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def run_reference(args) -> int:
    import importlib.util
    import os
    import subprocess
    import tempfile
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    exe = args.reference_bin if os.path.isabs(args.reference_bin) else os.path.join(root, args.reference_bin)
    if not os.path.exists(exe):
        print(json.dumps({"impl": "reference", "unavailable": f"{args.reference_bin} not built"}))
        return 0
    spec = importlib.util.spec_from_file_location("ref_assets", os.path.join(root, "baseline", "ref_assets.py"))
    ref_assets = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_assets)
    with tempfile.TemporaryDirectory() as d:
        ref_assets.write_checkpoint(d, "qwen3-0.6b", layers=args.layers or None)
        prompts = ref_assets.write_prompts(os.path.join(d, "prompts.json"), args.prompts, args.input_len)
        r = subprocess.run([exe, "--model", d, "--dataset-path", prompts, "--num-prompts", str(args.prompts),
                            "--input-len", str(args.input_len), "--output-len", str(args.output_len),
                            "--concurrency", str(args.prompts)], capture_output=True, text=True)
    rep = {}
    for line in r.stdout.splitlines():
        for label, key in (("Benchmark duration (s):", "wall_s"), ("Output token throughput (tok/s):", "output_tok_s"),
                           ("Input (prefill) token throughput (tok/s):", "input_tok_s"),
                           ("Median TTFT (ms):", "p50_ttft_ms"), ("Median TPOT (ms):", "p50_tpot_ms")):
            if line.startswith(label):
                rep[key] = float(line[len(label):].strip())
    if r.returncode != 0 or "wall_s" not in rep:
        print(json.dumps({"impl": "reference", "unavailable": (r.stderr or r.stdout)[-300:]}))
        return 0
    print(json.dumps({"config": "Qwen3-0.6B-shaped bf16, CPU, %d x %d -> %d, block 32 (fixed by the tool)"
                                % (args.prompts, args.input_len, args.output_len),
                      "impl": "reference", **rep}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="native", choices=["native", "torch"])
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (quick runs)")
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--input-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=64)
    ap.add_argument("--weight-quant", default=None, choices=["q8_0", "q4_0"],
                    help="keep the linear weights in GGUF blocks and multiply on the packed form (not the "
                         "bf16 configuration the reference numbers are quoted on)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reference-bin", default="baseline/_ref/cpu/bin/vllm-bench")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return run_reference(args)
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
                         cpu_weight_quant=args.weight_quant, seed=0))
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
        "config": "Qwen3-0.6B-shaped %s, CPU, %d x %d -> %d, block 16" % (args.weight_quant or "bf16", args.prompts,
                                                                      args.input_len, args.output_len),
        "backend": llm.model.be.name, "layers": cfg.num_layers,
        "threads": (__import__("vllm_cpp_b200.ops.cpu_native", fromlist=["x"]).num_threads()
                    if args.backend == "native" else torch.get_num_threads()),
        "gemm_tier": ({0: "scalar", 2: "avx2", 3: "avx512-bf16", 4: "amx-bf16"}.get(
            __import__("vllm_cpp_b200.ops.cpu_native", fromlist=["x"]).lib().b200cpu_simd_tier(), "?")
            if args.backend == "native" else "torch"),
        "prefill_tok_s": round(n_in / t_prefill, 1), "decode_tok_s": round(n_out / t_decode, 1),
        "decode_steps": steps, "wall_s": round(t_prefill + t_decode, 2),
        "output_tok_s": round(args.prompts * args.output_len / (t_prefill + t_decode), 2),
        "p50_ttft_ms": round(t_prefill * 1e3, 1), "p50_tpot_ms": round(t_decode / max(steps, 1) * 1e3, 2)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
