"""Serving benchmark: output tokens/s of the engine on the Llama-3.1-8B-shaped BF16 config.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (synthetic, random-init weights): continuous batching at concurrency 256, every
request 1024 uniform-random prompt ids and 256 greedy output tokens. The engine is first
brought to steady state (untimed ramp in which the initial requests get staggered output
lengths, so arrivals are spread evenly afterwards), then W warm-up steps, then EXACTLY K
engine steps are timed. One step = one iteration of the engine loop (schedule, one packed
host->device copy from pinned memory, forward, sample, device->host read of the sampled
ids, update).

Two numbers come out of the same K steps:
  value      output tokens / sum of per-step device time (CUDA events around each step's
             GPU work, max over ranks)
  e2e.value  output tokens / wall time of the K ``LLM.step()`` calls (public API, includes
             the host scheduler, the copies and the synchronisation), max over ranks
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

MODEL = "llama-3.1-8b"
CONCURRENCY = 256
INPUT_LEN = 1024
OUTPUT_LEN = 256
PUBLISHED_BASELINE = None  # the reference publishes no number for this model / hardware
MODEL_LABELS = {"llama-3.1-8b": "Llama-3.1-8B-shaped", "qwen3-0.6b": "Qwen3-0.6B-shaped",
                "qwen3-coder-30b-a3b": "Qwen3-Coder-30B-A3B-shaped",
                "deepseek-v2-lite": "DeepSeek-V2-Lite-shaped", "qwen3.6-27b": "Qwen3.6-27B-shaped"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "200", "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, since: float = 0.0) -> dict:
        """Summary of the samples taken at or after ``since`` (perf_counter time). The sampler is
        started before the warm-up steps: the start-up of nvidia-smi (NVML initialisation) stalls
        kernel launches of this process for a moment and must not land in the timed region."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, ln in self.lines:
            if ts < since:
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


REF_LABELS = {
    "Output token throughput (tok/s):": "output_tok_s",
    "Benchmark duration (s):": "duration_s",
    "Total generated tokens:": "total_output",
    "Total input tokens:": "total_input",
    "Successful requests:": "completed",
    "Median TTFT (ms):": "p50_ttft_ms",
    "Median TPOT (ms):": "p50_tpot_ms",
    "Median ITL (ms):": "p50_itl_ms",
}


def parse_reference_report(text: str) -> dict:
    """Numbers of the reference bench tool's result block (reference:
    examples/bench/bench_core.h `PrintReport`, fixed-width "label value" lines)."""
    out = {}
    for line in text.splitlines():
        for label, key in REF_LABELS.items():
            if line.startswith(label):
                try:
                    out[key] = float(line[len(label):].strip())
                except ValueError:
                    pass
    return out


def run_reference(args) -> int:
    """The reference arm: the unmodified reference engine, built from its own CMake project for
    sm_100a (`baseline/_ref/cuda/bin/vllm-bench`, its stock bench tool), loads a random-init
    checkpoint of the same architecture through its own loader and serves the same workload
    (concurrency, input and output lengths, greedy, ignore-eos) through its own engine loop.
    Nothing of this repository's package is imported here. The reference has no multi-GPU mode:
    at N > 1 every rank starts one stock process on its own GPU with 1/N of the concurrent
    requests; tokens add up and the slowest process sets the time."""
    here = os.path.dirname(os.path.abspath(__file__))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    def unavailable(why: str) -> int:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why[:400]}))
        return 0

    exe = os.path.join(here, "baseline", "_ref", "cuda", "bin", "vllm-bench")
    if not os.path.exists(exe):
        return unavailable("baseline/_ref/cuda/bin/vllm-bench is missing: the reference's CMake "
                           "build for sm_100a has not been installed into baseline/_ref")
    sys.path.insert(0, os.path.join(here, "baseline"))
    import ref_assets
    if args.model not in ref_assets.SHAPES:
        return unavailable(f"no reference checkpoint recipe for --model {args.model}")
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        return unavailable("no GPU visible to the reference arm")
    if world > 1:
        dist.init_process_group("gloo")
    scratch = os.environ.get("B200_BENCH_SCRATCH", "/tmp")
    ckpt = os.path.join(scratch, f"b200_ref_ckpt_{args.model}" + (f"_L{args.layers}" if args.layers else ""))
    C_total, IN, OUT = args.concurrency, args.input_len, args.output_len
    C = C_total // world + (1 if rank < C_total % world else 0)
    n_prompts = 2 * C
    try:
        if rank == 0 and not os.path.exists(os.path.join(ckpt, "done")):
            torch.cuda.set_device(local_rank)
            ref_assets.write_checkpoint(ckpt, args.model, layers=args.layers or None)
            open(os.path.join(ckpt, "done"), "w").close()
        if world > 1:
            dist.barrier()
        prompts = ref_assets.write_prompts(os.path.join(scratch, f"b200_ref_prompts_{rank}.json"),
                                           n_prompts, IN, seed=1 + rank)
    except OSError as e:
        return unavailable(f"could not write the synthetic checkpoint: {e}")
    torch.cuda.empty_cache()
    cmd = [exe, "--model", ckpt, "--dataset-path", prompts, "--num-prompts", str(n_prompts),
           "--input-len", str(IN), "--output-len", str(OUT), "--concurrency", str(C),
           "--max-num-batched-tokens", str(args.max_num_batched_tokens)]
    env = dict(os.environ)
    env["CUDA_VISIBLE_DEVICES"] = str(local_rank)
    sampler = ClockSampler(local_rank)
    if world > 1:
        dist.barrier()
    sampler.start()
    t0 = time.perf_counter()
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=args.watchdog)
        rc, out, err = r.returncode, r.stdout, r.stderr
    except subprocess.TimeoutExpired as e:
        rc, out, err = -9, (e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or ""), "timed out"
    wall = time.perf_counter() - t0
    clocks = sampler.stop(since=t0)
    rep = parse_reference_report(out)
    ok = rc == 0 and "output_tok_s" in rep and rep.get("duration_s", 0) > 0
    mine = {"ok": ok, "rc": rc, "rep": rep, "wall": wall, "err": (err or "")[-300:]}
    if world > 1:
        allr = [None] * world
        dist.all_gather_object(allr, mine)
    else:
        allr = [mine]
    if rank != 0:
        return 0
    bad = [a for a in allr if not a["ok"]]
    if bad:
        return unavailable(f"reference vllm-bench failed (exit {bad[0]['rc']}): {bad[0]['err']!r}")
    tokens = sum(a["rep"]["total_output"] for a in allr)
    dur = max(a["rep"]["duration_s"] for a in allr)
    value = tokens / dur
    print(json.dumps({
        "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random-digit prompts of the named length, random-init weights)",
        "impl": "reference",
        "config": {"model": MODEL_LABELS.get(args.model, args.model), "global_batch": C_total,
                   "seq_len": IN + OUT, "input_len": IN, "output_len": OUT,
                   "parallelism": "tp1" if world == 1 else f"dp{world}",
                   "reference_parallelism": ("1 stock process" if world == 1 else
                                             f"{world} stock processes, one per GPU (the reference "
                                             "has no multi-GPU mode)"),
                   "mode": f"closed loop, {n_prompts * world} requests at concurrency {C_total}, "
                           "whole run timed by the tool's own clock (steps/warmup do not apply)",
                   "max_num_batched_tokens": args.max_num_batched_tokens,
                   "command": " ".join(["vllm-bench"] + cmd[1:])},
        "clocks": clocks,
        "latency": {"p50_ttft_ms": max(a["rep"].get("p50_ttft_ms", -1) for a in allr),
                    "p50_tpot_ms": max(a["rep"].get("p50_tpot_ms", -1) for a in allr)},
        "e2e": {"value": round(value, 2), "unit": "tok/s", "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": None,
                "note": "the tool times its engine loop with the host clock from text in to "
                        "tokens out, so this is the same number as value"},
        "gpu_launches": None, "output_tokens": int(tokens), "wall_s_with_load": round(max(a["wall"] for a in allr), 1),
    }))
    return 0


def closed_loop(llm, torch, new_prompt, SamplingParams, concurrency: int, num_requests: int, out_len: int):
    """Runs ``num_requests`` requests with at most ``concurrency`` in flight to completion and
    times everything on the device: every step is bracketed by CUDA events, the timeline of a
    request is the event time between the first step that carried it and the steps that produced
    its first and last token. Returns output tok/s over the event timeline and p50 TTFT / TPOT."""
    r = llm.runner
    r.step_events = []
    r.time_steps = True
    submitted_at, first_at, last_at, count = {}, {}, {}, {}
    step_reqs = []                     # per engine step: (ids submitted before it, outputs)
    pending, done, nxt = [], 0, 0

    def admit():
        nonlocal nxt
        while nxt < num_requests and len(submitted_at) - done < concurrency:
            rid = llm.add_request(new_prompt(), SamplingParams(temperature=0.0, max_tokens=out_len, ignore_eos=True))
            submitted_at[rid] = None
            pending.append(rid)
            nxt += 1

    admit()
    step_no = 0
    while done < num_requests:
        n_ev = len(r.step_events)
        outs = llm.step()
        ran = len(r.step_events) > n_ev
        if ran:
            for rid in pending:
                submitted_at[rid] = len(r.step_events) - 1          # index of the first step that could carry it
            pending.clear()
        for st in outs:
            rid = st.request_id
            ev = len(r.step_events) - 1
            if rid not in first_at:
                first_at[rid] = ev
            last_at[rid] = ev
            count[rid] = count.get(rid, 0) + 1
            if st.finished:
                done += 1
        admit()
        step_no += 1
        if step_no > 200000:
            break
    torch.cuda.synchronize()
    ev = [e for e in r.step_events if e[1] is not None]
    r.time_steps = False
    r.step_events = []
    if not ev:
        return None
    t0 = ev[0][0]
    start = [t0.elapsed_time(a) for a, _ in ev]
    end = [t0.elapsed_time(b) for _, b in ev]
    # async scheduling delivers a step's tokens one call later: clamp indices into the recorded range
    def E(i):
        return end[min(max(i, 0), len(end) - 1)]
    ttft = sorted(E(first_at[x]) - start[min(submitted_at[x] or 0, len(start) - 1)] for x in first_at
                  if submitted_at.get(x) is not None)
    tpot = sorted((E(last_at[x]) - E(first_at[x])) / (count[x] - 1) for x in first_at if count.get(x, 0) > 1)
    tokens = sum(count.values())
    return {"concurrency": concurrency, "requests": num_requests, "output_tokens": tokens,
            "device_s": round(end[-1] / 1e3, 4), "output_tok_s": round(tokens / (end[-1] / 1e3), 2),
            "p50_ttft_ms": round(ttft[len(ttft) // 2], 2) if ttft else None,
            "p50_tpot_ms": round(tpot[len(tpot) // 2], 3) if tpot else None,
            "timing": "CUDA events around every step, one timeline per run"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--concurrency", type=int, default=CONCURRENCY)
    ap.add_argument("--input-len", type=int, default=INPUT_LEN)
    ap.add_argument("--output-len", type=int, default=OUTPUT_LEN)
    ap.add_argument("--parallelism", default="tp", choices=["tp", "dp"],
                    help="N > 1: tp = one tensor-parallel (and, for MoE models, expert-parallel) "
                         "engine over all GPUs with the fused GEMM + collective kernels; "
                         "dp = one engine replica per GPU, the concurrent requests split between "
                         "them (a comparison mode, no collective on the hot path)")
    ap.add_argument("--unfused", action="store_true",
                    help="tp: GEMM kernels + NCCL collectives instead of the fused kernels "
                         "(the baseline the fused path is compared with)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="diagnostic: override the number of layers (the JSON line then carries "
                         "layers_override and is not a benchmark result)")
    ap.add_argument("--verbose", action="store_true", help="phase timestamps on stderr")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="seconds after which every rank dumps its Python stacks and exits")
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra keys (the whole offline batch and the concurrency sweep)")
    ap.add_argument("--sync-scheduling", action="store_true",
                    help="schedule step N+1 only after step N's tokens are on the host")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3

    import faulthandler
    if args.watchdog > 0:
        # a rank stuck in a collective or a kernel wait must not hold the GPUs: dump and leave
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    import torch
    import torch.distributed as dist

    t_start = time.perf_counter()

    def note(msg):
        if args.verbose:
            print(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - t_start:7.1f}s] {msg}",
                  file=sys.stderr, flush=True)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n_gpus = world

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from vllm_cpp_b200.config import EngineArgs, ParallelConfig, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    from vllm_cpp_b200.ops import _lib

    dp = world > 1 and args.parallelism == "dp"
    cfg = synthetic_config(args.model)
    if args.layers > 0:
        cfg.num_layers = args.layers
        if cfg.layer_types:
            cfg.layer_types = cfg.layer_types[: args.layers]
    C_total, IN, OUT = args.concurrency, args.input_len, args.output_len
    # data parallel: this replica serves its share of the concurrent requests
    C = (C_total // world + (1 if rank < C_total % world else 0)) if dp else C_total
    block = 32
    max_len = IN + OUT + block
    llm = LLM(EngineArgs(
        model_config=cfg, device="cuda", block_size=block, max_model_len=max_len,
        max_num_seqs=C, max_num_batched_tokens=args.max_num_batched_tokens,
        num_blocks=C * ((max_len + block - 1) // block + 1) + 64,
        enable_cuda_graphs=not args.no_graphs, enable_prefix_caching=True,
        async_scheduling=not args.sync_scheduling,
        parallel=(ParallelConfig(local_rank=local_rank) if dp else
                  ParallelConfig(tensor_parallel_size=world, rank=rank, local_rank=local_rank,
                                 enable_expert_parallel=bool(cfg.num_experts) and world > 1,
                                 fused_collectives=not args.unfused))))
    note("engine built")
    gen = torch.Generator().manual_seed(1 + (rank if dp else 0))

    def new_prompt():
        return torch.randint(0, cfg.vocab_size, (IN,), generator=gen).tolist()

    # per-request latency bookkeeping (host clock): time to first token and time per output token
    t_submit, t_first, n_out = {}, {}, {}
    ttft_ms, tpot_ms = [], []

    def submit(out_len):
        rid = llm.add_request(new_prompt(), SamplingParams(temperature=0.0, max_tokens=out_len,
                                                           ignore_eos=True))
        t_submit[rid] = time.perf_counter()

    # ---- ramp to steady state (untimed): staggered output lengths for the first wave
    llm.runner.warmup_graphs()
    note("graphs captured")
    # First wave: staggered output lengths so that one request finishes per step afterwards. No
    # first-wave request may finish before the whole wave has been prefilled (C * IN tokens at
    # the batched-token budget per step): its replacement would queue behind the remaining
    # prompts, all such replacements would then be admitted together and finish together, and
    # that burst would come round every OUT steps for ever.
    fill_steps = min(OUT - 1, (C * IN + args.max_num_batched_tokens - 1) // args.max_num_batched_tokens + 2)
    for i in range(C):
        submit(fill_steps + (i * (OUT - fill_steps)) // C)
    ramp_steps = 0
    trace = []      # verbose: (scheduled tokens, finished, preempted so far, running, waiting) per step

    def step_and_refill():
        """One engine step; finished requests are replaced at once (closed loop)."""
        outs = llm.step()
        now = time.perf_counter()
        fin = 0
        for st in outs:
            rid = st.request_id
            if rid not in t_first:
                t_first[rid] = now
                if rid in t_submit:
                    ttft_ms.append((now - t_submit[rid]) * 1e3)
            n_out[rid] = n_out.get(rid, 0) + 1
            if st.finished:
                fin += 1
                if n_out[rid] > 1:
                    tpot_ms.append((now - t_first[rid]) * 1e3 / (n_out[rid] - 1))
                for d in (t_submit, t_first, n_out):
                    d.pop(rid, None)
        for _ in range(fin):
            submit(OUT)
        if args.verbose:
            ss = llm.step_stats()
            trace.append((ss["scheduled_tokens"], fin, ss["num_preempted"], ss["num_running"], ss["num_waiting"]))
        return outs

    # the ramp ends once every first-wave request has finished (all live requests are
    # full-length ones at evenly spread positions)
    first_wave = set(llm._states.keys())
    while first_wave & set(llm._states.keys()):
        step_and_refill()
        ramp_steps += 1
        if args.verbose and ramp_steps % 32 == 1:
            note(f"ramp step {ramp_steps}")
        if ramp_steps > 4 * OUT + 64:
            break
    note(f"ramp done after {ramp_steps} steps")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.5)                 # let nvidia-smi finish starting before anything is measured
    for _ in range(args.warmup):
        step_and_refill()

    # ---- timed region
    h2d0, d2h0 = llm.runner.h2d_bytes, llm.runner.d2h_bytes
    launches0 = _lib.LAUNCHES[0]
    tokens = 0
    barrier()
    llm.runner.step_events = []
    llm.runner.time_steps = True
    ttft_ms.clear()
    tpot_ms.clear()
    t0 = time.perf_counter()
    host_step, sched_tokens = [], []
    for i in range(args.steps):
        ts = time.perf_counter()
        outs = step_and_refill()
        host_step.append(time.perf_counter() - ts)
        if args.verbose:
            sched_tokens.append(llm.step_stats()["scheduled_tokens"])
        for st in outs:
            tokens += 1  # one new token per returned request per step (no speculative decode)
    barrier()
    wall = time.perf_counter() - t0
    if args.verbose:
        ev = [e for e in llm.runner.step_events if e[1] is not None]
        per = [round(a.elapsed_time(b), 2) for a, b in ev]
        gaps = [round(ev[i][1].elapsed_time(ev[i + 1][0]), 2) for i in range(len(ev) - 1)]
        note(f"device ms per step: {per}")
        note(f"device gaps between steps (ms): {gaps}")
        note(f"host wall per step (ms): {[round(x * 1e3, 2) for x in host_step]}")
        note(f"scheduled tokens per step: {sched_tokens}")
        note(f"(tokens, finished, preempted, running, waiting) around the start of the timed region: "
             f"{trace[-(args.steps + args.warmup + 8):][:24]}")
    clocks = sampler.stop(since=t0)
    dev_ms = llm.runner.device_step_ms()
    llm.runner.time_steps = False
    launches = _lib.LAUNCHES[0] - launches0
    h2d = (llm.runner.h2d_bytes - h2d0) / args.steps
    d2h = (llm.runner.d2h_bytes - d2h0) / args.steps
    status = llm.runner.ops.read_status()

    def p50(xs):
        return sorted(xs)[len(xs) // 2] if xs else -1.0

    # latencies of the requests that got their first token / finished inside the timed region
    t = torch.tensor([dev_ms, wall * 1e3, p50(ttft_ms), p50(tpot_ms)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if dp:
            # replicas: tokens, launches and copies add up; the time is the slowest replica's
            sums = torch.tensor([tokens, launches, h2d, d2h, status], dtype=torch.float64, device="cuda")
            dist.all_reduce(sums, op=dist.ReduceOp.SUM)
            tokens, launches, h2d, d2h, status = (int(sums[0]), int(sums[1]), float(sums[2]),
                                                  float(sums[3]), int(sums[4]))
    dev_ms, wall_ms = float(t[0]), float(t[1])
    lat = {"p50_ttft_ms": round(float(t[2]), 2) if float(t[2]) >= 0 else None,
           "p50_tpot_ms": round(float(t[3]), 3) if float(t[3]) >= 0 else None,
           "note": "host clock, requests whose first token / last token fell inside the timed "
                   "region; worst rank"}
    value = tokens / (dev_ms / 1e3)
    e2e = tokens / (wall_ms / 1e3)
    # ---- extra keys, outside the timed region: the whole offline batch of the configuration
    # (C requests submitted at once, run to completion) and the online sweep at lower concurrency
    extras = {}
    if not args.no_extras and not dp:
        try:
            note("extras: draining the steady-state requests")
            while llm.has_unfinished_requests():       # drain the steady-state requests
                llm.step()
            torch.cuda.synchronize()
            t_submit.clear(); t_first.clear(); n_out.clear()
            note("extras: offline batch")
            extras["offline_batch"] = closed_loop(llm, torch, new_prompt, SamplingParams, C_total, C_total, OUT)
            sweep = []
            for c in (1, 8, 64):
                if c < C_total:
                    note(f"extras: concurrency {c}")
                    sweep.append(closed_loop(llm, torch, new_prompt, SamplingParams, c, max(2, min(2 * c, 64)), OUT))
            extras["online_sweep"] = sweep
            note("extras done")
        except Exception as e:   # the headline number above stands on its own
            extras["error"] = f"{type(e).__name__}: {e}"
    if rank == 0:
        print(json.dumps({
            "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s",
            "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": (value / PUBLISHED_BASELINE) if PUBLISHED_BASELINE else None,
            "dtype": "bf16", "data": "synthetic (uniform-random prompt ids, random-init weights)",
            "impl": "ours",
            "config": {"model": MODEL_LABELS.get(args.model, args.model), "global_batch": C_total,
                       "seq_len": IN + OUT,
                       "input_len": IN, "output_len": OUT,
                       "parallelism": (f"dp{world}" if dp else
                                       (f"tp{world}+ep{world}" if cfg.num_experts and world > 1
                                        else f"tp{world}")),
                       "collectives": ("none" if world == 1 or dp else
                                       ("GEMM + NCCL" if (args.unfused or getattr(llm.model, "tpf", None) is None)
                                        else "fused GEMM + reduce-scatter / all-gather kernels over peer memory")),
                       "mode": "continuous batching, steady state",
                       "max_num_batched_tokens": args.max_num_batched_tokens,
                       "l2": "the weights and the KV cache read in every step exceed L2 (126 MB) many times over",
                       "ramp_steps": ramp_steps, "cuda_graphs": not args.no_graphs,
                       "async_scheduling": not args.sync_scheduling,
                       **({"layers_override": args.layers} if args.layers > 0 else {})},
            "clocks": clocks,
            "latency": lat,
            "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "wall_ms_per_step": round(wall_ms / args.steps, 4)},
            "gpu_launches": int(launches), "output_tokens": tokens, "kernel_status": status,
            **extras,
        }))
    if world > 1:
        # Orderly teardown: nothing in flight on any rank, drop what holds the communicator (the
        # captured decode graphs contain NCCL kernels, the fused-TP context maps peer memory),
        # then destroy the process group. Destruction has been seen to block with live graphs,
        # so it runs beside a timer; the process leaves with code 0 either way.
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        llm.runner.graphs.clear()
        if getattr(llm.model, "tpf", None) is not None:
            llm.model.tpf = None
        import gc
        import threading
        gc.collect()
        torch.cuda.synchronize()
        done = threading.Event()

        def destroy():
            try:
                dist.destroy_process_group()
            finally:
                done.set()

        threading.Thread(target=destroy, daemon=True).start()
        done.wait(timeout=30)
        note("process group destroyed" if done.is_set() else "process group destruction timed out")
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
