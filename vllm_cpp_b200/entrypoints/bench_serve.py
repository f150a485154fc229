"""Closed-loop serving benchmark in the shape of ``vllm bench serve``: keeps ``--concurrency``
requests in flight against an in-process engine and reports request / token throughput and
TTFT, TPOT, ITL, E2EL (mean, median, p99).

``python -m vllm_cpp_b200.entrypoints.bench_serve --shape llama-3.1-8b --num-prompts 256 \
    --input-len 1024 --output-len 256 --concurrency 64``

Without ``--model`` a random-weight engine of the named synthetic shape is used and prompts
are uniform-random token ids; ``--dataset-path`` takes a ShareGPT-style JSON (needs a model
with a tokenizer).

Reference: ``examples/bench/bench_core.h:1-643``, ``examples/bench/main.cpp:70-92``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import threading
import time

import torch


def _pct(xs, q):
    if not xs:
        return 0.0
    s = sorted(xs)
    return s[min(len(s) - 1, int(round(q * (len(s) - 1))))]


def summarize(records: list[dict], wall: float) -> dict:
    ok = [r for r in records if not r.get("error")]
    out_tokens = sum(r["output_tokens"] for r in ok)
    in_tokens = sum(r["input_tokens"] for r in ok)
    ttft = [r["ttft"] for r in ok if r["ttft"] is not None]
    e2el = [r["e2el"] for r in ok]
    tpot = [(r["e2el"] - r["ttft"]) / (r["output_tokens"] - 1) for r in ok
            if r["ttft"] is not None and r["output_tokens"] > 1]
    itl = [x for r in ok for x in r["itl"]]

    def stats(xs):
        return {"mean_ms": 1e3 * (statistics.fmean(xs) if xs else 0.0), "median_ms": 1e3 * _pct(xs, 0.5),
                "p99_ms": 1e3 * _pct(xs, 0.99)}

    return {"completed": len(ok), "failed": len(records) - len(ok), "duration_s": wall,
            "request_throughput": len(ok) / wall if wall > 0 else 0.0,
            "output_throughput": out_tokens / wall if wall > 0 else 0.0,
            "total_token_throughput": (in_tokens + out_tokens) / wall if wall > 0 else 0.0,
            "total_input_tokens": in_tokens, "total_output_tokens": out_tokens,
            "ttft": stats(ttft), "tpot": stats(tpot), "itl": stats(itl), "e2el": stats(e2el)}


def run_closed_loop(engine, prompts: list[list[int]], make_params, concurrency: int) -> tuple[list[dict], float]:
    """``engine``: an AsyncLLM. One worker thread per in-flight slot pulls the next prompt."""
    lock = threading.Lock()
    nxt = [0]
    records: list[dict] = []

    def worker():
        while True:
            with lock:
                i = nxt[0]
                if i >= len(prompts):
                    return
                nxt[0] += 1
            ids = prompts[i]
            t0 = time.monotonic()
            rec = {"index": i, "input_tokens": len(ids), "output_tokens": 0, "ttft": None, "itl": [],
                   "token_ids": []}
            try:
                rid = engine.submit(ids, make_params(i))
                last = None
                for item in engine.stream(rid):
                    if item.error:
                        rec["error"] = item.error
                        break
                    if item.token_ids:
                        if rec["ttft"] is None:
                            rec["ttft"] = item.t - t0
                        elif last is not None:
                            rec["itl"].append((item.t - last) / len(item.token_ids))
                        last = item.t
                        rec["output_tokens"] += len(item.token_ids)
                        rec["token_ids"].extend(item.token_ids)
            except Exception as e:  # keep the other slots going
                rec["error"] = f"{type(e).__name__}: {e}"
            rec["e2el"] = time.monotonic() - t0
            with lock:
                records.append(rec)

    threads = [threading.Thread(target=worker, daemon=True) for _ in range(max(1, concurrency))]
    t0 = time.monotonic()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return records, time.monotonic() - t0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("vllm_cpp_b200 bench")
    ap.add_argument("--model", default=None)
    ap.add_argument("--shape", default="qwen3-0.6b", help="synthetic shape when --model is not given")
    ap.add_argument("--dataset-path", default=None)
    ap.add_argument("--num-prompts", type=int, default=64)
    ap.add_argument("--input-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--output-token-ids", default=None, help="write the generated ids as JSON")
    ap.add_argument("--max-num-batched-tokens", type=int, default=0)
    ap.add_argument("--num-blocks", type=int, default=0)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--async-scheduling", action="store_true")
    a = ap.parse_args(argv)
    from .. import _engine as E
    from ..config import EngineArgs, synthetic_config
    from ..engine import LLM, SamplingParams
    from .async_llm import AsyncLLM
    kw = dict(device=a.device, max_num_seqs=max(a.concurrency, 1), num_blocks=a.num_blocks,
              max_num_batched_tokens=a.max_num_batched_tokens, max_model_len=a.input_len + a.output_len + 16,
              async_scheduling=a.async_scheduling or None)
    if a.model:
        llm = LLM(EngineArgs(model=a.model, **kw))
    else:
        llm = LLM(EngineArgs(model_config=synthetic_config(a.shape), **kw))
    g = torch.Generator().manual_seed(a.seed)
    if a.dataset_path:
        if llm.tokenizer is None:
            raise SystemExit("--dataset-path needs a model with a tokenizer")
        data = json.load(open(a.dataset_path))
        texts = [d["conversations"][0]["value"] for d in data if d.get("conversations")][: a.num_prompts]
        prompts = [llm.tokenizer.encode(t)[: a.input_len] for t in texts]
    else:
        prompts = [torch.randint(0, llm.cfg.vocab_size, (a.input_len,), generator=g).tolist()
                   for _ in range(a.num_prompts)]

    def make_params(i):
        sp = SamplingParams(temperature=a.temperature, max_tokens=a.output_len, ignore_eos=True,
                            seed=a.seed + i if a.temperature > 0 else None, detokenize=False)
        sp.output_kind = E.OutputKind.DELTA
        return sp

    eng = AsyncLLM(llm)
    records, wall = run_closed_loop(eng, prompts, make_params, a.concurrency)
    eng.shutdown()
    res = summarize(records, wall)
    res["config"] = {"model": a.model or a.shape, "num_prompts": a.num_prompts, "input_len": a.input_len,
                     "output_len": a.output_len, "concurrency": a.concurrency}
    print(json.dumps(res, indent=1))
    if a.output_token_ids:
        with open(a.output_token_ids, "w") as f:
            json.dump({str(r["index"]): r["token_ids"] for r in records}, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
