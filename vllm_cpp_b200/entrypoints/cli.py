"""Command-line generation: ``python -m vllm_cpp_b200.entrypoints.cli --model DIR --prompt TEXT``.

Reference: ``examples/cli/main.cpp:69-89`` (same flags) and ``examples/tokenize/main.cpp``
(``--tokenize-only`` prints the ids of the prompt).
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("vllm_cpp_b200 cli")
    ap.add_argument("--model", required=True)
    ap.add_argument("--tokenizer-config", dest="tokenizer", default=None)
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--max-model-len", type=int, default=0)
    ap.add_argument("--tokenize-only", action="store_true")
    a = ap.parse_args(argv)
    if a.tokenize_only:
        from ..loader import load_tokenizer
        tok = load_tokenizer(a.tokenizer or a.model)
        ids = tok.encode(a.prompt)
        print(" ".join(map(str, ids)))
        print(f"{len(ids)} tokens", file=sys.stderr)
        return 0
    from ..config import EngineArgs
    from ..engine import LLM, SamplingParams
    from .async_llm import AsyncLLM
    llm = LLM(EngineArgs(model=a.model, tokenizer=a.tokenizer, device=a.device, max_model_len=a.max_model_len,
                         max_num_seqs=1))
    kw = dict(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, max_tokens=a.max_tokens)
    if a.seed is not None:
        kw["seed"] = a.seed
    sp = SamplingParams(**kw)
    if not a.stream:
        out = llm.generate([a.prompt], sp)[0]
        print(out.outputs[0].text)
        return 0
    from .. import _engine as E
    sp.output_kind = E.OutputKind.DELTA
    eng = AsyncLLM(llm)
    rid = eng.submit(llm.tokenizer.encode(a.prompt), sp)
    for item in eng.stream(rid):
        sys.stdout.write(item.text)
        sys.stdout.flush()
    sys.stdout.write("\n")
    eng.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
