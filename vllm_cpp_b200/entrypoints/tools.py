"""Small verification and measurement tools: ``python -m vllm_cpp_b200.entrypoints.tools <command>``.

``tokenize``         corpus file -> one line of ids per entry (reference ``examples/tokenize/main.cpp``:
                     ``#`` lines skipped, an empty line is the empty string, ``\\n \\r \\t \\\\`` escapes,
                     ``EMPTY`` for an entry without ids)
``dequant-nvfp4``    one packed NVFP4 weight of a safetensors shard -> raw little-endian bf16
                     (reference ``examples/dequant_nvfp4/main.cpp``; prints ``<out> <in>``)
``dump-container``   sorted per-tensor manifest of a ``.safetensors`` / ``.gguf`` file, one line
                     ``<name> <dtype> [dims] <nbytes> <sha256 of the first 64 KiB>`` and a ``TOTAL`` line
                     (reference ``examples/dump_container/main.cpp``)
``quant-gemm-bench`` times the quantised GEMMs (NVFP4 W4A16, fp8, bf16) at a model's projection
                     shapes (reference ``examples/quant_gemm_bench/main.cpp``, which does the same
                     for its block-quant CPU GEMM)
``dump-ops``         writes inputs and fp32 oracle outputs of the kernel library's ops to an ``.npz``
                     file, for comparing another implementation op by op (reference
                     ``tools/parity/dump_ops.py``)
``list-recipes``     the fusion-recipe catalogue: steps, available tiers, reference recipe, as JSON
``dump-greedy``      greedy token ids of a checkpoint for a prompt file, as JSON (reference
                     ``tools/parity/dump_27b_emulation_greedy.py``: the end-to-end golden)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time

import numpy as np
import torch

HASH_PREFIX_BYTES = 65536


# ------------------------------------------------------------------------------ tokenize
def unescape(line: str) -> str:
    out, i = [], 0
    while i < len(line):
        c = line[i]
        if c != "\\":
            out.append(c)
            i += 1
            continue
        if i + 1 >= len(line):
            raise ValueError(f"bad escape at end of corpus line: {line!r}")
        nxt = line[i + 1]
        table = {"n": "\n", "r": "\r", "t": "\t", "\\": "\\"}
        if nxt not in table:
            raise ValueError(f"bad escape in corpus line: {line!r}")
        out.append(table[nxt])
        i += 2
    return "".join(out)


def read_corpus(path: str) -> list[str]:
    text = open(path, "rb").read().decode("utf-8")
    lines = text.split("\n")
    if lines and lines[-1] == "":
        lines.pop()                      # the file's trailing newline makes no entry
    return [unescape(l) for l in lines if not l.startswith("#")]


def cmd_tokenize(a) -> int:
    from ..loader import load_tokenizer
    tok = load_tokenizer(a.tokenizer)
    for entry in read_corpus(a.corpus):
        ids = tok.encode(entry)
        print(" ".join(map(str, ids)) if len(ids) else "EMPTY")
    return 0


# ------------------------------------------------------------------------------ dequant-nvfp4
def cmd_dequant_nvfp4(a) -> int:
    from ..loader.safetensors import SafetensorsFile
    from ..ops.quant import ref_dequant_nvfp4
    f = SafetensorsFile(a.shard)
    packed, sf, g = f.get(a.weight), f.get(a.scale), f.get(a.scale2)
    if packed.dtype != torch.uint8:
        raise SystemExit(f"tensor '{a.weight}' has dtype {packed.dtype}, expected uint8")
    if sf.dtype not in (torch.float8_e4m3fn, torch.uint8):
        raise SystemExit(f"tensor '{a.scale}' has dtype {sf.dtype}, expected float8_e4m3fn")
    w = ref_dequant_nvfp4(packed, sf.view(torch.uint8), g.float().reshape(1)).to(torch.bfloat16)
    w.contiguous().view(torch.int16).numpy().astype("<i2").tofile(a.out)
    print(w.shape[0], w.shape[1])
    return 0


# ------------------------------------------------------------------------------ dump-container
def manifest_lines(path: str) -> list[str]:
    rows = []
    if path.endswith(".gguf"):
        from ..loader.gguf import GGUFFile
        g = GGUFFile(path)
        for name, info in g.tensors.items():
            raw = g.raw(name)
            rows.append((name, f"ggml{info.ggml_type}", list(info.shape), int(raw.size),
                         hashlib.sha256(raw[:HASH_PREFIX_BYTES].tobytes()).hexdigest()))
    else:
        from ..loader.safetensors import SafetensorsFile
        f = SafetensorsFile(path)
        for name, (dt, shape, b, en) in f.entries.items():
            lo = f.data_start + b
            raw = f._mm[lo: lo + min(en - b, HASH_PREFIX_BYTES)] if en > b else b""
            rows.append((name, dt, list(shape), en - b, hashlib.sha256(raw).hexdigest()))
    rows.sort()
    out = [f"{n} {d} [{','.join(map(str, s))}] {nb} {h}" for n, d, s, nb, h in rows]
    out.append(f"TOTAL {len(rows)} tensors")
    return out


def cmd_dump_container(a) -> int:
    print("\n".join(manifest_lines(a.path)))
    return 0


# ------------------------------------------------------------------------------ quant-gemm-bench
MODEL_GEMMS = {
    # (name, N, K) of the per-layer projections; M is the token count of the step
    "qwen3.6-27b": [("qkv", 8192, 5120), ("o", 5120, 6144), ("gate_up", 34816, 5120), ("down", 5120, 17408)],
    "llama-3.1-8b": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)],
}


def cmd_quant_gemm_bench(a) -> int:
    from .. import ops
    from ..ops import quant
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for name, N, K in MODEL_GEMMS[a.shape]:
        for M in a.m:
            x = (torch.randn(M, K, device=dev) * 0.1).to(torch.bfloat16)
            w = (torch.randn(N, K, device=dev) * 0.02)
            packed, sf, g = quant.ref_quant_nvfp4_weights(w)
            wb = w.to(torch.bfloat16)
            w8 = w.to(torch.float8_e4m3fn)
            x8 = x.to(torch.float8_e4m3fn)
            one = torch.ones(1, device=dev)
            sf_chunks = quant.nvfp4_sf_chunks(sf, 256)
            g_a = (448.0 * 6.0 / x.float().abs().max()).reshape(1)
            xq, xsf = quant.quant_nvfp4(x, g_a, swizzle=True)
            w_ch = torch.ones(N, device=dev)
            x8r, xs = quant.quant_fp8_rowwise(x)
            arms = {"bf16": lambda: ops.gemm(x, wb),
                    "fp8": lambda: quant.gemm_fp8(x8, w8, one, one),
                    # W8A8 as the models run it: one scale per token and per output channel, the
                    # row-wise quantiser in front
                    "fp8+quant": lambda: (quant.quant_fp8_rowwise(x, out=x8r, scales=xs),
                                          quant.gemm_fp8(x8r, w8, xs, w_ch))}
            if M <= 128:
                arms["w4a16"] = lambda: quant.gemm_w4a16(x, packed, sf, g)
            if K % 256 == 0:
                # the GEMM alone (activations already quantised), then with the quantiser in front
                arms["w4a4"] = lambda: quant.gemm_nvfp4(xq, xsf, g_a, packed, sf_chunks, g)
                arms["w4a4+quant"] = lambda: quant.gemm_nvfp4(
                    *quant.quant_nvfp4(x, g_a, swizzle=True, out=(xq, xsf)), g_a, packed, sf_chunks, g)
            for arm, fn in arms.items():
                for _ in range(3):
                    fn()
                best = float("inf")
                for _ in range(a.repeat):
                    flush.zero_()                       # weights leave L2 between timed runs
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    fn()
                    e1.record()
                    torch.cuda.synchronize()
                    best = min(best, e0.elapsed_time(e1))
                wbytes = {"bf16": 2.0, "fp8": 1.0, "fp8+quant": 1.0}.get(arm, 0.5 + 1 / 16) * N * K
                rows.append({"proj": name, "M": M, "N": N, "K": K, "arm": arm, "ms": round(best, 4),
                             "tflops": round(2.0 * M * N * K / best / 1e9, 1),
                             "weight_gbs": round(wbytes / best / 1e6, 1)})
                print(json.dumps(rows[-1]), flush=True)
    return 0


# ------------------------------------------------------------------------------ list-recipes
def cmd_list_recipes(a) -> int:
    from ..ops import recipes
    json.dump(recipes.describe(), sys.stdout, indent=1)
    sys.stdout.write("\n")
    return 0


# ------------------------------------------------------------------------------ dump-ops
def cmd_dump_ops(a) -> int:
    """Inputs are drawn from a seeded CPU generator; outputs come from the fp32 references in
    ``ops.reference`` (the same functions the kernel numerics tests compare against)."""
    from ..ops import reference as R
    g = torch.Generator().manual_seed(a.seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    T, H, I, V = 24, 256, 512, 1000
    x, w, res = rn(T, H), rn(H) * 0.1 + 1, rn(T, H)
    out: dict[str, np.ndarray] = {}

    def put(name, **tensors):
        for k, t in tensors.items():
            out[f"{name}.{k}"] = t.detach().float().numpy() if t.is_floating_point() else t.numpy()

    put("rmsnorm", x=x, weight=w, out=R.rmsnorm(x, w, 1e-6)[0])
    y, r2 = R.rmsnorm(x, w, 1e-6, residual=res)
    put("add_rmsnorm", x=x, residual=res, weight=w, out=y, residual_out=r2)
    put("layernorm", x=x, weight=w, bias=res[0], out=R.layernorm(x, w, res[0], 1e-5))
    gu = rn(T, 2 * I)
    for kind, nm in ((0, "silu_and_mul"), (1, "gelu_tanh_and_mul"), (2, "gelu_erf_and_mul")):
        put(nm, x=gu, out=R.act_and_mul(gu, kind))
    a_, b_ = rn(T, H), rn(I, H)
    put("gemm", a=a_, w=b_, out=R.gemm(a_, b_, out_dtype=torch.float32))
    inv = R.rope_inv_freq(64, 10000.0)
    put("rope_table", inv_freq=inv, out=R.rope_table(inv, 128))
    logits = rn(T, V)
    put("argmax", logits=logits, out=logits.argmax(-1))
    put("softmax", logits=logits, out=torch.softmax(logits, -1))
    np.savez(a.out, **out)
    print(f"wrote {len(out)} arrays to {a.out}")
    return 0


# ------------------------------------------------------------------------------ dump-greedy
def cmd_dump_greedy(a) -> int:
    from ..config import EngineArgs
    from ..engine import LLM, SamplingParams
    llm = LLM(EngineArgs(model=a.model, device=a.device, max_num_seqs=8))
    prompts = read_corpus(a.prompts)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=a.max_tokens))
    rec = [{"prompt": p, "prompt_token_ids": list(o.prompt_token_ids),
            "token_ids": list(o.outputs[0].token_ids), "text": o.outputs[0].text}
           for p, o in zip(prompts, outs)]
    json.dump(rec, open(a.out, "w") if a.out != "-" else sys.stdout, indent=1)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("vllm_cpp_b200 tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("tokenize")
    p.add_argument("tokenizer", help="tokenizer.json, a model directory or a .gguf file")
    p.add_argument("corpus")
    p.set_defaults(fn=cmd_tokenize)
    p = sub.add_parser("dequant-nvfp4")
    for n in ("shard", "weight", "scale", "scale2", "out"):
        p.add_argument(n)
    p.set_defaults(fn=cmd_dequant_nvfp4)
    p = sub.add_parser("dump-container")
    p.add_argument("path")
    p.set_defaults(fn=cmd_dump_container)
    p = sub.add_parser("quant-gemm-bench")
    p.add_argument("--shape", default="qwen3.6-27b", choices=sorted(MODEL_GEMMS))
    p.add_argument("--m", type=int, nargs="+", default=[1, 16, 64, 256, 2048])
    p.add_argument("--repeat", type=int, default=10)
    p.set_defaults(fn=cmd_quant_gemm_bench)
    p = sub.add_parser("dump-ops")
    p.add_argument("out")
    p.add_argument("--seed", type=int, default=0)
    p.set_defaults(fn=cmd_dump_ops)
    p = sub.add_parser("list-recipes")
    p.set_defaults(fn=cmd_list_recipes)
    p = sub.add_parser("dump-greedy")
    p.add_argument("--model", required=True)
    p.add_argument("--prompts", required=True)
    p.add_argument("--out", default="-")
    p.add_argument("--max-tokens", type=int, default=32)
    p.add_argument("--device", default="cuda")
    p.set_defaults(fn=cmd_dump_greedy)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    raise SystemExit(main())
