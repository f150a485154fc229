"""Inputs for the reference arm of the benchmark: a random-init checkpoint directory in
Hugging Face layout (config.json, tokenizer.json, bf16 safetensors shards) and a ShareGPT-style
prompt file, for the unmodified reference engine to load through its own model loader
(reference: src/vllm/entrypoints/model_loader.cpp `LoadedEngine::FromModelDir`) and its own
bench tool (reference: examples/bench/main.cpp, `--model`, `--dataset-path`).

Stand-alone on purpose: it imports nothing from this repository's package, so the reference arm
shares no code with the engine it is compared with. Only torch (random numbers, bf16 bytes) and
the standard library are used; the safetensors container is written by hand (8-byte little-endian
header length, JSON header, raw tensor bytes).
"""
from __future__ import annotations

import json
import os
import struct

SHAPES = {
    # BASELINE config 2
    "llama-3.1-8b": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096,
        num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
        max_position_embeddings=131072, tie_word_embeddings=False, hidden_act="silu",
        attention_bias=False, mlp_bias=False,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)),
    # BASELINE config 1
    "qwen3-0.6b": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=1024,
        num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
        intermediate_size=3072, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1000000.0,
        max_position_embeddings=40960, tie_word_embeddings=True, hidden_act="silu",
        attention_bias=False),
    # BASELINE config 3
    "qwen3-coder-30b-a3b": dict(
        architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=2048,
        num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
        intermediate_size=6144, moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8,
        norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], vocab_size=151936,
        rms_norm_eps=1e-6, rope_theta=10000000.0, max_position_embeddings=262144,
        tie_word_embeddings=False, hidden_act="silu", attention_bias=False),
}


def _byte_to_unicode() -> list[str]:
    """GPT-2's printable stand-in for each byte value (the byte-level BPE alphabet)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    out, extra = {}, 0
    for b in range(256):
        if b in keep:
            out[b] = chr(b)
        else:
            out[b] = chr(256 + extra)
            extra += 1
    return [out[b] for b in range(256)]


def tokenizer_json(vocab_size: int) -> str:
    """A byte-level BPE tokenizer whose vocabulary has no holes: ids 0..255 are the byte tokens
    (so every digit is one token), every other id is a unique filler string that no merge
    produces but that decodes to text. The last id is the end-of-text special token."""
    alphabet = _byte_to_unicode()
    vocab = {c: i for i, c in enumerate(alphabet)}
    letters = "abcdefghijklmnopqrstuvwxyz"
    i = 256
    while i < vocab_size - 1:
        n, s = i, ""
        while True:
            s = letters[n % 26] + s
            n //= 26
            if n == 0:
                break
        vocab["q" + s + "x"] = i          # at least three characters: cannot collide with a byte
        i += 1
    added = [{"id": vocab_size - 1, "content": "<|endoftext|>", "single_word": False,
              "lstrip": False, "rstrip": False, "normalized": False, "special": True}]
    pattern = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?[\p{L}\p{M}]+|\p{N}| ?[^\s\p{L}\p{M}\p{N}]+[\r\n]*"
               r"|\s*[\r\n]+|\s+(?!\S)|\s+")
    doc = {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": added,
        "normalizer": None,
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": pattern}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False,
             "use_regex": False}]},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False,
                    "use_regex": False},
        "model": {"type": "BPE", "dropout": None, "unk_token": None,
                  "continuing_subword_prefix": "", "end_of_word_suffix": "", "fuse_unk": False,
                  "byte_fallback": False, "ignore_merges": False, "vocab": vocab, "merges": []},
    }
    return json.dumps(doc, ensure_ascii=False)


def _tensor_list(cfg: dict) -> list[tuple[str, tuple[int, ...], str]]:
    """(HF tensor name, shape, kind) for the dense / Qwen3-MoE decoder families; kind is
    'w' (N(0, std)) or 'one' (norm weights)."""
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nq, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    V, I = cfg["vocab_size"], cfg["intermediate_size"]
    qk_norm = cfg["model_type"] in ("qwen3", "qwen3_moe")
    E, MI = cfg.get("num_experts", 0), cfg.get("moe_intermediate_size", 0)
    out = [("model.embed_tokens.weight", (V, H), "w")]
    for l in range(L):
        p = f"model.layers.{l}."
        out += [(p + "input_layernorm.weight", (H,), "one"),
                (p + "self_attn.q_proj.weight", (nq * D, H), "w"),
                (p + "self_attn.k_proj.weight", (nkv * D, H), "w"),
                (p + "self_attn.v_proj.weight", (nkv * D, H), "w"),
                (p + "self_attn.o_proj.weight", (H, nq * D), "w"),
                (p + "post_attention_layernorm.weight", (H,), "one")]
        if qk_norm:
            out += [(p + "self_attn.q_norm.weight", (D,), "one"),
                    (p + "self_attn.k_norm.weight", (D,), "one")]
        if E:
            out.append((p + "mlp.gate.weight", (E, H), "w"))
            for e in range(E):
                q = p + f"mlp.experts.{e}."
                out += [(q + "gate_proj.weight", (MI, H), "w"), (q + "up_proj.weight", (MI, H), "w"),
                        (q + "down_proj.weight", (H, MI), "w")]
        else:
            out += [(p + "mlp.gate_proj.weight", (I, H), "w"), (p + "mlp.up_proj.weight", (I, H), "w"),
                    (p + "mlp.down_proj.weight", (H, I), "w")]
    out.append(("model.norm.weight", (H,), "one"))
    if not cfg.get("tie_word_embeddings", False):
        out.append(("lm_head.weight", (V, H), "w"))
    return out


def write_checkpoint(out_dir: str, model: str, seed: int = 0, std: float = 0.02,
                     shard_bytes: int = 4 << 30, layers: int | None = None) -> str:
    """Writes config.json, tokenizer.json, tokenizer_config.json and model-XXXXX.safetensors
    shards of random N(0, std) bf16 weights (norm weights are ones). Random numbers come from the
    GPU when there is one (an 8B checkpoint takes seconds instead of minutes)."""
    import torch
    cfg = dict(SHAPES[model])
    if layers:
        cfg["num_hidden_layers"] = layers
    cfg.update(torch_dtype="bfloat16", bos_token_id=cfg["vocab_size"] - 1,
               eos_token_id=cfg["vocab_size"] - 1)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    with open(os.path.join(out_dir, "tokenizer.json"), "w", encoding="utf-8") as f:
        f.write(tokenizer_json(cfg["vocab_size"]))
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|endoftext|>", "bos_token": "<|endoftext|>",
                   "tokenizer_class": "PreTrainedTokenizerFast"}, f)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)
    tensors = _tensor_list(cfg)
    shards, cur, cur_bytes = [], [], 0
    for t in tensors:
        nbytes = 2
        for d in t[1]:
            nbytes *= d
        if cur and cur_bytes + nbytes > shard_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append(t)
        cur_bytes += nbytes
    if cur:
        shards.append(cur)
    weight_map = {}
    for si, shard in enumerate(shards):
        fname = f"model-{si + 1:05d}-of-{len(shards):05d}.safetensors"
        header, off = {}, 0
        for name, shape, _ in shard:
            n = 2
            for d in shape:
                n *= d
            header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]}
            off += n
            weight_map[name] = fname
        hj = json.dumps(header, separators=(",", ":")).encode()
        hj += b" " * ((8 - len(hj) % 8) % 8)
        with open(os.path.join(out_dir, fname), "wb") as f:
            f.write(struct.pack("<Q", len(hj)))
            f.write(hj)
            for name, shape, kind in shard:
                if kind == "one":
                    t = torch.ones(shape, dtype=torch.bfloat16)
                else:
                    t = (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std
                         ).to(torch.bfloat16).cpu()
                f.write(t.contiguous().view(torch.uint8).numpy().tobytes())
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    return out_dir


def write_prompts(path: str, num_prompts: int, input_len: int, seed: int = 1) -> str:
    """ShareGPT-format file whose first turns are strings of ``input_len`` random decimal digits:
    the number pre-tokenisation rule makes every digit its own token, so each prompt is exactly
    ``input_len`` tokens under `tokenizer_json`."""
    import random
    rng = random.Random(seed)
    data = [{"id": str(i), "conversations": [
        {"from": "human", "value": "".join(rng.choice("0123456789") for _ in range(input_len))}]}
        for i in range(num_prompts)]
    with open(path, "w") as f:
        json.dump(data, f)
    return path


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b", choices=sorted(SHAPES))
    ap.add_argument("--out", required=True)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--num-prompts", type=int, default=0)
    ap.add_argument("--input-len", type=int, default=1024)
    a = ap.parse_args()
    write_checkpoint(a.out, a.model, layers=a.layers or None)
    if a.num_prompts:
        write_prompts(os.path.join(a.out, "prompts.json"), a.num_prompts, a.input_len)
    print(a.out)
