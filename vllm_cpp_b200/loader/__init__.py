"""Checkpoint loading: a Hugging Face model directory (config.json + *.safetensors +
tokenizer.json) or a single GGUF file -> (ModelConfig, iterator of HF-named bf16 tensors,
tokenizer). Quantised checkpoints (NVFP4 in the compressed-tensors and ModelOpt layouts, FP8
per-tensor / per-channel / 128x128-block) are expanded to bf16 while streaming, so every model
class sees plain weights; the quantised GEMM paths re-quantise from those when enabled.

Also writes small random checkpoints (config + safetensors + a byte-level BPE tokenizer) so the
whole engine can be exercised without any download.

Reference: ``src/vllm/model_executor/model_loader/{safetensors,gguf,hf_config,nvfp4_dequant}.cpp``,
``src/vllm/entrypoints/model_loader.cpp:273-366``; synthetic model/tokenizer builders in
``examples/bench/bench_core.h:187-330``.
"""
from __future__ import annotations

import json
import os
from typing import Iterator, Optional

import torch

from ..config import ModelConfig, load_model_config, model_config_from_hf
from .safetensors import SafetensorsFile, open_shards, save_file  # noqa: F401

# e2m1 code -> value (sign in bit 3)
_FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                            -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=torch.float32)


def dequant_nvfp4(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor,
                  scale_is_divisor: bool) -> torch.Tensor:
    """``packed`` uint8 [N, K/2] (low nibble = even column), ``block_scale`` fp8-e4m3 [N, K/16],
    one fp32 per-tensor scale. compressed-tensors stores the per-tensor scale as a divisor
    (``weight_global_scale``), ModelOpt as a multiplier (``weight_scale_2``)."""
    n, kh = packed.shape
    p = packed.to(torch.int64)
    vals = torch.stack([_FP4_VALUES[p & 15], _FP4_VALUES[p >> 4]], dim=-1).reshape(n, kh * 2)
    s = block_scale.to(torch.float32)
    g = global_scale.to(torch.float32).reshape(-1)[0]
    s = s / g if scale_is_divisor else s * g
    out = vals.reshape(n, -1, 16) * s.reshape(n, -1, 1)
    return out.reshape(n, kh * 2).to(torch.bfloat16)


def dequant_fp8(weight: torch.Tensor, scale: torch.Tensor, block: Optional[tuple] = None) -> torch.Tensor:
    """fp8-e4m3 weight with a per-tensor, per-output-channel or [ceil(N/bn), ceil(K/bk)] block
    scale (multiplier)."""
    w = weight.to(torch.float32)
    s = scale.to(torch.float32)
    if s.numel() == 1:
        return (w * s.reshape(())).to(torch.bfloat16)
    if s.dim() == 2 and s.shape[0] == w.shape[0] and s.shape[1] == 1 or s.dim() == 1 and s.numel() == w.shape[0]:
        return (w * s.reshape(-1, 1)).to(torch.bfloat16)
    bn, bk = block or (128, 128)
    s_full = s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
    return (w * s_full).to(torch.bfloat16)


_QUANT_SUFFIXES = (".weight_packed", ".weight_scale", ".weight_global_scale", ".weight_scale_2",
                   ".weight_scale_inv", ".input_global_scale", ".input_scale", ".k_scale", ".v_scale")


def _iter_safetensors_dequant(model_dir: str, quant: dict | None) -> Iterator[tuple[str, torch.Tensor]]:
    """Streams tensors shard by shard; groups the pieces of a quantised linear layer (they sit
    in the same shard) and yields the bf16 weight under the plain ``<prefix>.weight`` name."""
    block = None
    if quant and quant.get("weight_block_size"):
        block = tuple(quant["weight_block_size"])
    for sf in open_shards(model_dir):
        keys = list(sf.keys())
        keyset = set(keys)
        for k in keys:
            if k.endswith(_QUANT_SUFFIXES):
                if k.endswith(".weight_packed"):
                    pre = k[: -len(".weight_packed")]
                    yield pre + ".weight", dequant_nvfp4(sf.get(k), sf.get(pre + ".weight_scale"),
                                                         sf.get(pre + ".weight_global_scale"), True)
                continue
            t = sf.get(k)
            if k.endswith(".weight"):
                pre = k[: -len(".weight")]
                if t.dtype == torch.uint8 and pre + ".weight_scale_2" in keyset:
                    t = dequant_nvfp4(t, sf.get(pre + ".weight_scale"), sf.get(pre + ".weight_scale_2"), False)
                elif t.dtype in (torch.float8_e4m3fn,):
                    if pre + ".weight_scale_inv" in keyset:
                        t = dequant_fp8(t, sf.get(pre + ".weight_scale_inv"), block)
                    elif pre + ".weight_scale" in keyset:
                        t = dequant_fp8(t, sf.get(pre + ".weight_scale"), block)
                    else:
                        t = t.to(torch.bfloat16)
            yield k, t
        sf.close()


def _tokenizer_from_gguf(g):
    from .. import _engine as E
    m = g.metadata
    toks = m.get("tokenizer.ggml.tokens")
    if not toks:
        return None
    enc = [t.encode("utf-8") if isinstance(t, str) else bytes(t) for t in toks]
    merges = [x.encode("utf-8") if isinstance(x, str) else bytes(x) for x in m.get("tokenizer.ggml.merges", [])]
    types = [int(x) for x in m.get("tokenizer.ggml.token_type", [1] * len(enc))]
    model = m.get("tokenizer.ggml.model", "gpt2")
    return E.Tokenizer.from_gguf(model, m.get("tokenizer.ggml.pre", "default"), enc, merges, types,
                                 int(m.get("tokenizer.ggml.bos_token_id", -1)),
                                 int(m.get("tokenizer.ggml.eos_token_id", -1)),
                                 bool(m.get("tokenizer.ggml.add_bos_token", model == "llama")),
                                 bool(m.get("tokenizer.ggml.add_eos_token", False)))


def load_tokenizer(path: str):
    """Tokenizer from a model directory, a tokenizer.json path or a GGUF file (None if absent)."""
    from .. import _engine as E
    if path.endswith(".gguf"):
        from .gguf import GGUFFile
        g = GGUFFile(path)
        try:
            return _tokenizer_from_gguf(g)
        finally:
            g.close()
    if os.path.isdir(path):
        if not os.path.exists(os.path.join(path, "tokenizer.json")):
            return None
        return E.Tokenizer.from_dir(path)
    with open(path, encoding="utf-8") as f:
        tj = f.read()
    cfgp = os.path.join(os.path.dirname(path), "tokenizer_config.json")
    cj = open(cfgp, encoding="utf-8").read() if os.path.exists(cfgp) else ""
    return E.Tokenizer.from_hf_json(tj, cj)


def load_model_dir(model: str, tokenizer: Optional[str] = None):
    """-> (ModelConfig, iterator of (hf_name, tensor), tokenizer or None)."""
    if model.endswith(".gguf"):
        from .gguf import GGUFFile, iter_hf_tensors
        g = GGUFFile(model)
        cfg = model_config_from_hf(g.hf_config())
        tok = load_tokenizer(tokenizer) if tokenizer else _tokenizer_from_gguf(g)
        return cfg, iter_hf_tensors(g), tok
    cfg = load_model_config(model)
    with open(os.path.join(model, "config.json")) as f:
        raw = json.load(f)
    quant = raw.get("quantization_config") or (raw.get("text_config") or {}).get("quantization_config")
    tok = load_tokenizer(tokenizer or model)
    return cfg, _iter_safetensors_dequant(model, quant), tok


# ------------------------------------------------------------------ synthetic checkpoints
def synthetic_tokenizer_json(vocab_size: int, specials=("<|endoftext|>", "<|im_start|>", "<|im_end|>")) -> str:
    """A byte-level BPE tokenizer.json with 256 byte tokens, deterministic merges of frequent
    English byte pairs and the given special tokens at the top of the id range."""
    from .. import _engine as E
    byte_chars = [chr(E.byte_to_codepoint(b)) for b in range(256)]
    vocab = {c: i for i, c in enumerate(byte_chars)}
    merges = []
    sp = byte_chars[ord(" ")]
    seeds = ["th", "he", "in", "er", "an", "re", "on", "at", "en", "nd", "ti", "es", "or", "te", "of",
             "ed", "is", "it", "al", "ar", "st", "to", "nt", "ng", "se", "ha", "as", "ou", "io", "le",
             sp + "t", sp + "a", sp + "s", sp + "w", sp + "o", sp + "i", sp + "c", sp + "b", sp + "p",
             "the", sp + "th", sp + "the", "ing", "and", sp + "an", sp + "and", "ion", "ent", sp + "of",
             sp + "to", sp + "in", "tion", "ther", "ould"]
    budget = vocab_size - 256 - len(specials)
    for s in seeds:
        if len(merges) >= budget:
            break
        if s in vocab or len(s) < 2:
            continue
        # split so that both halves already exist
        for cut in range(len(s) - 1, 0, -1):
            if s[:cut] in vocab and s[cut:] in vocab:
                merges.append([s[:cut], s[cut:]])
                vocab[s] = len(vocab)
                break
    added = []
    next_id = max(len(vocab), vocab_size - len(specials))
    for i, s in enumerate(specials):
        added.append({"id": next_id + i, "content": s, "single_word": False, "lstrip": False,
                      "rstrip": False, "normalized": False, "special": True})
    pattern = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
               r"|\s*[\r\n]+|\s+(?!\S)|\s+")
    tj = {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": added,
        "normalizer": None,
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": pattern}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False}]},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": "",
                  "end_of_word_suffix": "", "fuse_unk": False, "byte_fallback": False,
                  "ignore_merges": False, "vocab": vocab, "merges": merges},
    }
    return json.dumps(tj, ensure_ascii=False)


def hf_config_dict(cfg: ModelConfig) -> dict:
    """config.json for a ModelConfig of the dense / Qwen3-MoE families."""
    d = {
        "architectures": [cfg.architecture], "hidden_size": cfg.hidden_size,
        "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
        "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
        "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
        "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope.theta,
        "max_position_embeddings": cfg.max_position_embeddings,
        "tie_word_embeddings": cfg.tie_word_embeddings, "torch_dtype": "bfloat16",
        "eos_token_id": cfg.eos_token_id, "bos_token_id": cfg.bos_token_id,
        "hidden_act": cfg.hidden_act,
    }
    if cfg.num_experts:
        d.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                 moe_intermediate_size=cfg.moe_intermediate_size, norm_topk_prob=True)
    return d


def write_synthetic_checkpoint(out_dir: str, cfg: ModelConfig, seed: int = 0, std: float = 0.02,
                               with_tokenizer: bool = True) -> str:
    """Random N(0, std) weights in HF layout + config.json (+ tokenizer files)."""
    from ..models import registry
    os.makedirs(out_dir, exist_ok=True)
    _, cls = registry.resolve(cfg.architecture)
    model = cls(cfg, device="cpu")
    captured: dict[str, torch.Tensor] = {}
    real_load = model.load_weights

    def capture(named):
        def tee():
            for n, t in named:
                captured[n] = t.detach().to(torch.bfloat16).contiguous().cpu()
                yield n, t
        real_load(tee())

    model.load_weights = capture
    model.init_random(seed, std) if "std" in model.init_random.__code__.co_varnames else model.init_random(seed)
    save_file(captured, os.path.join(out_dir, "model.safetensors"), {"format": "pt"})
    hf = hf_config_dict(cfg)
    if with_tokenizer:
        hf["eos_token_id"] = cfg.vocab_size - 3      # <|endoftext|> in the synthetic tokenizer
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(hf, f, indent=1)
    if with_tokenizer:
        specials = ("<|endoftext|>", "<|im_start|>", "<|im_end|>")
        with open(os.path.join(out_dir, "tokenizer.json"), "w", encoding="utf-8") as f:
            f.write(synthetic_tokenizer_json(cfg.vocab_size, specials))
        with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
            json.dump({"eos_token": "<|endoftext|>", "pad_token": "<|endoftext|>",
                       "chat_template": ("{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}"
                                         "<|im_end|>\n{% endfor %}{% if add_generation_prompt %}"
                                         "<|im_start|>assistant\n{% endif %}")}, f)
    return out_dir
