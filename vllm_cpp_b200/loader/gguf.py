"""GGUF v3 reader and block-quant dequantisation (F32, F16, BF16, Q4_0, Q8_0, Q3_K, Q4_K,
Q5_K, Q6_K), vectorised with numpy.

Gives: typed key/value metadata, tensor infos (name, shape in torch order, ggml type, file
offset), ``HF-style config`` derived from the ``<arch>.*`` keys, the tokenizer vocabulary
(tokens / merges / token types) and dequantised tensors.

Reference: ``src/vllm/model_executor/model_loader/gguf_reader.cpp`` (539 lines),
``gguf_dequant.cpp`` and ``gguf_keep_quant.cpp``.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
_VAL = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q",
        12: "<d"}
# ggml type -> (block elements, block bytes)
GGML = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 8: ("Q8_0", 32, 34),
        11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176),
        14: ("Q6_K", 256, 210), 30: ("BF16", 1, 2)}


class GGUFError(ValueError):
    pass


@dataclass
class GGUFTensorInfo:
    name: str
    shape: tuple        # torch order (outermost first)
    ggml_type: int
    offset: int         # absolute file offset
    nbytes: int


class GGUFFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        size = len(self._mm)
        magic, version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise GGUFError(f"{path}: not a GGUF file")
        if version not in (2, 3):
            raise GGUFError(f"{path}: unsupported GGUF version {version}")
        n_tensors, n_kv = self._unpack("<QQ")
        if n_tensors > 1 << 20 or n_kv > 1 << 20:
            raise GGUFError(f"{path}: implausible counts")
        self.metadata: dict = {}
        for _ in range(n_kv):
            k = self._string()
            (t,) = self._unpack("<I")
            self.metadata[k] = self._value(t)
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            if nd > 8:
                raise GGUFError(f"{path}: tensor {name!r} has {nd} dims")
            dims = self._unpack("<" + "Q" * nd)
            gt, off = self._unpack("<IQ")
            infos.append((name, tuple(reversed(dims)), gt, off))
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (self._pos + align - 1) // align * align
        self.tensors: dict[str, GGUFTensorInfo] = {}
        for name, shape, gt, off in infos:
            if gt not in GGML:
                raise GGUFError(f"{path}: tensor {name!r} has unsupported ggml type {gt}")
            _, be, bb = GGML[gt]
            n = int(np.prod(shape)) if shape else 1
            if n % be:
                raise GGUFError(f"{path}: tensor {name!r} size is not a multiple of its block")
            nbytes = n // be * bb
            ab = self.data_start + off
            if ab + nbytes > size:
                raise GGUFError(f"{path}: tensor {name!r} runs past the end of the file")
            self.tensors[name] = GGUFTensorInfo(name, shape, gt, ab, nbytes)

    # ---- primitive readers (bounds-checked)
    def _unpack(self, fmt):
        n = struct.calcsize(fmt)
        if self._pos + n > len(self._mm):
            raise GGUFError(f"{self.path}: truncated header")
        v = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += n
        return v

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        if n > 1 << 28 or self._pos + n > len(self._mm):
            raise GGUFError(f"{self.path}: string length out of bounds")
        s = bytes(self._mm[self._pos:self._pos + n]).decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, t):
        if t in _VAL:
            return self._unpack(_VAL[t])[0]
        if t == 8:
            return self._string()
        if t == 9:
            (et,) = self._unpack("<I")
            (n,) = self._unpack("<Q")
            if n > 1 << 28:
                raise GGUFError(f"{self.path}: array too long")
            if et in _VAL:
                fmt = _VAL[et]
                sz = struct.calcsize(fmt)
                if self._pos + n * sz > len(self._mm):
                    raise GGUFError(f"{self.path}: truncated array")
                arr = np.frombuffer(self._mm, dtype=np.dtype(fmt), count=n, offset=self._pos).tolist()
                self._pos += n * sz
                return arr
            return [self._value(et) for _ in range(n)]
        raise GGUFError(f"{self.path}: unknown metadata value type {t}")

    # ---- tensors
    def raw(self, name: str) -> np.ndarray:
        i = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=i.nbytes, offset=i.offset)

    def get(self, name: str, dtype=torch.bfloat16) -> torch.Tensor:
        i = self.tensors[name]
        return torch.from_numpy(dequantize(self.raw(name), i.ggml_type, i.shape)).to(dtype)

    def architecture(self) -> str:
        return self.metadata.get("general.architecture", "llama")

    def hf_config(self) -> dict:
        """HF-style config dict from the ``<arch>.*`` metadata."""
        a, m = self.architecture(), self.metadata

        def g(k, d=None):
            return m.get(f"{a}.{k}", d)
        heads = int(g("attention.head_count", 32))
        hidden = int(g("embedding_length", 4096))
        arch_map = {"llama": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM",
                    "qwen2": "Qwen2ForCausalLM", "qwen3moe": "Qwen3MoeForCausalLM",
                    "gemma": "GemmaForCausalLM", "gemma2": "Gemma2ForCausalLM",
                    "gemma3": "Gemma3ForCausalLM", "phi3": "Phi3ForCausalLM",
                    "mistral": "MistralForCausalLM", "deepseek2": "DeepseekV2ForCausalLM",
                    "glm4": "Glm4ForCausalLM", "olmo2": "Olmo2ForCausalLM",
                    "granite": "GraniteForCausalLM", "qwen35": "Qwen3_5ForConditionalGeneration",
                    "qwen35moe": "Qwen3_5MoeForConditionalGeneration"}
        vocab = g("vocab_size") or len(m.get("tokenizer.ggml.tokens", [])) or 32000
        cfg = {
            "architectures": [arch_map.get(a, "LlamaForCausalLM")],
            "hidden_size": hidden, "num_hidden_layers": int(g("block_count", 32)),
            "num_attention_heads": heads,
            "num_key_value_heads": int(g("attention.head_count_kv", heads)),
            "intermediate_size": int(g("feed_forward_length", 4 * hidden)),
            "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-6)),
            "rope_theta": float(g("rope.freq_base", 10000.0)),
            "max_position_embeddings": int(g("context_length", 4096)),
            "vocab_size": int(vocab),
            "bos_token_id": m.get("tokenizer.ggml.bos_token_id"),
            "eos_token_id": m.get("tokenizer.ggml.eos_token_id"),
        }
        if g("attention.key_length"):
            cfg["head_dim"] = int(g("attention.key_length"))
        if g("expert_count"):
            cfg["num_experts"] = int(g("expert_count"))
            cfg["num_experts_per_tok"] = int(g("expert_used_count", 8))
            cfg["moe_intermediate_size"] = int(g("expert_feed_forward_length", 768))
        if g("rope.scaling.type"):
            cfg["rope_scaling"] = {"rope_type": g("rope.scaling.type"),
                                   "factor": float(g("rope.scaling.factor", 1.0)),
                                   "original_max_position_embeddings":
                                       int(g("rope.scaling.original_context_length", 8192))}
        cfg["tie_word_embeddings"] = "output.weight" not in self.tensors
        return cfg

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


# ----------------------------------------------------------------------------- dequantisation
def _f16(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


def _scale_min_k4(sc: np.ndarray):
    """K-quant 6-bit scale/min unpack: sc [nb, 12] uint8 -> (scales [nb, 8], mins [nb, 8])."""
    d = np.empty(sc.shape[:-1] + (8,), dtype=np.uint8)
    m = np.empty_like(d)
    d[..., :4] = sc[..., 0:4] & 63
    m[..., :4] = sc[..., 4:8] & 63
    d[..., 4:] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    m[..., 4:] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    return d.astype(np.float32), m.astype(np.float32)


def dequantize(raw: np.ndarray, ggml_type: int, shape) -> np.ndarray:
    name, be, bb = GGML[ggml_type]
    n = int(np.prod(shape)) if len(shape) else 1
    if name == "F32":
        return raw.view(np.float32).reshape(shape).copy()
    if name == "F16":
        return _f16(raw).reshape(shape)
    if name == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
    blk = raw.reshape(n // be, bb)
    if name == "Q8_0":
        d = _f16(blk[:, :2].copy()).reshape(-1, 1)
        q = blk[:, 2:].view(np.int8).astype(np.float32)
        return (d * q).reshape(shape)
    if name == "Q4_0":
        d = _f16(blk[:, :2].copy()).reshape(-1, 1)
        qs = blk[:, 2:]
        lo = (qs & 0xF).astype(np.int8) - 8
        hi = (qs >> 4).astype(np.int8) - 8
        return (d * np.concatenate([lo, hi], axis=1).astype(np.float32)).reshape(shape)
    if name == "Q4_K":
        d = _f16(blk[:, 0:2].copy()).reshape(-1, 1)
        dmin = _f16(blk[:, 2:4].copy()).reshape(-1, 1)
        sc, mn = _scale_min_k4(blk[:, 4:16])
        qs = blk[:, 16:144].reshape(-1, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
        y = (d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]
        return y.reshape(shape)
    if name == "Q5_K":
        d = _f16(blk[:, 0:2].copy()).reshape(-1, 1)
        dmin = _f16(blk[:, 2:4].copy()).reshape(-1, 1)
        sc, mn = _scale_min_k4(blk[:, 4:16])
        qh = blk[:, 16:48]                               # [nb, 32]
        qs = blk[:, 48:176].reshape(-1, 4, 32)
        lo = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32)
        bits = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1) << 4
        q = (lo | bits).astype(np.float32)
        y = (d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]
        return y.reshape(shape)
    if name == "Q6_K":
        ql = blk[:, 0:128].reshape(-1, 2, 64)
        qh = blk[:, 128:192].reshape(-1, 2, 32)
        sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
        d = _f16(blk[:, 208:210].copy()).reshape(-1, 1, 1)
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q1 = (l0 & 0xF) | (((qh >> 0) & 3) << 4)
        q2 = (l1 & 0xF) | (((qh >> 2) & 3) << 4)
        q3 = (l0 >> 4) | (((qh >> 4) & 3) << 4)
        q4 = (l1 >> 4) | (((qh >> 6) & 3) << 4)
        q = np.stack([q1, q2, q3, q4], axis=2).astype(np.int8) - 32     # [nb, 2, 4, 32]
        q = q.reshape(-1, 2, 8, 16).astype(np.float32)
        y = d[..., None] * sc[..., None] * q
        return y.reshape(shape)
    if name == "Q3_K":
        hmask = blk[:, 0:32]
        qs = blk[:, 32:96].reshape(-1, 2, 32)
        scr = blk[:, 96:108].astype(np.uint32)
        d = _f16(blk[:, 108:110].copy()).reshape(-1, 1, 1)
        # 16 six-bit scales packed in 12 bytes
        a = scr[:, 0:4].view(np.uint8).reshape(-1, 4).astype(np.uint32)
        a0 = (scr[:, 0] | (scr[:, 1] << 8) | (scr[:, 2] << 16) | (scr[:, 3] << 24))
        a1 = (scr[:, 4] | (scr[:, 5] << 8) | (scr[:, 6] << 16) | (scr[:, 7] << 24))
        tmp = (scr[:, 8] | (scr[:, 9] << 8) | (scr[:, 10] << 16) | (scr[:, 11] << 24))
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        w = np.stack([(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                      ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4),
                      ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)], axis=1).astype(np.uint32)
        scales = w.view(np.uint8).reshape(-1, 16).astype(np.int8).astype(np.float32) - 32.0
        out = np.empty((blk.shape[0], 256), dtype=np.float32)
        idx = 0
        for half in range(2):
            for shift in range(4):
                m = np.uint8(1 << (half * 4 + shift))
                for part in range(2):
                    ql = (qs[:, half, part * 16:(part + 1) * 16] >> (2 * shift)) & 3
                    hb = (hmask[:, part * 16:(part + 1) * 16] & m) == 0
                    q = ql.astype(np.int8) - np.where(hb, 4, 0).astype(np.int8)
                    s = scales[:, idx // 16]
                    out[:, idx:idx + 16] = (d[:, 0, 0] * s)[:, None] * q.astype(np.float32)
                    idx += 16
        return out.reshape(shape)
    raise GGUFError(f"no dequantiser for {name}")


# GGUF tensor name -> HF name
def hf_name(name: str) -> str | None:
    fixed = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
             "output.weight": "lm_head.weight"}
    if name in fixed:
        return fixed[name]
    if not name.startswith("blk."):
        return None
    _, l, rest = name.split(".", 2)
    m = {"attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
         "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.o_proj.weight",
         "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias",
         "attn_v.bias": "self_attn.v_proj.bias", "attn_q_norm.weight": "self_attn.q_norm.weight",
         "attn_k_norm.weight": "self_attn.k_norm.weight", "attn_norm.weight": "input_layernorm.weight",
         "ffn_norm.weight": "post_attention_layernorm.weight", "ffn_gate.weight": "mlp.gate_proj.weight",
         "ffn_up.weight": "mlp.up_proj.weight", "ffn_down.weight": "mlp.down_proj.weight",
         "post_attention_norm.weight": "post_attention_layernorm.weight",
         "post_ffw_norm.weight": "post_feedforward_layernorm.weight",
         "ffn_gate_inp.weight": "mlp.gate.weight", "ffn_gate_exps.weight": "mlp.experts.gate_proj.weight",
         "ffn_up_exps.weight": "mlp.experts.up_proj.weight",
         "ffn_down_exps.weight": "mlp.experts.down_proj.weight"}
    if rest not in m:
        return None
    return f"model.layers.{l}.{m[rest]}"


def _unpermute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """llama.cpp stores Llama q/k rows permuted for its interleaved RoPE; undo it."""
    rows = w.shape[0]
    return w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def iter_hf_tensors(g: GGUFFile, dtype=torch.bfloat16):
    cfg = g.hf_config()
    arch = g.architecture()
    for name in g.tensors:
        hn = hf_name(name)
        if hn is None:
            continue
        t = g.get(name, dtype)
        if arch == "llama" and hn.endswith("q_proj.weight"):
            t = _unpermute_qk(t, cfg["num_attention_heads"])
        elif arch == "llama" and hn.endswith("k_proj.weight"):
            t = _unpermute_qk(t, cfg["num_key_value_heads"])
        yield hn, t
