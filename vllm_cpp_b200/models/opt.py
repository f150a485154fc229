"""OPT decoder: learned absolute positions (offset 2), LayerNorm before each block, biased
projections, ReLU MLP, tied lm_head, plain multi-head attention without rotary embedding.

Reference: ``src/vllm/model_executor/models/opt.cpp``.
"""
from __future__ import annotations

import torch

from ..config import ModelConfig, ParallelConfig
from ..ops import reference as ref
from .base import StepContext, shard_cols, shard_rows
from .dense import DenseModel


class OPTModel(DenseModel):
    POS_OFFSET = 2

    def __init__(self, cfg: ModelConfig, device="cuda", parallel: ParallelConfig | None = None,
                 comm=None, max_position: int | None = None):
        cfg.num_kv_heads = cfg.num_heads
        super().__init__(cfg, device, parallel, comm, max_position)
        self.ln_eps = 1e-5

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        c = self.cfg
        H, I = c.hidden_size, c.intermediate_size
        g = torch.Generator().manual_seed(seed)

        def full(shape, s=std):
            return torch.empty(shape, dtype=torch.float32).normal_(0.0, s, generator=g).to(self.dtype)

        def gen():
            yield "model.decoder.embed_tokens.weight", full((c.vocab_size, H))
            yield "model.decoder.embed_positions.weight", full((self.max_position + self.POS_OFFSET, H))
            for l in range(c.num_layers):
                p = f"model.decoder.layers.{l}."
                for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                    yield p + f"self_attn.{n}.weight", full((H, H))
                    yield p + f"self_attn.{n}.bias", full((H,), 0.01)
                for n in ("self_attn_layer_norm", "final_layer_norm"):
                    yield p + n + ".weight", torch.ones(H, dtype=self.dtype)
                    yield p + n + ".bias", torch.zeros(H, dtype=self.dtype)
                yield p + "fc1.weight", full((I, H))
                yield p + "fc1.bias", full((I,), 0.01)
                yield p + "fc2.weight", full((H, I))
                yield p + "fc2.bias", full((H,), 0.01)
            yield "model.decoder.final_layer_norm.weight", torch.ones(H, dtype=self.dtype)
            yield "model.decoder.final_layer_norm.bias", torch.zeros(H, dtype=self.dtype)

        self.load_weights(gen())

    def load_weights(self, named_tensors) -> None:
        c = self.cfg
        tp, r = self.tp, self.rank
        dev, dt = self.device, self.dtype

        def put(t):
            return t.to(dt).contiguous().to(dev)

        self.layers = [dict() for _ in range(c.num_layers)]
        pend: dict = {}
        for name, t in named_tensors:
            name = name.replace("model.decoder.", "").replace("decoder.", "")
            if name == "embed_tokens.weight":
                pad = self.vocab_shard * tp - c.vocab_size
                if pad:
                    t = torch.cat([t, torch.zeros(pad, t.shape[1], dtype=t.dtype)], 0)
                self.w["embed"] = put(t[self.vocab_start:self.vocab_start + self.vocab_shard])
                self.w["lm_head"] = self.w["embed"]
            elif name == "embed_positions.weight":
                self.w["pos"] = put(t)
            elif name == "final_layer_norm.weight":
                self.w["final_norm"] = put(t)
            elif name == "final_layer_norm.bias":
                self.w["final_norm_b"] = put(t)
            elif name.startswith("layers."):
                parts = name.split(".")
                l = int(parts[1])
                L, P = self.layers[l], pend.setdefault(l, {})
                rest = ".".join(parts[2:])
                if rest.startswith("self_attn.") and parts[3] in ("q_proj", "k_proj", "v_proj"):
                    P[(parts[3], parts[4])] = t
                    for kind in ("weight", "bias"):
                        if all((n, kind) in P for n in ("q_proj", "k_proj", "v_proj")):
                            cat = torch.cat([shard_rows(P[(n, kind)], r, tp) for n in ("q_proj", "k_proj", "v_proj")], 0)
                            L["qkv" if kind == "weight" else "qkv_bias"] = put(cat)
                            for n in ("q_proj", "k_proj", "v_proj"):
                                del P[(n, kind)]
                elif rest == "self_attn.out_proj.weight":
                    L["o"] = put(shard_cols(t, r, tp))
                elif rest == "self_attn.out_proj.bias":
                    L["o_bias"] = put(t if r == 0 else torch.zeros_like(t))   # added once across ranks
                elif rest == "self_attn_layer_norm.weight":
                    L["ln1"] = put(t)
                elif rest == "self_attn_layer_norm.bias":
                    L["ln1_b"] = put(t)
                elif rest == "final_layer_norm.weight":
                    L["ln2"] = put(t)
                elif rest == "final_layer_norm.bias":
                    L["ln2_b"] = put(t)
                elif rest == "fc1.weight":
                    L["fc1"] = put(shard_rows(t, r, tp))
                elif rest == "fc1.bias":
                    L["fc1_b"] = put(shard_rows(t, r, tp))
                elif rest == "fc2.weight":
                    L["fc2"] = put(shard_cols(t, r, tp))
                elif rest == "fc2.bias":
                    L["fc2_b"] = put(t if r == 0 else torch.zeros_like(t))

    def reserve_buffers(self, max_tokens: int, max_reqs: int) -> None:
        super().reserve_buffers(max_tokens, max_reqs)
        self.bufs.reserve("fc1", max_tokens, self.inter)

    def fused_tp_supported(self) -> bool:
        return False

    def _ln(self, x, w, b):
        if self.device.type == "cuda":
            return self.be.ops.layernorm(x, w, b, self.ln_eps)
        return ref.layernorm(x, w, b, self.ln_eps)

    def _relu(self, x):
        if self.device.type == "cuda":
            return self.be.ops.relu(x)
        return torch.relu(x)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        c, be, T = self.cfg, self.be, ctx.num_tokens
        H = c.hidden_size
        qkv = self.bufs.get("qkv", T, 3 * self.hq * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        ids = ctx.input_ids[:T]
        tok = be.embedding(ids, self.w["embed"], out=self.bufs.get("hidden", T, H), vocab_start=self.vocab_start,
                           vocab_total=c.vocab_size)
        if self.tp > 1:
            self.comm.all_reduce(tok)
        pos = ctx.positions[:T]
        x = be.add(tok, self.w["pos"][(pos + self.POS_OFFSET).long()])
        for l, L in enumerate(self.layers):
            h = self._ln(x, L["ln1"], L["ln1_b"])
            be.gemm(h, L["qkv"], bias=L["qkv_bias"], out=qkv)
            be.rope_kv(qkv, pos, None, num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                       rot_dim=self.D, neox=True, q_norm=None, k_norm=None, eps=1e-6, gemma=False,
                       slot_mapping=ctx.slot_mapping[0][:T], kv_cache=self.kv_caches[l],
                       block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, 0, num_q_heads=self.hq,
                         num_kv_heads=self.hkv, head_dim=self.D, block_size=self.block_size,
                         scale=self.D ** -0.5, out=attn)
            o = be.gemm(attn, L["o"], bias=L["o_bias"])
            if self.tp > 1:
                self.comm.all_reduce(o)
            x = be.add(x, o)
            h = self._ln(x, L["ln2"], L["ln2_b"])
            f = be.gemm(h, L["fc1"], bias=L["fc1_b"], out=self.bufs.get("fc1", T, self.inter))
            f = self._relu(f)
            o = be.gemm(f, L["fc2"], bias=L["fc2_b"])
            if self.tp > 1:
                self.comm.all_reduce(o)
            x = be.add(x, o)
        full = self._ln(x, self.w["final_norm"], self.w["final_norm_b"])
        if ctx.decode_only_full_logits:
            n, last = T, full
        else:
            n = ctx.num_logits
            last = be.gather_rows(full, ctx.logits_indices[:n], out=self.bufs.get("last", n, H))
        logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
        be.gemm(last, self.w["lm_head"], out=logits, out_dtype=torch.float32)
        if self.tp > 1:
            logits = self.comm.all_gather(logits, dim=-1)
        return logits[:, : c.vocab_size] if logits.shape[1] != c.vocab_size else logits
