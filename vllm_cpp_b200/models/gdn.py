"""Qwen3.5 / Qwen3.6 / Qwen3-Next hybrid decoders: three Gated-DeltaNet layers then one gated
full-attention layer, repeated; dense SwiGLU MLP (27B shape) or routed experts + a gated
shared expert (35B-A3B shape).

GDN layer: merged in-projection [q | k | v | z | b | a] -> causal conv1d over [q|k|v]
(per-request state of the last three inputs) -> per-head L2 norm of q, k and g / beta ->
gated delta rule (packed recurrent kernel for decode rows, tcgen05 chunked scan for prefill
rows; per-request state [Hv, Dv, Dk] fp32) -> rmsnorm(o) * w * silu(z) -> out_proj.
Attention layer: q_proj emits [q | gate] per head, (1 + w) RMSNorm on q and k per head,
partial RoPE, paged attention with head_dim 256, output * sigmoid(gate), o_proj.

Reference: ``src/vllm/model_executor/models/qwen3_5.cpp:3138-3490`` (GdnBlockPaged),
``:3608-3780`` (FullAttnBlockPaged); semantics ``.agents/specs/gdn-semantics.md:27-260``.
"""
from __future__ import annotations

import os

import torch

from ..config import ModelConfig, ParallelConfig
from .base import StepContext, shard_cols, shard_rows
from .dense import ACT_KIND, DenseModel
from .moe import MoeModel


def _round_up(a, b):
    return (a + b - 1) // b * b


class Qwen35Model(DenseModel):
    def __init__(self, cfg: ModelConfig, device="cuda", parallel: ParallelConfig | None = None,
                 comm=None, max_position: int | None = None):
        super().__init__(cfg, device, parallel, comm, max_position)
        c = cfg
        assert c.linear_key_head_dim == 128 and c.linear_value_head_dim == 128
        assert c.linear_num_key_heads % self.tp == 0 and c.linear_num_value_heads % self.tp == 0
        self.gk = c.linear_num_key_heads // self.tp       # local GDN key heads
        self.gv = c.linear_num_value_heads // self.tp     # local GDN value heads
        self.Dk = self.Dv = 128
        self.conv_dim = 2 * self.gk * self.Dk + self.gv * self.Dv
        self.z_off = self.conv_dim
        self.b_off = self.z_off + self.gv * self.Dv
        self.a_off = self.b_off + self.gv
        self.in_w = self.a_off + self.gv
        self.in_w_pad = _round_up(self.in_w, 8)
        self.is_gdn = [t == "linear_attention" for t in c.layer_types]
        self.attn_layers = [l for l in range(c.num_layers) if not self.is_gdn[l]]
        self.gdn_layers = [l for l in range(c.num_layers) if self.is_gdn[l]]
        self.has_moe = bool(c.num_experts)
        if self.has_moe:
            # expert block of the MoE hybrids (35B-A3B, Qwen3-Next): routed experts sharded whole
            # per rank, one shared expert sharded like a dense MLP, scaled by a sigmoid gate
            self.E, self.k, self.moe_inter = c.num_experts, c.num_experts_per_tok, c.moe_intermediate_size
            self.ep = self.tp
            assert self.E % self.ep == 0
            self.e_local = self.E // self.ep
            self.e0 = self.rank * self.e_local if self.ep > 1 else 0
            self.shared_inter = c.shared_expert_intermediate_size // self.tp
            self.moe_ws = None
        self.gdn_ws = None
        self.conv_state: dict[int, torch.Tensor] = {}
        self.ssm_state: dict[int, torch.Tensor] = {}

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        c = self.cfg
        H, D = c.hidden_size, c.head_dim
        Hk, Hv = c.linear_num_key_heads, c.linear_num_value_heads
        big = c.num_layers * H * (3 * c.intermediate_size + 4 * Hv * 128) > 5e8
        gdev = self.device if (self.device.type == "cuda" and big) else torch.device("cpu")
        g = torch.Generator(device=gdev).manual_seed(seed)

        def full(shape, s=std):
            w = torch.empty(shape, dtype=torch.float32, device=gdev)
            w.normal_(0.0, s, generator=g)
            return w.to(self.dtype)

        def gen():
            yield "model.embed_tokens.weight", full((c.vocab_size, H))
            for l in range(c.num_layers):
                p = f"model.layers.{l}."
                zeros = torch.zeros(H, dtype=self.dtype)        # (1 + w) norms: w = 0 is identity
                yield p + "input_layernorm.weight", zeros.clone()
                yield p + "post_attention_layernorm.weight", zeros.clone()
                if self.is_gdn[l]:
                    q = p + "linear_attn."
                    yield q + "in_proj_qkv.weight", full((2 * Hk * 128 + Hv * 128, H))
                    yield q + "in_proj_z.weight", full((Hv * 128, H))
                    yield q + "in_proj_b.weight", full((Hv, H))
                    yield q + "in_proj_a.weight", full((Hv, H))
                    yield q + "conv1d.weight", full((2 * Hk * 128 + Hv * 128, 1, 4), 0.3)
                    u = torch.empty(Hv, dtype=torch.float32, device=gdev).uniform_(1.0, 16.0, generator=g)
                    yield q + "A_log", torch.log(u)
                    yield q + "dt_bias", torch.empty(Hv, dtype=torch.float32, device=gdev).normal_(0, 0.5, generator=g)
                    yield q + "norm.weight", torch.ones(128, dtype=self.dtype)
                    yield q + "out_proj.weight", full((H, Hv * 128))
                else:
                    q = p + "self_attn."
                    yield q + "q_proj.weight", full((c.num_heads * D * 2, H))
                    yield q + "k_proj.weight", full((c.num_kv_heads * D, H))
                    yield q + "v_proj.weight", full((c.num_kv_heads * D, H))
                    yield q + "o_proj.weight", full((H, c.num_heads * D))
                    yield q + "q_norm.weight", torch.zeros(D, dtype=self.dtype)
                    yield q + "k_norm.weight", torch.zeros(D, dtype=self.dtype)
                if self.has_moe:
                    I, S = c.moe_intermediate_size, c.shared_expert_intermediate_size
                    yield p + "mlp.gate.weight", full((c.num_experts, H), 0.5)
                    yield p + "mlp.experts.gate_up_proj", full((c.num_experts, 2 * I, H))
                    yield p + "mlp.experts.down_proj", full((c.num_experts, H, I))
                    if S:
                        yield p + "mlp.shared_expert.gate_proj.weight", full((S, H))
                        yield p + "mlp.shared_expert.up_proj.weight", full((S, H))
                        yield p + "mlp.shared_expert.down_proj.weight", full((H, S))
                        yield p + "mlp.shared_expert_gate.weight", full((1, H), 0.2)
                    continue
                yield p + "mlp.gate_proj.weight", full((c.intermediate_size, H))
                yield p + "mlp.up_proj.weight", full((c.intermediate_size, H))
                yield p + "mlp.down_proj.weight", full((H, c.intermediate_size))
            yield "model.norm.weight", torch.zeros(H, dtype=self.dtype)
            if not c.tie_word_embeddings:
                yield "lm_head.weight", full((c.vocab_size, H))

        self.load_weights(gen())

    def load_weights(self, named_tensors) -> None:
        """HF names. GDN in-projections either split (``in_proj_qkv/z/b/a``) or merged
        Qwen3-Next style (``in_proj_qkvz`` / ``in_proj_ba``, interleaved per key head)."""
        c, D = self.cfg, self.cfg.head_dim
        tp, r = self.tp, self.rank
        dev, dt = self.device, self.dtype
        Hk, Hv = c.linear_num_key_heads, c.linear_num_value_heads
        rep = Hv // Hk
        gk, gv = self.gk, self.gv

        def put(t, dtype=None):
            return t.to(dtype or dt).contiguous().to(dev)

        def kv_shard(w):
            if self.kv_rep > 1:
                h = r // self.kv_rep
                return w[h * D:(h + 1) * D]
            return shard_rows(w, r, tp)

        def qkv_rows(w):
            """[q | k | v] rows of the full tensor -> this rank's heads."""
            q, k, v = w[: Hk * 128], w[Hk * 128: 2 * Hk * 128], w[2 * Hk * 128:]
            return torch.cat([q[r * gk * 128:(r + 1) * gk * 128], k[r * gk * 128:(r + 1) * gk * 128],
                              v[r * gv * 128:(r + 1) * gv * 128]], 0)

        self.layers = [dict() for _ in range(c.num_layers)]
        pend: dict = {}
        for name, t in named_tensors:
            if name.startswith("model.language_model."):
                name = "model." + name[len("model.language_model."):]
            if name == "model.embed_tokens.weight":
                pad = self.vocab_shard * tp - c.vocab_size
                if pad:
                    t = torch.cat([t, torch.zeros(pad, t.shape[1], dtype=t.dtype, device=t.device)], 0)
                self.w["embed"] = put(t[self.vocab_start:self.vocab_start + self.vocab_shard])
                continue
            if name == "lm_head.weight":
                pad = self.vocab_shard * tp - c.vocab_size
                if pad:
                    t = torch.cat([t, torch.zeros(pad, t.shape[1], dtype=t.dtype, device=t.device)], 0)
                self.w["lm_head"] = put(t[self.vocab_start:self.vocab_start + self.vocab_shard])
                continue
            if name == "model.norm.weight":
                self.w["final_norm"] = put(t)
                continue
            if not name.startswith("model.layers."):
                continue
            parts = name.split(".")
            l = int(parts[2])
            if l >= c.num_layers:
                continue   # MTP / extra heads are handled elsewhere
            L = self.layers[l]
            rest = ".".join(parts[3:])
            P = pend.setdefault(l, {})
            if rest == "input_layernorm.weight":
                L["ln1"] = put(t)
            elif rest == "post_attention_layernorm.weight":
                L["ln2"] = put(t)
            elif rest.startswith("linear_attn."):
                key = rest[len("linear_attn."):]
                if key == "in_proj_qkvz.weight":
                    # per key head: [q 128 | k 128 | v rep*128 | z rep*128]
                    w = t.reshape(Hk, 2 * 128 + 2 * rep * 128, -1)
                    P["qkv"] = torch.cat([w[:, :128].reshape(Hk * 128, -1), w[:, 128:256].reshape(Hk * 128, -1),
                                          w[:, 256:256 + rep * 128].reshape(Hv * 128, -1)], 0)
                    P["z"] = w[:, 256 + rep * 128:].reshape(Hv * 128, -1)
                elif key == "in_proj_ba.weight":
                    w = t.reshape(Hk, 2 * rep, -1)
                    P["b"], P["a"] = w[:, :rep].reshape(Hv, -1), w[:, rep:].reshape(Hv, -1)
                elif key == "in_proj_qkv.weight":
                    P["qkv"] = t
                elif key == "in_proj_z.weight":
                    P["z"] = t
                elif key == "in_proj_b.weight":
                    P["b"] = t
                elif key == "in_proj_a.weight":
                    P["a"] = t
                elif key == "conv1d.weight":
                    L["conv_w"] = put(qkv_rows(t.reshape(t.shape[0], -1)))
                elif key == "A_log":
                    L["A_log"] = put(t[r * gv:(r + 1) * gv], torch.float32)
                elif key == "dt_bias":
                    L["dt_bias"] = put(t[r * gv:(r + 1) * gv], torch.float32)
                elif key == "norm.weight":
                    L["gnorm"] = put(t)
                elif key == "out_proj.weight":
                    L["out"] = put(shard_cols(t, r, tp))
                if all(k in P for k in ("qkv", "z", "b", "a")):
                    pad = torch.zeros(self.in_w_pad - self.in_w, P["qkv"].shape[1], dtype=P["qkv"].dtype,
                                      device=P["qkv"].device)
                    L["in_proj"] = put(torch.cat([qkv_rows(P["qkv"]), P["z"][r * gv * 128:(r + 1) * gv * 128],
                                                  P["b"][r * gv:(r + 1) * gv], P["a"][r * gv:(r + 1) * gv],
                                                  pad], 0))
                    for k in ("qkv", "z", "b", "a"):
                        del P[k]
            elif rest in ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"):
                P[parts[4]] = t
                if all(k in P for k in ("q_proj", "k_proj", "v_proj")):
                    L["qkv"] = put(torch.cat([shard_rows(P["q_proj"], r, tp), kv_shard(P["k_proj"]),
                                              kv_shard(P["v_proj"])], 0))
                    for k in ("q_proj", "k_proj", "v_proj"):
                        del P[k]
            elif rest == "self_attn.o_proj.weight":
                L["o"] = put(shard_cols(t, r, tp))
            elif rest == "self_attn.q_norm.weight":
                L["q_norm"] = put(t)
            elif rest == "self_attn.k_norm.weight":
                L["k_norm"] = put(t)
            elif rest in ("mlp.gate_proj.weight", "mlp.up_proj.weight"):
                P[parts[4]] = t
                if "gate_proj" in P and "up_proj" in P:
                    L["gate_up"] = put(torch.cat([shard_rows(P["gate_proj"], r, tp),
                                                  shard_rows(P["up_proj"], r, tp)], 0))
                    del P["gate_proj"], P["up_proj"]
            elif rest == "mlp.down_proj.weight":
                L["down"] = put(shard_cols(t, r, tp))
            elif self.has_moe and rest.startswith("mlp."):
                self._load_moe_tensor(L, P, parts, rest, t, put)
        if self.has_moe:
            e0, el = self.e0, self.e_local
            for l, P in pend.items():
                pe = P.get("pe")
                if not pe:
                    continue
                L = self.layers[l]
                L["w_gate_up"] = put(torch.stack([torch.cat([pe[(e, "gate_proj")], pe[(e, "up_proj")]], 0)
                                                  for e in range(e0, e0 + el)], 0))
                L["w_down"] = put(torch.stack([pe[(e, "down_proj")] for e in range(e0, e0 + el)], 0))
        if c.tie_word_embeddings or "lm_head" not in self.w:
            self.w["lm_head"] = self.w["embed"]

    def _load_moe_tensor(self, L, P, parts, rest, t, put) -> None:
        """Expert-block tensors: fused ``experts.gate_up_proj`` [E, 2I, H] / ``experts.down_proj``
        [E, H, I] or one tensor per expert, the shared expert and its scalar gate."""
        tp, r = self.tp, self.rank
        e0, el = self.e0, self.e_local
        if rest == "mlp.gate.weight":
            L["router"] = put(t)
        elif rest in ("mlp.experts.gate_up_proj", "mlp.experts.gate_up_proj.weight"):
            L["w_gate_up"] = put(t[e0:e0 + el])
        elif rest in ("mlp.experts.down_proj", "mlp.experts.down_proj.weight"):
            L["w_down"] = put(t[e0:e0 + el])
        elif len(parts) >= 8 and parts[4] == "experts" and parts[5].isdigit():
            e = int(parts[5])
            if e0 <= e < e0 + el:
                P.setdefault("pe", {})[(e, parts[6])] = t
        elif rest in ("mlp.shared_expert.gate_proj.weight", "mlp.shared_expert.up_proj.weight"):
            P["s_" + parts[5]] = t
            if "s_gate_proj" in P and "s_up_proj" in P:
                L["s_gate_up"] = put(torch.cat([shard_rows(P["s_gate_proj"], r, tp),
                                                shard_rows(P["s_up_proj"], r, tp)], 0))
                del P["s_gate_proj"], P["s_up_proj"]
        elif rest == "mlp.shared_expert.down_proj.weight":
            L["s_down"] = put(shard_cols(t, r, tp))
        elif rest == "mlp.shared_expert_gate.weight":
            # [1, H] padded to 8 rows so that it runs through the GEMM path
            g = torch.zeros(8, t.shape[-1], dtype=t.dtype, device=t.device)
            g[0] = t.reshape(-1)
            L["s_gate"] = put(g)

    # ------------------------------------------------------------------ caches
    def kv_cache_groups(self, block_size: int):
        spec = dict(kind="full", block_size=block_size, num_kv_heads=self.hkv, head_size=self.D,
                    dtype_bytes=2)
        return [(list(self.attn_layers), spec)]

    def alloc_kv_cache(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.kv_caches = {l: torch.zeros((num_blocks, 2, block_size, self.hkv, self.D), dtype=self.dtype,
                                         device=self.device) for l in self.attn_layers}
        self.layer_group = [0] * self.cfg.num_layers
        return [self.kv_caches[l] for l in self.attn_layers]

    def kv_bytes_per_block(self, block_size: int) -> int:
        return len(self.attn_layers) * 2 * block_size * self.hkv * self.D * 2

    # ---- recurrent state across a speculative step
    def snapshot_state(self, slots: list) -> None:
        """Saves the convolution and recurrent state of the given request slots. A step that
        verifies draft tokens advances the state over all of them; when some are rejected there is
        nothing to subtract, so the runner restores this copy and has the kept tokens run again."""
        if not slots or not self.gdn_layers:
            return
        if not getattr(self, "_snap", None):
            self._snap = {l: (torch.empty_like(self.conv_state[l]), torch.empty_like(self.ssm_state[l]))
                          for l in self.gdn_layers}
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        for l in self.gdn_layers:
            c, s = self._snap[l]
            c.index_copy_(0, idx, self.conv_state[l].index_select(0, idx))
            s.index_copy_(0, idx, self.ssm_state[l].index_select(0, idx))

    def restore_state(self, slots: list) -> None:
        if not slots or not self.gdn_layers:
            return
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        for l in self.gdn_layers:
            c, s = self._snap[l]
            self.conv_state[l].index_copy_(0, idx, c.index_select(0, idx))
            self.ssm_state[l].index_copy_(0, idx, s.index_select(0, idx))

    def state_bytes_per_request(self) -> int:
        return len(self.gdn_layers) * (self.conv_dim * 3 * 2 + self.gv * 128 * 128 * 4)

    def reserve_buffers(self, max_tokens: int, max_reqs: int) -> None:
        c = self.cfg
        qkv_w = (2 * self.hq + 2 * self.hkv) * self.D
        for name, cols in (("hidden", c.hidden_size), ("resid", c.hidden_size), ("normed", c.hidden_size),
                           ("qkv", qkv_w), ("attn", self.hq * self.D), ("gate_up", 2 * self.inter),
                           ("act", self.inter), ("gdn_in", self.in_w_pad), ("gdn_conv", self.conv_dim),
                           ("gdn_core", self.gv * 128), ("gdn_q", self.gk * 128), ("gdn_k", self.gk * 128),
                           ("q_compact", self.hq * self.D), ("gate_compact", self.hq * self.D)):
            self.bufs.reserve(name, max_tokens, cols)
        self.bufs.reserve("gdn_g", max_tokens, self.gv, torch.float32)
        self.bufs.reserve("gdn_beta", max_tokens, self.gv, torch.float32)
        self.bufs.reserve("last", max_reqs, c.hidden_size)
        self.bufs.reserve("logits", max_reqs, self.vocab_shard, torch.float32)
        self.bufs.reserve("argmax_cand", max_reqs, 2, torch.int32)
        for l in self.gdn_layers:
            self.conv_state[l] = torch.zeros((max_reqs, self.conv_dim, 3), dtype=self.dtype, device=self.device)
            self.ssm_state[l] = torch.zeros((max_reqs, self.gv, 128, 128), dtype=torch.float32,
                                            device=self.device)
        if self.device.type == "cuda":
            from ..ops.gdn import GdnWorkspace
            self.gdn_ws = GdnWorkspace(self.device, max_tokens, max_reqs, self.gv)
        if self.has_moe:
            self.bufs.reserve("router", max_tokens, self.E, torch.float32)
            self.bufs.reserve("moe_out", max_tokens, c.hidden_size)
            self.bufs.reserve("s_gate_up", max_tokens, max(2 * self.shared_inter, 8))
            self.bufs.reserve("s_act", max_tokens, max(self.shared_inter, 8))
            self.bufs.reserve("s_out", max_tokens, c.hidden_size)
            self.bufs.reserve("s_gate", max_tokens, 8, torch.float32)
            if self.device.type == "cuda":
                from ..ops.moe import MoeWorkspace
                self.moe_ws = MoeWorkspace(self.device, max_tokens, self.k, self.e_local,
                                           c.hidden_size, self.moe_inter)

    def fused_tp_supported(self) -> bool:
        # the fused GEMMs take bf16 weights; NVFP4 checkpoints run tensor parallel over NCCL
        return (self.tp > 1 and self.par.fused_collectives and self.device.type == "cuda"
                and self.cfg.hidden_size % 8 == 0 and not getattr(self, "quantized", None)
                and not self.cfg.quant)

    # ------------------------------------------------------------------ expert block
    _moe_block = MoeModel._moe_block
    _moe_block_cpu = MoeModel._moe_block_cpu
    eplb = None
    enable_eplb = MoeModel.enable_eplb
    eplb_end_step = MoeModel.eplb_end_step

    def _expert_block(self, x: torch.Tensor, L: dict, T: int, act_kind: int) -> torch.Tensor:
        """routed(x) + sigmoid(x . w_g) * shared(x); each rank returns its partial sum (its
        experts, its slice of the shared expert), the caller all-reduces."""
        c, be = self.cfg, self.be
        H = c.hidden_size
        routed = self._moe_block(x, L, T)
        hidden = self.bufs.get("hidden", T, H)
        if "s_gate_up" not in L:
            hidden.copy_(routed)
            return hidden
        gu = self.bufs.get("s_gate_up", T, 2 * self.shared_inter)
        be.gemm(x, L["s_gate_up"], out=gu)
        a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("s_act", T, self.shared_inter))
        so = be.gemm(a_, L["s_down"], out=self.bufs.get("s_out", T, H))
        g = be.gemm(x, L["s_gate"], out=self.bufs.get("s_gate", T, 8, torch.float32),
                    out_dtype=torch.float32)
        hidden.copy_(torch.addcmul(routed.float(), torch.sigmoid(g[:, :1]), so.float()))
        return hidden

    # ------------------------------------------------------------------ GDN layer
    def _gdn_layer(self, l: int, L: dict, x: torch.Tensor | None, ctx: StepContext, T: int, meta: dict,
                   proj: torch.Tensor | None = None):
        """x: normed hidden [T, H] -> core attention output after the gated norm [T, gv*128].
        ``proj``: the in_proj output when the caller already ran it (fused with the norm). ``x``
        None without ``proj``: the input is the gathered activation buffer of the fused
        tensor-parallel path (the in_proj GEMM waits for its rows tile by tile)."""
        be = self.be
        if proj is None:
            proj = self.bufs.get("gdn_in", T, self.in_w_pad)
            if x is None:
                self.tpf.gemm_gather(T, L["in_proj"], proj)
            else:
                be.gemm(x, L["in_proj"], out=proj)
        core = self.bufs.get("gdn_core", T, self.gv * 128)
        nd = ctx.num_decodes
        mixed = proj[:, : self.conv_dim]
        z = proj[:, self.z_off: self.z_off + self.gv * 128]
        b = proj[:, self.b_off: self.b_off + self.gv]
        a = proj[:, self.a_off: self.a_off + self.gv]
        conv_state, ssm = self.conv_state[l], self.ssm_state[l]
        if self.device.type != "cuda":
            from ..ops import gdn as G
            self._gdn_layer_cpu(L, mixed, a, b, conv_state, ssm, ctx, T, core)
            core.copy_(G.ref_rmsnorm_gated(core, z, L["gnorm"], self.cfg.rms_norm_eps, heads=self.gv))
        else:
            from ..ops import gdn as G
            xc = self.bufs.get("gdn_conv", T, self.conv_dim)
            slots = ctx.state_slots
            if nd > 0:
                G.conv1d_update(mixed[:nd], L["conv_w"], conv_state, slots[:nd], xc[:nd])
                G.packed_decode(xc[:nd], a[:nd], b[:nd], L["A_log"], L["dt_bias"], ssm, slots[:nd],
                                core[:nd].view(nd, self.gv, 128), self.gk, self.gv)
            if ctx.num_prefills > 0:
                P, Tp = ctx.num_prefills, T - nd
                pslots = slots[nd:nd + P]
                G.conv1d_fwd(mixed[nd:], L["conv_w"], conv_state, meta["pqs"], pslots, meta["has_init"], xc[nd:])
                q = self.bufs.get("gdn_q", Tp, self.gk * 128).view(Tp, self.gk, 128)
                k = self.bufs.get("gdn_k", Tp, self.gk * 128).view(Tp, self.gk, 128)
                g = self.bufs.get("gdn_g", Tp, self.gv, torch.float32)
                beta = self.bufs.get("gdn_beta", Tp, self.gv, torch.float32)
                G.post_conv(xc[nd:], self.gk, self.gv, a[nd:], b[nd:], L["A_log"], L["dt_bias"], q, k, g, beta)
                G.chunk_scan(q, k, xc[nd:], g, beta, ssm, meta["pqs_host"], pslots, meta["has_init"],
                             core[nd:].view(Tp, self.gv, 128), self.gdn_ws, v_col0=2 * self.gk * 128,
                             table=meta["table"])
            G.rmsnorm_gated(core, z, L["gnorm"], core, eps=self.cfg.rms_norm_eps, heads=self.gv)
        return core

    def _gdn_layer_cpu(self, L, mixed, a, b, conv_state, ssm, ctx, T, core):
        from ..ops import gdn as G
        R = ctx.num_reqs
        qsl = ctx.query_start[: R + 1].tolist()
        seq = ctx.seq_lens[:R].tolist()
        slots = ctx.state_slots[:R].tolist()
        has_init = [1 if seq[i] - (qsl[i + 1] - qsl[i]) > 0 else 0 for i in range(R)]
        if (mixed.dtype == torch.bfloat16 and ssm.dtype == torch.float32 and conv_state.is_contiguous()
                and ssm.is_contiguous() and os.environ.get("B200_CPU_ORACLE", "0") != "1"):
            # native thread-pool ops (csrc/cpu/cpu_ops_ext.cpp); the PyTorch path below is their oracle
            from ..ops import cpu_native as N
            xc = N.gdn_conv1d(mixed, L["conv_w"], conv_state, qsl, slots, has_init)
            q, k, g, beta = N.gdn_post_conv(xc, self.gk, self.gv, a, b, L["A_log"], L["dt_bias"])
            v = xc[:, 2 * self.gk * 128:].view(T, self.gv, 128)
            out = N.gdn_recurrent(q, k, v, g, beta, ssm, qsl, slots, has_init)
            core.copy_(out.reshape(T, -1).to(core.dtype))
            return
        xc, st = G.ref_conv1d(mixed, L["conv_w"], conv_state, qsl, slots, has_init)
        conv_state.copy_(st)
        q, k, g, beta = G.ref_post_conv(xc, self.gk, self.gv, a, b, L["A_log"], L["dt_bias"])
        v = xc[:, 2 * self.gk * 128:].reshape(T, self.gv, 128)
        out = torch.empty(T, self.gv, 128, dtype=torch.float32)
        for i in range(R):
            s0 = ssm[slots[i]] if has_init[i] else torch.zeros_like(ssm[0])
            bgn, end = qsl[i], qsl[i + 1]
            o, s1 = G.ref_recurrent(q[bgn:end], k[bgn:end], v[bgn:end], g[bgn:end], beta[bgn:end], s0)
            out[bgn:end] = o
            ssm[slots[i]] = s1
        core.copy_(out.reshape(T, -1).to(core.dtype))

    def _step_meta(self, ctx: StepContext, T: int) -> dict:
        """Per-step GDN metadata for the prefill rows: device query_start / has_init and the
        chunk table (built on the host from the step's pinned arrays, one small copy)."""
        meta: dict = {}
        if self.device.type != "cuda" or ctx.num_prefills == 0:
            return meta
        import numpy as np
        from ..ops import gdn as G
        nd, P = ctx.num_decodes, ctx.num_prefills
        host = ctx.extra.get("host")
        if host is not None:
            pqs_host = host["prefill_q_start"][: P + 1].numpy().copy()
            seq_host = host["seq_lens"][nd:nd + P].numpy()
        else:
            pqs_host = ctx.prefill_q_start[: P + 1].cpu().numpy()
            seq_host = ctx.seq_lens[nd:nd + P].cpu().numpy()
        has_init = ((seq_host - (pqs_host[1:] - pqs_host[:-1])) > 0).astype(np.int32)
        t0, ln, s0 = G.build_chunk_table(pqs_host)
        NT = len(t0)
        ws = self.gdn_ws
        packed = np.concatenate([t0, ln, s0, has_init]).astype(np.int32)
        ws.table[: packed.size].copy_(torch.from_numpy(packed))
        meta["table"] = (ws.table[:NT], ws.table[NT:2 * NT], ws.table[2 * NT:2 * NT + P + 1])
        meta["has_init"] = ws.table[2 * NT + P + 1: 2 * NT + 2 * P + 1]
        meta["pqs"] = ctx.prefill_q_start[: P + 1]
        meta["pqs_host"] = pqs_host
        return meta

    # ------------------------------------------------------------------ forward
    def _forward_tp_fused_gdn(self, ctx: StepContext):
        """The hybrid stack with every collective inside a kernel: out_proj / o_proj / down_proj
        scatter their partial rows in the GEMM epilogue, the owner reduces + adds the residual +
        normalises (Gemma-style weight) + all-gathers, in_proj / qkv / gate_up wait for gathered
        rows tile by tile, and the MoE combine (routed sum + gated shared expert) stores into the
        owners' receive slots."""
        c, be, T, tpf = self.cfg, self.be, ctx.num_tokens, self.tpf
        H, eps, D = c.hidden_size, c.rms_norm_eps, self.D
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, H)
        normed = self.bufs.get("normed", T, H)
        qkv = self.bufs.get("qkv", T, (2 * self.hq + 2 * self.hkv) * D)
        attn = self.bufs.get("attn", T, self.hq * D)
        be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                     vocab_total=c.vocab_size)
        self.comm.all_reduce(hidden)
        tpf.first_norm(hidden, self.layers[0]["ln1"], eps, True)
        pos = ctx.positions[:T]
        meta = self._step_meta(ctx, T)
        k_off = 2 * self.hq * D
        sc = None
        if self.has_moe:
            from ..ops import moe as M
            sc = M.B200MoeScatter()
            sc.world, sc.rank, sc.rows_per_rank = tpf.world, tpf.rank, tpf.rows_per_rank(T)
            for r in range(tpf.world):
                sc.peer_recv[r] = tpf.recv.ptrs[r]
                sc.peer_rs_flags[r] = tpf._rs_flags(r)
            sc.recv_parity_stride, sc.rs_flag_parity_stride = tpf.recv_parity, tpf.rs_groups
            sc.op_counter = tpf._op_counter()
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            if self.is_gdn[l]:
                core = self._gdn_layer(l, L, None, ctx, T, meta)
                exp = tpf.gemm_scatter(core, L["out"])
            else:
                tpf.gemm_gather(T, L["qkv"], qkv)
                qv = qkv[:, :k_off].view(T, self.hq, 2 * D)
                qc = self.bufs.get("q_compact", T, self.hq * D)
                be.ops.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                               head_dim=D, rot_dim=self.rot, neox=c.rope.neox, q_norm=L.get("q_norm"),
                               k_norm=L.get("k_norm"), eps=eps, gemma=True,
                               slot_mapping=ctx.slot_mapping[0][:T], kv_cache=self.kv_caches[l],
                               block_size=self.block_size, q_out=qc, q_head_stride=2 * D,
                               offsets=(0, k_off, k_off + self.hkv * D))
                be.attention(qc, self.kv_caches[l], ctx, 0, num_q_heads=self.hq, num_kv_heads=self.hkv,
                             head_dim=D, block_size=self.block_size, scale=self.scale, out=attn)
                gate = self.bufs.get("gate_compact", T, self.hq * D)
                gate.view(T, self.hq, D).copy_(qv[:, :, D:])
                gated = be.sigmoid_mul(attn, gate)
                exp = tpf.gemm_scatter(gated, L["o"])
            tpf.reduce_norm_gather(T, exp, L["ln2"], eps, True)
            nw = self.layers[l + 1]["ln1"] if l + 1 < n_layers else self.w["final_norm"]
            if self.has_moe:
                from ..ops import moe as M
                tpf.gather_all(T, normed)
                so = sg = None
                if "s_gate_up" in L:
                    gu = self.bufs.get("s_gate_up", T, 2 * self.shared_inter)
                    be.gemm(normed, L["s_gate_up"], out=gu)
                    a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("s_act", T, self.shared_inter))
                    so = be.gemm(a_, L["s_down"], out=self.bufs.get("s_out", T, H))
                    sg = M.shared_gate(normed, L["s_gate"][0])
                self._moe_block(normed, L, T, scatter=sc, shared=so, shared_gate=sg)
                tpf.reduce_norm_gather(T, tpf.world * 32, nw, eps, True, nsrc=tpf.world)
            else:
                gate_up = self.bufs.get("gate_up", T, 2 * self.inter)
                tpf.gemm_gather(T, L["gate_up"], gate_up)
                a_ = be.act_and_mul(gate_up, act_kind, out=self.bufs.get("act", T, self.inter))
                exp = tpf.gemm_scatter(a_, L["down"])
                tpf.reduce_norm_gather(T, exp, nw, eps, True)
        return self._tp_fused_logits(ctx, T)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        if getattr(self, "tpf", None) is not None:
            return self._forward_tp_fused_gdn(ctx)
        c, be, T = self.cfg, self.be, ctx.num_tokens
        H, eps, D = c.hidden_size, c.rms_norm_eps, self.D
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, H)
        resid = self.bufs.get("resid", T, H)
        normed = self.bufs.get("normed", T, H)
        qkv_w = (2 * self.hq + 2 * self.hkv) * D
        qkv = self.bufs.get("qkv", T, qkv_w)
        attn = self.bufs.get("attn", T, self.hq * D)
        gate_up = self.bufs.get("gate_up", T, 2 * self.inter)
        act = self.bufs.get("act", T, self.inter)
        given = ctx.extra.get("inputs_embeds")
        if given is not None:
            # a draft head runs this stack on its own input rows instead of token embeddings
            hidden.copy_(given[:T])
        else:
            e = be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                             vocab_total=c.vocab_size)
            if e is not hidden:
                hidden.copy_(e)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
        pos = ctx.positions[:T]
        meta = self._step_meta(ctx, T)
        k_off = 2 * self.hq * D
        for l, L in enumerate(self.layers):
            if l == 0:
                resid.copy_(hidden)
            res_in = None if l == 0 else resid
            if self.is_gdn[l]:
                # the norm hands its rows to in_proj (as quantised activations when the weights take them)
                proj = self.bufs.get("gdn_in", T, self.in_w_pad)
                be.norm_gemm(hidden, L["ln1"], eps, L["in_proj"], proj, residual=res_in, gemma=True, normed=normed)
                core = self._gdn_layer(l, L, None, ctx, T, meta, proj=proj)
                be.gemm(core, L["out"], out=hidden)
            else:
                be.norm_gemm(hidden, L["ln1"], eps, L["qkv"], qkv, residual=res_in, gemma=True, normed=normed)
                # q rows are [q | gate] per head (head stride 2D): the fused norm + RoPE kernel
                # reads them strided and writes the rotated q compactly
                qv = qkv[:, :k_off].view(T, self.hq, 2 * D)
                if self.device.type == "cuda":
                    qc = self.bufs.get("q_compact", T, self.hq * D)
                    be.ops.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                                   head_dim=D, rot_dim=self.rot, neox=c.rope.neox, q_norm=L.get("q_norm"),
                                   k_norm=L.get("k_norm"), eps=eps, gemma=True,
                                   slot_mapping=ctx.slot_mapping[0][:T], kv_cache=self.kv_caches[l],
                                   block_size=self.block_size, q_out=qc, q_head_stride=2 * D,
                                   offsets=(0, k_off, k_off + self.hkv * D))
                else:
                    tmp = torch.cat([qv[:, :, :D].reshape(T, -1), qkv[:, k_off:]], 1).contiguous()
                    be.rope_kv(tmp, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                               head_dim=D, rot_dim=self.rot, neox=c.rope.neox, q_norm=L.get("q_norm"),
                               k_norm=L.get("k_norm"), eps=eps, gemma=True,
                               slot_mapping=ctx.slot_mapping[0][:T], kv_cache=self.kv_caches[l],
                               block_size=self.block_size)
                    qc = tmp[:, : self.hq * D]
                be.attention(qc, self.kv_caches[l], ctx, 0, num_q_heads=self.hq, num_kv_heads=self.hkv,
                             head_dim=D, block_size=self.block_size, scale=self.scale, out=attn)
                gate = self.bufs.get("gate_compact", T, self.hq * D)
                gate.view(T, self.hq, D).copy_(qv[:, :, D:])
                be.sigmoid_gate_gemm(attn, gate, L["o"], hidden)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
            if self.has_moe:
                x = be.rmsnorm(hidden, L["ln2"], eps, residual=resid, out=normed, gemma=True)
                hidden = self._expert_block(x, L, T, act_kind)
            else:
                be.norm_gemm(hidden, L["ln2"], eps, L["gate_up"], gate_up, residual=resid, gemma=True, normed=normed)
                be.act_gemm(gate_up, act_kind, L["down"], hidden, act=act)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
        full = be.rmsnorm(hidden, self.w["final_norm"], eps, residual=resid, out=normed, gemma=True)
        self.last_full = full          # every row after the final norm: what a draft head continues from
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
