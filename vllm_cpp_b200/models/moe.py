"""Qwen3-MoE family (Qwen3-Coder-30B-A3B shape): the dense attention block plus a routed
expert MLP (softmax router over all experts, greedy top-k with lowest-index ties, renormalised
weights, SwiGLU experts, fp32 weighted combine rounded once to bf16).

Expert parallelism: experts are split whole across the ranks of the tensor-parallel group.
Activations are already replicated on every rank by the fused all-gather of the attention
block, so "dispatch" is a local selection of the (token, expert) pairs whose expert lives
here; the combine kernel stores each token's partial sum straight into the receive slot of
the rank that owns that row (combine + reduce-scatter), after which the usual
reduce + residual + RMSNorm + all-gather kernel finishes the block.

Reference forward: ``src/vllm/model_executor/models/qwen3_moe.cpp:64-95`` and ``RunMoeBlock``
(``qwen3_5.cpp:5027``); semantics ``.agents/specs/moe-semantics.md:93-205``.
"""
from __future__ import annotations

import os

import torch

from ..config import ModelConfig, ParallelConfig
from .base import StepContext, shard_cols, shard_rows
from .dense import ACT_KIND, DenseModel


class MoeModel(DenseModel):
    def __init__(self, cfg: ModelConfig, device="cuda", parallel: ParallelConfig | None = None,
                 comm=None, max_position: int | None = None):
        super().__init__(cfg, device, parallel, comm, max_position)
        c = cfg
        self.E = c.num_experts
        self.k = c.num_experts_per_tok
        self.moe_inter = c.moe_intermediate_size
        # expert parallel: whole experts per rank (tp ranks double as ep ranks)
        self.ep = self.tp if (self.par.enable_expert_parallel or self.tp > 1) else 1
        assert self.E % self.ep == 0
        self.e_local = self.E // self.ep
        self.e0 = self.rank * self.e_local if self.ep > 1 else 0
        self.moe_ws = None
        self.eplb = None

    # ------------------------------------------------------------------ expert load balancing
    def enable_eplb(self, eplb_cfg) -> None:
        """Switches the MoE layers from the contiguous expert split to balanced physical slots
        (``parallel/eplb.py``): the expert tensors are rearranged (redundant slots filled with
        replicas), the router's ids go through the placement table from now on, and
        ``eplb_end_step`` rebalances on schedule. Collective over the expert-parallel ranks."""
        from ..parallel.comm import SingleComm
        from ..parallel.eplb import EplbState
        moe_layers = [l for l, L in enumerate(self.layers) if "w_gate_up" in L]
        comm = self.comm if self.ep > 1 else SingleComm()
        st = EplbState(eplb_cfg, comm, len(moe_layers), self.E, self.device)
        new = st.initial([[self.layers[l]["w_gate_up"], self.layers[l]["w_down"]] for l in moe_layers])
        for i, l in enumerate(moe_layers):
            self.layers[l]["w_gate_up"], self.layers[l]["w_down"] = new[i]
            self.layers[l]["_eplb_idx"] = i
        self._eplb_layers = moe_layers
        self.eplb = st
        self.e_local = st.S
        self.e0 = self.rank * st.S if self.ep > 1 else 0
        if self.moe_ws is not None:
            from ..ops.moe import MoeWorkspace
            self.moe_ws = MoeWorkspace(self.device, self.moe_ws.max_pairs // self.k, self.k, self.e_local,
                                       self.cfg.hidden_size, self.moe_inter)

    def eplb_end_step(self) -> bool:
        """Called once per engine step; True when the experts were rebalanced in this call. The
        rearranged tensors replace the old ones in place (same shapes, same storage), so captured
        graphs stay valid."""
        st = self.eplb
        if st is None or not st.end_step():
            return False
        layers = self._eplb_layers
        new = st.rebalance_now([[self.layers[l]["w_gate_up"], self.layers[l]["w_down"]] for l in layers])
        for i, l in enumerate(layers):
            self.layers[l]["w_gate_up"].copy_(new[i][0])
            self.layers[l]["w_down"].copy_(new[i][1])
        return True

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        c = self.cfg
        H, D, I = c.hidden_size, c.head_dim, self.moe_inter
        n_params = c.num_layers * (2 * c.num_heads * D * H + 3 * self.E * I * H)
        gdev = self.device if (self.device.type == "cuda" and n_params > 5e8) else torch.device("cpu")
        g = torch.Generator(device=gdev).manual_seed(seed)

        def full(shape):
            w = torch.empty(shape, dtype=torch.float32, device=gdev)
            w.normal_(0.0, std, generator=g)
            return w.to(self.dtype)

        def gen():
            yield "model.embed_tokens.weight", full((c.vocab_size, H))
            for l in range(c.num_layers):
                p = f"model.layers.{l}."
                yield p + "self_attn.q_proj.weight", full((c.num_heads * D, H))
                yield p + "self_attn.k_proj.weight", full((c.num_kv_heads * D, H))
                yield p + "self_attn.v_proj.weight", full((c.num_kv_heads * D, H))
                yield p + "self_attn.o_proj.weight", full((H, c.num_heads * D))
                ones = torch.ones(H, dtype=self.dtype)
                yield p + "input_layernorm.weight", ones.clone()
                yield p + "post_attention_layernorm.weight", ones.clone()
                if c.qk_norm:
                    yield p + "self_attn.q_norm.weight", torch.ones(D, dtype=self.dtype)
                    yield p + "self_attn.k_norm.weight", torch.ones(D, dtype=self.dtype)
                yield p + "mlp.gate.weight", full((self.E, H))
                # stacked expert tensors (one draw each keeps start-up short)
                yield p + "mlp.experts.gate_proj.weight", full((self.E, I, H))
                yield p + "mlp.experts.up_proj.weight", full((self.E, I, H))
                yield p + "mlp.experts.down_proj.weight", full((self.E, H, I))
            yield "model.norm.weight", torch.ones(H, dtype=self.dtype)
            if not c.tie_word_embeddings:
                yield "lm_head.weight", full((c.vocab_size, H))

        self.load_weights(gen())

    def load_weights(self, named_tensors) -> None:
        """HF names; experts either stacked (``mlp.experts.{gate,up,down}_proj.weight`` with a
        leading expert dim) or per expert (``mlp.experts.<e>.gate_proj.weight``)."""
        c, D = self.cfg, self.cfg.head_dim
        tp, r = self.tp, self.rank
        dev, dt = self.device, self.dtype
        H, I = c.hidden_size, self.moe_inter
        e0, el = self.e0, self.e_local

        def put(t):
            return t.to(dt).contiguous().to(dev)

        def kv_shard(w):
            if self.kv_rep > 1:
                h = r // self.kv_rep
                return w[h * D:(h + 1) * D]
            return shard_rows(w, r, tp)

        self.layers = [dict() for _ in range(c.num_layers)]
        pend: dict = {}
        for name, t in named_tensors:
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
            L = self.layers[l]
            rest = ".".join(parts[3:])
            if rest in ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"):
                pend.setdefault((l, "qkv"), {})[parts[4]] = t
                d = pend[(l, "qkv")]
                if len(d) == 3:
                    L["qkv"] = put(torch.cat([shard_rows(d["q_proj"], r, tp), kv_shard(d["k_proj"]),
                                              kv_shard(d["v_proj"])], 0))
                    del pend[(l, "qkv")]
            elif rest == "self_attn.o_proj.weight":
                L["o"] = put(shard_cols(t, r, tp))
            elif rest == "input_layernorm.weight":
                L["ln1"] = put(t)
            elif rest == "post_attention_layernorm.weight":
                L["ln2"] = put(t)
            elif rest == "self_attn.q_norm.weight":
                L["q_norm"] = put(t)
            elif rest == "self_attn.k_norm.weight":
                L["k_norm"] = put(t)
            elif rest == "mlp.gate.weight":
                L["router"] = put(t)
            elif rest in ("mlp.experts.gate_proj.weight", "mlp.experts.up_proj.weight"):
                pend.setdefault((l, "gu"), {})[parts[5]] = t[e0:e0 + el]
                d = pend[(l, "gu")]
                if len(d) == 2:
                    L["w_gate_up"] = put(torch.cat([d["gate_proj"], d["up_proj"]], 1))  # [El, 2I, H]
                    del pend[(l, "gu")]
            elif rest == "mlp.experts.down_proj.weight":
                L["w_down"] = put(t[e0:e0 + el])                                        # [El, H, I]
            elif len(parts) >= 8 and parts[3] == "mlp" and parts[4] == "experts" and parts[5].isdigit():
                e = int(parts[5])
                if e0 <= e < e0 + el:
                    pend.setdefault((l, "pe"), {})[(e, parts[6])] = t
        # per-expert checkpoints: stack once everything has arrived
        for (l, kind), d in list(pend.items()):
            if kind != "pe":
                continue
            L = self.layers[l]
            gu = [torch.cat([d[(e, "gate_proj")], d[(e, "up_proj")]], 0) for e in range(e0, e0 + el)]
            L["w_gate_up"] = put(torch.stack(gu, 0))
            L["w_down"] = put(torch.stack([d[(e, "down_proj")] for e in range(e0, e0 + el)], 0))
        if c.tie_word_embeddings or "lm_head" not in self.w:
            self.w["lm_head"] = self.w["embed"]

    def reserve_buffers(self, max_tokens: int, max_reqs: int) -> None:
        c = self.cfg
        qkv_w = (self.hq + 2 * self.hkv) * self.D
        for name, cols in (("hidden", c.hidden_size), ("resid", c.hidden_size),
                           ("normed", c.hidden_size), ("qkv", qkv_w), ("attn", self.hq * self.D),
                           ("moe_out", c.hidden_size)):
            self.bufs.reserve(name, max_tokens, cols)
        self.bufs.reserve("router", max_tokens, self.E, torch.float32)
        self.bufs.reserve("last", max_reqs, c.hidden_size)
        self.bufs.reserve("logits", max_reqs, self.vocab_shard, torch.float32)
        self.bufs.reserve("argmax_cand", max_reqs, 2, torch.int32)
        if self.device.type == "cuda":
            from ..ops.moe import MoeWorkspace
            self.moe_ws = MoeWorkspace(self.device, max_tokens, self.k, self.e_local,
                                       c.hidden_size, self.moe_inter)

    def weight_bytes(self) -> int:
        return super().weight_bytes()

    # ------------------------------------------------------------------ MoE block
    def _moe_block(self, x: torch.Tensor, L: dict, T: int, scatter=None, shared=None,
                   shared_gate=None) -> torch.Tensor:
        """Routed experts over ``x`` [T, H]. Returns this rank's (partial, if EP) output, or
        stores it into the owners' receive slots when ``scatter`` is given. ``shared`` [T, H]
        (this rank's part of the shared experts' output), scaled per row by ``shared_gate`` [T]
        when given, is added in the combine kernel."""
        c = self.cfg
        if self.device.type != "cuda":
            return self._moe_block_cpu(x, L)
        from ..ops import moe as M
        ws = self.moe_ws
        logits = self.bufs.get("router", T, self.E, torch.float32)
        self.be.gemm(x, L["router"], out=logits, out_dtype=torch.float32)
        ids, w = M.router_topk(logits, self.k, renorm=c.norm_topk_prob,
                               routed_scale=c.routed_scaling_factor)
        if self.eplb is not None:
            ids = self.eplb.remap(L["_eplb_idx"], ids)       # logical expert -> physical slot
        M.moe_sort(ids, self.e0, self.e0 + self.e_local, ws)
        P = T * self.k
        chunks = min(ws.max_chunks, self.e_local + (P + 255) // 256)
        M.moe_gather(x, ws, self.e_local, P)
        if os.environ.get("B200_MOE_FUSED_ACT", "1") != "0":
            M.grouped_gemm_gated(ws.xs, L["w_gate_up"], ws.act, ws, P, chunks, kind=ACT_KIND.get(c.hidden_act, 0))
        else:
            M.grouped_gemm(ws.xs, L["w_gate_up"], ws.gu, ws, P, chunks)
            self.be.act_and_mul(ws.gu[:P], ACT_KIND.get(c.hidden_act, 0), out=ws.act[:P])
        M.grouped_gemm(ws.act, L["w_down"], ws.y, ws, P, chunks)
        out = None if scatter is not None else self.bufs.get("moe_out", T, c.hidden_size)
        M.combine(ws.y, ws, w, out, shared=shared, shared_gate=shared_gate, scatter=scatter)
        return out

    def _moe_block_cpu(self, x, L):
        from ..ops import moe as M
        c = self.cfg
        if x.dtype == torch.bfloat16 and os.environ.get("B200_CPU_ORACLE", "0") != "1":
            # native thread-pool ops (csrc/cpu/cpu_ops_ext.cpp); the PyTorch restatement below is
            # their oracle
            from ..ops import cpu_native as N
            logits = N.gemm(x.contiguous(), L["router"], out_dtype=torch.float32)
            ids, w = N.moe_router_topk(logits, self.k, renorm=c.norm_topk_prob,
                                       routed_scale=c.routed_scaling_factor)
            if self.eplb is not None:
                ids = self.eplb.remap(L["_eplb_idx"], ids)
            return N.moe_experts(x.contiguous(), ids, w, L["w_gate_up"], L["w_down"], e0=self.e0,
                                 act_kind=ACT_KIND.get(c.hidden_act, 0))
        logits = (x.float() @ L["router"].float().t())
        ids, w = M.ref_router_topk(logits, self.k, renorm=c.norm_topk_prob,
                                   routed_scale=c.routed_scaling_factor)
        if self.eplb is not None:
            ids = self.eplb.remap(L["_eplb_idx"], ids)
        return M.ref_moe_block(x, ids, w, L["w_gate_up"], L["w_down"], e0=self.e0)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext) -> torch.Tensor:
        if getattr(self, "tpf", None) is not None:
            return self._forward_tp_fused_moe(ctx)
        c, be, T = self.cfg, self.be, ctx.num_tokens
        H, eps = c.hidden_size, c.rms_norm_eps
        hidden = self.bufs.get("hidden", T, H)
        resid = self.bufs.get("resid", T, H)
        normed = self.bufs.get("normed", T, H)
        qkv = self.bufs.get("qkv", T, (self.hq + 2 * self.hkv) * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        e = be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden,
                         vocab_start=self.vocab_start, vocab_total=c.vocab_size)
        if e is not hidden:
            hidden.copy_(e)
        if self.tp > 1:
            self.comm.all_reduce(hidden)
        pos = ctx.positions[:T]
        for l, L in enumerate(self.layers):
            grp = self.layer_group[l]
            if l == 0:
                resid.copy_(hidden)
                x = be.rmsnorm(hidden, L["ln1"], eps, out=normed)
            else:
                x = be.rmsnorm(hidden, L["ln1"], eps, residual=resid, out=normed)
            be.gemm(x, L["qkv"], out=qkv)
            be.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                       head_dim=self.D, rot_dim=self.rot, neox=c.rope.neox,
                       q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=eps, gemma=False,
                       slot_mapping=ctx.slot_mapping[grp][:T], kv_cache=self.kv_caches[l],
                       block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, grp,
                         num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                         block_size=self.block_size, scale=self.scale, out=attn)
            be.gemm(attn, L["o"], out=hidden)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
            x = be.rmsnorm(hidden, L["ln2"], eps, residual=resid, out=normed)
            m = self._moe_block(x, L, T)
            hidden = self.bufs.get("hidden", T, H)
            hidden.copy_(m)
            if self.ep > 1:
                self.comm.all_reduce(hidden)
        full = be.rmsnorm(hidden, self.w["final_norm"], eps, residual=resid, out=normed)
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

    def fused_tp_supported(self) -> bool:
        # the fused GEMMs take bf16 weights; quantised checkpoints run tensor parallel over NCCL
        return (self.tp > 1 and self.par.fused_collectives and self.device.type == "cuda"
                and not getattr(self, "quantized", None))

    def _forward_tp_fused_moe(self, ctx: StepContext) -> torch.Tensor:
        """TP attention + EP experts with every collective fused into a kernel."""
        from ..ops.moe import B200MoeScatter
        c, be, T, tpf = self.cfg, self.be, ctx.num_tokens, self.tpf
        H, eps = c.hidden_size, c.rms_norm_eps
        hidden = self.bufs.get("hidden", T, H)
        qkv = self.bufs.get("qkv", T, (self.hq + 2 * self.hkv) * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        normed = self.bufs.get("normed", T, H)
        be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                     vocab_total=c.vocab_size)
        self.comm.all_reduce(hidden)
        tpf.first_norm(hidden, self.layers[0]["ln1"], eps, False)
        pos = ctx.positions[:T]
        sc = B200MoeScatter()
        sc.world, sc.rank, sc.rows_per_rank = tpf.world, tpf.rank, tpf.rows_per_rank(T)
        for r in range(tpf.world):
            sc.peer_recv[r] = tpf.recv.ptrs[r]
            sc.peer_rs_flags[r] = tpf._rs_flags(r)
        sc.recv_parity_stride, sc.rs_flag_parity_stride = tpf.recv_parity, tpf.rs_groups
        sc.op_counter = tpf._op_counter()
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            grp = self.layer_group[l]
            tpf.gemm_gather(T, L["qkv"], qkv)
            be.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                       head_dim=self.D, rot_dim=self.rot, neox=c.rope.neox,
                       q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=eps, gemma=False,
                       slot_mapping=ctx.slot_mapping[grp][:T], kv_cache=self.kv_caches[l],
                       block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, grp,
                         num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                         block_size=self.block_size, scale=self.scale, out=attn)
            exp = tpf.gemm_scatter(attn, L["o"])
            tpf.reduce_norm_gather(T, exp, L["ln2"], eps, False)
            # gathered rows -> local copy the MoE kernels can index (waits for every group)
            tpf.gather_all(T, normed)
            self._moe_block(normed, L, T, scatter=sc)
            nw = self.layers[l + 1]["ln1"] if l + 1 < n_layers else self.w["final_norm"]
            # every source rank delivers 32 arrivals per 32-row group (see moe_combine_kernel)
            tpf.reduce_norm_gather(T, tpf.world * 32, nw, eps, False, nsrc=tpf.world)
        return self._tp_fused_logits(ctx, T)
