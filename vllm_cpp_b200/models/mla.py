"""DeepSeek-V2 family (DeepSeek-V2-Lite shape; GLM-4-MoE-Lite shares the block): multi-head
latent attention + routed experts with shared experts; the first ``first_k_dense_replace``
layers use a dense MLP.

Attention per layer: one merged GEMM x -> [q (H x 192) | kv_c 512 | k_pe 64]; GPT-J RoPE on
q_pe / k_pe; RMSNorm on kv_c; [kv_c | k_pe] goes to the latent cache (576 values per token).
Decode rows run the absorbed form (q_nope W_UK -> multi-query attention over latent rows ->
W_UV), prefill rows the expanded form: the requests' latent rows are gathered, expanded by
kv_b_proj into per-head K = [k_nope | k_pe] and V (padded to 256 columns) and fed to the
head_dim-256 paged prefill kernel. o_proj's weight is padded to match, so both paths write
one [T, H x 256] buffer.

Reference: ``src/vllm/model_executor/models/deepseek_v2.cpp``, ``mla_attention.cpp:257-490``
(ForwardMlaAttentionBlock), ``include/vllm/model_executor/models/mla_attention.h:44-62``.
"""
from __future__ import annotations

import os

import torch

from ..config import ModelConfig, ParallelConfig
from ..ops import reference as ref
from .base import StepContext, shard_cols, shard_rows
from .dense import ACT_KIND
from .moe import MoeModel


class DeepseekV2Model(MoeModel):
    def __init__(self, cfg: ModelConfig, device="cuda", parallel: ParallelConfig | None = None,
                 comm=None, max_position: int | None = None):
        c = cfg
        assert c.kv_lora_rank == 512 and c.qk_rope_head_dim == 64 and c.qk_nope_head_dim == 128 \
            and c.v_head_dim == 128, "MLA kernels are built for the 512/64/128/128 layout"
        c.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        c.rope.rotary_dim = c.qk_rope_head_dim
        c.rope.neox = False
        super().__init__(cfg, device, parallel, comm, max_position)
        self.H = c.num_heads // self.tp            # local heads
        self.hq, self.hkv, self.D = self.H, 1, 576
        self.q_w = self.H * 192
        self.qa_w = self.q_w + 576
        self.dense_layers = c.first_k_dense_replace
        self.shared_inter = c.num_shared_experts * c.moe_intermediate_size // self.tp
        self._splits: dict[int, tuple] = {}
        self._tmp: dict = {}

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        c = self.cfg
        Hd, Hh, I = c.hidden_size, c.num_heads, c.moe_intermediate_size
        big = c.num_layers * 3 * self.E * I * Hd > 5e8
        gdev = self.device if (self.device.type == "cuda" and big) else torch.device("cpu")
        g = torch.Generator(device=gdev).manual_seed(seed)

        def full(shape, s=std):
            w = torch.empty(shape, dtype=torch.float32, device=gdev)
            w.normal_(0.0, s, generator=g)
            return w.to(self.dtype)

        def gen():
            yield "model.embed_tokens.weight", full((c.vocab_size, Hd))
            for l in range(c.num_layers):
                p = f"model.layers.{l}."
                yield p + "input_layernorm.weight", torch.ones(Hd, dtype=self.dtype)
                yield p + "post_attention_layernorm.weight", torch.ones(Hd, dtype=self.dtype)
                yield p + "self_attn.q_proj.weight", full((Hh * 192, Hd))
                yield p + "self_attn.kv_a_proj_with_mqa.weight", full((576, Hd))
                yield p + "self_attn.kv_a_layernorm.weight", torch.ones(512, dtype=self.dtype)
                yield p + "self_attn.kv_b_proj.weight", full((Hh * 256, 512))
                yield p + "self_attn.o_proj.weight", full((Hd, Hh * 128))
                if l < self.dense_layers:
                    yield p + "mlp.gate_proj.weight", full((c.intermediate_size, Hd))
                    yield p + "mlp.up_proj.weight", full((c.intermediate_size, Hd))
                    yield p + "mlp.down_proj.weight", full((Hd, c.intermediate_size))
                else:
                    yield p + "mlp.gate.weight", full((self.E, Hd))
                    yield p + "mlp.experts.gate_proj.weight", full((self.E, I, Hd))
                    yield p + "mlp.experts.up_proj.weight", full((self.E, I, Hd))
                    yield p + "mlp.experts.down_proj.weight", full((self.E, Hd, I))
                    if c.num_shared_experts:
                        S = c.num_shared_experts * I
                        yield p + "mlp.shared_experts.gate_proj.weight", full((S, Hd))
                        yield p + "mlp.shared_experts.up_proj.weight", full((S, Hd))
                        yield p + "mlp.shared_experts.down_proj.weight", full((Hd, S))
            yield "model.norm.weight", torch.ones(Hd, dtype=self.dtype)
            if not c.tie_word_embeddings:
                yield "lm_head.weight", full((c.vocab_size, Hd))

        self.load_weights(gen())

    def load_weights(self, named_tensors) -> None:
        c = self.cfg
        tp, r = self.tp, self.rank
        dev, dt = self.device, self.dtype
        H = self.H
        e0, el = self.e0, self.e_local

        def put(t):
            return t.to(dt).contiguous().to(dev)

        self.layers = [dict() for _ in range(c.num_layers)]
        pend: dict = {}
        for name, t in named_tensors:
            if name in ("model.embed_tokens.weight", "lm_head.weight"):
                pad = self.vocab_shard * tp - c.vocab_size
                if pad:
                    t = torch.cat([t, torch.zeros(pad, t.shape[1], dtype=t.dtype, device=t.device)], 0)
                key = "embed" if name.startswith("model.embed") else "lm_head"
                self.w[key] = put(t[self.vocab_start:self.vocab_start + self.vocab_shard])
                continue
            if name == "model.norm.weight":
                self.w["final_norm"] = put(t)
                continue
            if not name.startswith("model.layers."):
                continue
            parts = name.split(".")
            l = int(parts[2])
            if l >= c.num_layers:
                continue
            L = self.layers[l]
            P = pend.setdefault(l, {})
            rest = ".".join(parts[3:])
            if rest == "input_layernorm.weight":
                L["ln1"] = put(t)
            elif rest == "post_attention_layernorm.weight":
                L["ln2"] = put(t)
            elif rest in ("self_attn.q_proj.weight", "self_attn.kv_a_proj_with_mqa.weight"):
                P[parts[4]] = t
                if "q_proj" in P and "kv_a_proj_with_mqa" in P:
                    L["qkv_a"] = put(torch.cat([shard_rows(P["q_proj"], r, tp), P["kv_a_proj_with_mqa"]], 0))
                    del P["q_proj"], P["kv_a_proj_with_mqa"]
            elif rest == "self_attn.kv_a_layernorm.weight":
                L["kv_ln"] = put(t)
            elif rest == "self_attn.kv_b_proj.weight":
                w = shard_rows(t, r, tp)                            # [H*256, 512]
                L["kv_b"] = put(w)
                w3 = w.reshape(H, 256, 512)
                L["w_uk_t"] = put(w3[:, :128, :].transpose(1, 2))   # [H, 512, 128]
                L["w_uv"] = put(w3[:, 128:, :])                     # [H, 128, 512]
            elif rest == "self_attn.o_proj.weight":
                w = shard_cols(t, r, tp).reshape(t.shape[0], H, 128)
                wp = torch.zeros(t.shape[0], H, 256, dtype=w.dtype, device=w.device)
                wp[:, :, :128] = w
                L["o"] = put(wp.reshape(t.shape[0], H * 256))
                L["o_plain"] = put(shard_cols(t, r, tp)) if dev.type != "cuda" else None
            elif rest in ("mlp.gate_proj.weight", "mlp.up_proj.weight"):
                P[parts[4]] = t
                if "gate_proj" in P and "up_proj" in P:
                    L["gate_up"] = put(torch.cat([shard_rows(P["gate_proj"], r, tp),
                                                  shard_rows(P["up_proj"], r, tp)], 0))
                    del P["gate_proj"], P["up_proj"]
            elif rest == "mlp.down_proj.weight":
                L["down"] = put(shard_cols(t, r, tp))
            elif rest in ("mlp.shared_experts.gate_proj.weight", "mlp.shared_experts.up_proj.weight"):
                P["s_" + parts[5]] = t
                if "s_gate_proj" in P and "s_up_proj" in P:
                    L["s_gate_up"] = put(torch.cat([shard_rows(P["s_gate_proj"], r, tp),
                                                    shard_rows(P["s_up_proj"], r, tp)], 0))
                    del P["s_gate_proj"], P["s_up_proj"]
            elif rest == "mlp.shared_experts.down_proj.weight":
                L["s_down"] = put(shard_cols(t, r, tp))
            elif rest == "mlp.gate.weight":
                L["router"] = put(t)
            elif rest in ("mlp.experts.gate_proj.weight", "mlp.experts.up_proj.weight"):
                P["e_" + parts[5]] = t[e0:e0 + el]
                if "e_gate_proj" in P and "e_up_proj" in P:
                    L["w_gate_up"] = put(torch.cat([P["e_gate_proj"], P["e_up_proj"]], 1))
                    del P["e_gate_proj"], P["e_up_proj"]
            elif rest == "mlp.experts.down_proj.weight":
                L["w_down"] = put(t[e0:e0 + el])
            elif len(parts) >= 8 and parts[4] == "experts" and parts[5].isdigit():
                e = int(parts[5])
                if e0 <= e < e0 + el:
                    P.setdefault("pe", {})[(e, parts[6])] = t
        for l, P in pend.items():
            d = P.get("pe")
            if d:
                L = self.layers[l]
                L["w_gate_up"] = put(torch.stack([torch.cat([d[(e, "gate_proj")], d[(e, "up_proj")]], 0)
                                                  for e in range(e0, e0 + el)], 0))
                L["w_down"] = put(torch.stack([d[(e, "down_proj")] for e in range(e0, e0 + el)], 0))
        if c.tie_word_embeddings or "lm_head" not in self.w:
            self.w["lm_head"] = self.w["embed"]

    # ------------------------------------------------------------------ caches / buffers
    def kv_cache_groups(self, block_size: int):
        spec = dict(kind="mla", block_size=block_size, num_kv_heads=1, head_size=576, dtype_bytes=2)
        return [(list(range(self.cfg.num_layers)), spec)]

    def alloc_kv_cache(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.kv_caches = [torch.zeros((num_blocks, block_size, 576), dtype=self.dtype, device=self.device)
                          for _ in range(self.cfg.num_layers)]
        self.layer_group = [0] * self.cfg.num_layers
        return self.kv_caches

    def kv_bytes_per_block(self, block_size: int) -> int:
        return self.cfg.num_layers * block_size * 576 * 2

    def reserve_buffers(self, max_tokens: int, max_reqs: int) -> None:
        c = self.cfg
        H = self.H
        inter = max(self.inter, self.shared_inter)
        for name, cols in (("hidden", c.hidden_size), ("resid", c.hidden_size), ("normed", c.hidden_size),
                           ("qa", self.qa_w), ("attn_pad", H * 256), ("gate_up", 2 * inter), ("act", inter),
                           ("moe_out", c.hidden_size), ("shared_out", c.hidden_size)):
            self.bufs.reserve(name, max_tokens, cols)
        self.bufs.reserve("qabs", max_reqs, H * 576)
        self.bufs.reserve("olat", max_reqs, H * 512)
        self.bufs.reserve("qpad", max_tokens, H * 256)
        self.bufs.reserve("router", max_tokens, self.E, torch.float32)
        self.bufs.reserve("last", max_reqs, c.hidden_size)
        self.bufs.reserve("logits", max_reqs, self.vocab_shard, torch.float32)
        self.bufs.reserve("argmax_cand", max_reqs, 2, torch.int32)
        # never-written pad columns of the attention buffer must stay finite
        self.bufs.get("attn_pad", max_tokens, H * 256).zero_()
        if self.device.type == "cuda":
            from ..ops.moe import MoeWorkspace
            self.moe_ws = MoeWorkspace(self.device, max_tokens, self.k, self.e_local, c.hidden_size,
                                       self.moe_inter)

    def fused_tp_supported(self) -> bool:
        return (self.tp > 1 and self.par.fused_collectives and self.device.type == "cuda"
                and self.cfg.hidden_size % 8 == 0 and not getattr(self, "quantized", None))

    # ------------------------------------------------------------------ attention
    def _decode_plan(self, B: int, max_seq_len: int):
        key = B
        if key not in self._splits:
            from ..ops import num_sms
            tiles = max(1, -(-max(self.max_position, 1) // 128))
            # one CTA fits on an SM (the latent ring takes the shared memory): split only while all
            # (sequence, split) CTAs still run in one wave
            s = max(1, min(num_sms() // max(B, 1), max(1, tiles // 2), 16))
            tmp = None
            if s > 1:
                tmp = (torch.empty((B, self.H, s, 512), dtype=torch.float32, device=self.device),
                       torch.empty((B, self.H, s), dtype=torch.float32, device=self.device))
            self._splits[key] = (s, tmp)
        return self._splits[key]

    def _prefill_meta(self, ctx: StepContext) -> dict:
        """Dense layout of the prefill requests' contexts (block aligned) and its identity
        block table; built from the step's host arrays, one small copy."""
        import numpy as np
        nd, P, bs = ctx.num_decodes, ctx.num_prefills, self.block_size
        host = ctx.extra.get("host")
        seq = (host["seq_lens"][nd:nd + P].numpy() if host is not None
               else ctx.seq_lens[nd:nd + P].cpu().numpy()).astype(np.int64)
        nblk = (seq + bs - 1) // bs
        base_blk = np.concatenate([[0], np.cumsum(nblk)[:-1]])
        total_blk = int(nblk.sum())
        mb = int(nblk.max())
        bt = np.zeros((P, mb), dtype=np.int32)
        for i in range(P):
            bt[i, : nblk[i]] = base_blk[i] + np.arange(nblk[i])
        packed = np.concatenate([(base_blk * bs).astype(np.int32), bt.reshape(-1)])
        dev = torch.from_numpy(packed).to(self.device)
        return dict(base=dev[:P], bt=dev[P:].view(P, mb), total=total_blk * bs, max_blocks=mb)

    def _attention_gpu(self, l: int, L: dict, qa: torch.Tensor, ctx: StepContext, T: int, meta: dict,
                       attn: torch.Tensor):
        from ..ops import mla as M
        ops = self.be.ops
        H, bs, nd = self.H, self.block_size, ctx.num_decodes
        cache = self.kv_caches[l]
        if nd > 0:
            qabs = self.bufs.get("qabs", nd, H * 576)
            olat = self.bufs.get("olat", nd, H * 512)
            M.gemm_batched(qa[:nd], 192, L["w_uk_t"], qabs, 576, nd, 512, 128, H)
            M.copy_qpe(qa[:nd], qabs, nd, H)
            s, tmp = self._decode_plan(nd, ctx.max_seq_len)
            M.mla_decode(qabs.view(nd, H, 576), cache, ctx.block_table[0][:nd], ctx.seq_lens[:nd],
                         olat, self.scale, bs, splits=s, tmp=tmp)
            M.gemm_batched(olat, 512, L["w_uv"], attn[:nd], 256, nd, 128, 512, H)
        if ctx.num_prefills > 0:
            P, Tp = ctx.num_prefills, T - nd
            n_ctx = meta["total"]
            dense = self._scratch("mla_dense", n_ctx, 576)
            kvb = self._scratch("mla_kvb", n_ctx, H * 256)
            tmpc = self._scratch("mla_cache", n_ctx * 2, H * 256)
            M.gather_latent(cache, ctx.block_table[0][nd:nd + P], ctx.seq_lens[nd:nd + P], meta["base"], bs,
                            dense, P, meta["max_blocks"])
            ops.gemm(dense[:, :512], L["kv_b"], out=kvb)
            M.assemble_kv(kvb, dense, tmpc, n_ctx, H, bs)
            qpad = self.bufs.get("qpad", Tp, H * 256)
            M.pad_q(qa[nd:], qpad, Tp, H)
            ops.attn_prefill(qpad, tmpc.view(n_ctx // bs, 2, bs, H, 256), block_table=meta["bt"],
                             seq_lens=ctx.seq_lens[nd:nd + P], q_start=ctx.prefill_q_start,
                             tile_req=ctx.tile_req[:ctx.num_tiles], tile_q0=ctx.tile_q0[:ctx.num_tiles],
                             num_q_heads=H, num_kv_heads=H, head_dim=256, block_size=bs, scale=self.scale,
                             out=attn[nd:])

    def _scratch(self, name: str, rows: int, cols: int) -> torch.Tensor:
        t = self._tmp.get(name)
        if t is None or t.shape[0] < rows or t.shape[1] != cols:
            t = torch.zeros((max(rows, 1), cols), dtype=self.dtype, device=self.device)
            self._tmp[name] = t
        return t[:rows]

    def _attention_cpu(self, l: int, L: dict, qa: torch.Tensor, ctx: StepContext, T: int, attn: torch.Tensor):
        from ..ops import mla as M
        H = self.H
        if qa.dtype == torch.bfloat16 and os.environ.get("B200_CPU_ORACLE", "0") != "1":
            # native thread-pool op (csrc/cpu/cpu_ops_ext.cpp); the PyTorch restatement is its oracle
            from ..ops import cpu_native as N
            q = qa[:, : self.q_w].view(T, H, 192)
            R = ctx.num_reqs
            out = N.mla_attention(q, self.kv_caches[l], ctx.block_table[0][:R], ctx.seq_lens[:R],
                                  ctx.query_start[: R + 1], L["kv_b"], H, self.scale, self.block_size)
        else:
            q = qa[:, : self.q_w].reshape(T, H, 192)
            out = M.ref_mla_attention(q, self.kv_caches[l], ctx.block_table[0], ctx.seq_lens, ctx.query_start,
                                      L["kv_b"], H, self.scale, self.block_size)
        a = attn.view(T, H, 256)
        a.zero_()
        a[:, :, :128] = out.to(attn.dtype)

    def _rope_cpu(self, qa: torch.Tensor, pos: torch.Tensor, T: int):
        """GPT-J (interleaved) rotation of q_pe of every head and of k_pe, in place."""
        cs = self.rope_table[pos.long()].float()             # [T, 64] = cos(32) | sin(32)
        cos, sin = cs[:, :32], cs[:, 32:]

        def rot(x):                                          # x [T, n, 64]
            xf = x.float()
            a, b = xf[..., 0::2], xf[..., 1::2]
            o = torch.empty_like(xf)
            o[..., 0::2] = a * cos[:, None] - b * sin[:, None]
            o[..., 1::2] = b * cos[:, None] + a * sin[:, None]
            return o.to(x.dtype)

        q = qa[:, : self.q_w].view(T, self.H, 192)
        q[:, :, 128:] = rot(q[:, :, 128:])
        kpe = qa[:, self.q_w + 512:].view(T, 1, 64)
        kpe.copy_(rot(kpe))

    # ------------------------------------------------------------------ forward
    def _forward_tp_fused_mla(self, ctx: StepContext):
        """Tensor-parallel heads + expert-parallel experts with every collective inside a kernel:
        o_proj / down_proj scatter their partial rows to the owners in the GEMM epilogue, the owner
        reduces + adds the residual + normalises + all-gathers, q / kv_a / gate_up GEMMs wait for the
        gathered rows tile by tile, and the MoE combine (routed sum + this rank's part of the shared
        experts) stores straight into the owners' receive slots. The would-be collective sites in
        the reference: ``src/vllm/model_executor/layers/attention/mla_attention.cpp:487`` and
        ``src/vllm/model_executor/models/deepseek_v2.cpp:289,464-466``."""
        from ..ops.moe import B200MoeScatter
        c, be, T, tpf = self.cfg, self.be, ctx.num_tokens, self.tpf
        Hd, eps = c.hidden_size, c.rms_norm_eps
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, Hd)
        normed = self.bufs.get("normed", T, Hd)
        qa = self.bufs.get("qa", T, self.qa_w)
        attn = self.bufs.get("attn_pad", T, self.H * 256)
        be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                     vocab_total=c.vocab_size)
        self.comm.all_reduce(hidden)
        tpf.first_norm(hidden, self.layers[0]["ln1"], eps, False)
        pos = ctx.positions[:T]
        meta = self._prefill_meta(ctx) if ctx.num_prefills > 0 else {}
        kvc = qa[:, self.q_w: self.q_w + 512]
        kpe = qa[:, self.q_w + 512:]
        sc = B200MoeScatter()
        sc.world, sc.rank, sc.rows_per_rank = tpf.world, tpf.rank, tpf.rows_per_rank(T)
        for r in range(tpf.world):
            sc.peer_recv[r] = tpf.recv.ptrs[r]
            sc.peer_rs_flags[r] = tpf._rs_flags(r)
        sc.recv_parity_stride, sc.rs_flag_parity_stride = tpf.recv_parity, tpf.rs_groups
        sc.op_counter = tpf._op_counter()
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            tpf.gemm_gather(T, L["qkv_a"], qa)
            be.ops.rope_kv(qa, pos, self.rope_table, num_q_heads=self.H, num_kv_heads=1, head_dim=64,
                           rot_dim=64, neox=False, q_head_stride=192, offsets=(128, self.q_w + 512, 0))
            be.ops.rmsnorm(kvc, L["kv_ln"], eps, out=kvc)
            be.ops.concat_and_cache_mla(kvc, kpe, ctx.slot_mapping[0][:T], self.kv_caches[l])
            self._attention_gpu(l, L, qa, ctx, T, meta, attn)
            exp = tpf.gemm_scatter(attn, L["o"])
            tpf.reduce_norm_gather(T, exp, L["ln2"], eps, False)
            nw = self.layers[l + 1]["ln1"] if l + 1 < n_layers else self.w["final_norm"]
            if l < self.dense_layers:
                gu = self.bufs.get("gate_up", T, 2 * self.inter)
                tpf.gemm_gather(T, L["gate_up"], gu)
                a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("act", T, self.inter))
                exp = tpf.gemm_scatter(a_, L["down"])
                tpf.reduce_norm_gather(T, exp, nw, eps, False)
                continue
            # gathered rows -> local copy that the router, the expert gather and the shared experts read
            tpf.gather_all(T, normed)
            shared = None
            if "s_gate_up" in L:
                gu = self.bufs.get("gate_up", T, 2 * self.shared_inter)
                be.gemm(normed, L["s_gate_up"], out=gu)
                a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("act", T, self.shared_inter))
                shared = be.gemm(a_, L["s_down"], out=self.bufs.get("shared_out", T, Hd))
            self._moe_block(normed, L, T, scatter=sc, shared=shared)
            # every source rank delivers 32 arrivals per 32-row group (see moe_combine_kernel)
            tpf.reduce_norm_gather(T, tpf.world * 32, nw, eps, False, nsrc=tpf.world)
        return self._tp_fused_logits(ctx, T)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        if getattr(self, "tpf", None) is not None:
            return self._forward_tp_fused_mla(ctx)
        c, be, T = self.cfg, self.be, ctx.num_tokens
        Hd, eps = c.hidden_size, c.rms_norm_eps
        cuda = self.device.type == "cuda"
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, Hd)
        resid = self.bufs.get("resid", T, Hd)
        normed = self.bufs.get("normed", T, Hd)
        qa = self.bufs.get("qa", T, self.qa_w)
        attn = self.bufs.get("attn_pad", T, self.H * 256)
        e = be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                         vocab_total=c.vocab_size)
        if e is not hidden:
            hidden.copy_(e)
        if self.tp > 1:
            self.comm.all_reduce(hidden)
        pos = ctx.positions[:T]
        meta = self._prefill_meta(ctx) if (cuda and ctx.num_prefills > 0) else {}
        kvc = qa[:, self.q_w: self.q_w + 512]
        kpe = qa[:, self.q_w + 512:]
        for l, L in enumerate(self.layers):
            if l == 0:
                resid.copy_(hidden)
                x = be.rmsnorm(hidden, L["ln1"], eps, out=normed)
            else:
                x = be.rmsnorm(hidden, L["ln1"], eps, residual=resid, out=normed)
            be.gemm(x, L["qkv_a"], out=qa)
            if cuda:
                be.ops.rope_kv(qa, pos, self.rope_table, num_q_heads=self.H, num_kv_heads=1, head_dim=64,
                               rot_dim=64, neox=False, q_head_stride=192,
                               offsets=(128, self.q_w + 512, 0))
                be.ops.rmsnorm(kvc, L["kv_ln"], eps, out=kvc)
                be.ops.concat_and_cache_mla(kvc, kpe, ctx.slot_mapping[0][:T], self.kv_caches[l])
                self._attention_gpu(l, L, qa, ctx, T, meta, attn)
            else:
                self._rope_cpu(qa, pos, T)
                n, _ = ref.rmsnorm(kvc.contiguous(), L["kv_ln"], eps, None, False)
                kvc.copy_(n)
                flat = self.kv_caches[l].view(-1, 576)
                slots = ctx.slot_mapping[0][:T].long()
                ok = slots >= 0
                flat[slots[ok]] = torch.cat([kvc, kpe], 1)[ok]
                self._attention_cpu(l, L, qa, ctx, T, attn)
            be.gemm(attn, L["o"], out=hidden)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
            x = be.rmsnorm(hidden, L["ln2"], eps, residual=resid, out=normed)
            if l < self.dense_layers:
                gu = self.bufs.get("gate_up", T, 2 * self.inter)
                be.gemm(x, L["gate_up"], out=gu)
                a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("act", T, self.inter))
                be.gemm(a_, L["down"], out=hidden)
            else:
                m = self._moe_block(x, L, T)
                if "s_gate_up" in L:
                    gu = self.bufs.get("gate_up", T, 2 * self.shared_inter)
                    be.gemm(x, L["s_gate_up"], out=gu)
                    a_ = be.act_and_mul(gu, act_kind, out=self.bufs.get("act", T, self.shared_inter))
                    # shared experts add onto the routed sum (residual input of the GEMM epilogue)
                    be.gemm(a_, L["s_down"], residual=m, out=hidden)
                else:
                    hidden.copy_(m)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
        full = be.rmsnorm(hidden, self.w["final_norm"], eps, residual=resid, out=normed)
        if ctx.decode_only_full_logits:
            n, last = T, full
        else:
            n = ctx.num_logits
            last = be.gather_rows(full, ctx.logits_indices[:n], out=self.bufs.get("last", n, Hd))
        logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
        be.gemm(last, self.w["lm_head"], out=logits, out_dtype=torch.float32)
        if self.tp > 1:
            logits = self.comm.all_gather(logits, dim=-1)
        return logits[:, : c.vocab_size] if logits.shape[1] != c.vocab_size else logits
