"""Dense decoder family: Llama / Mistral / Qwen3 / Gemma(2,3) / GLM-4 / OLMo-2,3 / Phi-3 /
Granite, all expressed as one block with switches (per-head qk-norm, biases, sandwich or
post norms, GeGLU, soft-caps, scalar multipliers, sliding-window layers, tied embeddings).

Per layer:  (add+)RMSNorm -> merged QKV GEMM -> fused qk-norm + RoPE + KV write -> paged
attention -> o_proj GEMM [TP: reduce] -> add+RMSNorm -> merged gate_up GEMM -> act*mul ->
down GEMM [TP: reduce]. Only the rows that sample a token go through the lm_head.

Reference forward: ``src/vllm/model_executor/models/qwen3.cpp:135-244``,
``include/vllm/model_executor/models/dense_attn_block.h:311-512``; the other families are
``gemma*.cpp``, ``glm4.cpp``, ``olmo2.cpp``, ``phi3.cpp``, ``granite.cpp``.
"""
from __future__ import annotations

import os

import torch

from ..config import ModelConfig, ParallelConfig
from ..utils import nvtx
from .backend import make_backend
from .base import BufferPool, StepContext, normal_, shard_cols, shard_rows
from .rope import rope_parameters, softmax_scale

ACT_KIND = {"silu": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "gelu": 2}


class DenseModel:
    def __init__(self, cfg: ModelConfig, device="cuda", parallel: ParallelConfig | None = None,
                 comm=None, max_position: int | None = None):
        from ..parallel.comm import SingleComm
        self.cfg = cfg
        self.device = torch.device(device)
        self.par = parallel or ParallelConfig()
        self.comm = comm or SingleComm()
        self.tp = self.par.tensor_parallel_size
        self.rank = self.par.rank
        self.be = make_backend(self.device)
        self.dtype = torch.bfloat16
        c = cfg
        assert c.num_heads % self.tp == 0
        self.hq = c.num_heads // self.tp
        # kv heads are replicated when there are more ranks than kv heads
        self.hkv = max(1, c.num_kv_heads // self.tp)
        self.kv_rep = max(1, self.tp // c.num_kv_heads)
        self.D = c.head_dim
        self.inter = c.intermediate_size // self.tp
        self.vocab_shard = (c.vocab_size + self.tp - 1) // self.tp
        self.vocab_start = self.rank * self.vocab_shard
        self.max_position = max_position or c.max_position_embeddings
        inv, msc, tlen = rope_parameters(c.rope, c.head_dim, self.max_position)
        self.rot = c.rope.rotary_dim or c.head_dim
        self.rope_table = self.be.rope_table(inv, min(tlen, self.max_position), msc)
        self.scale = c.attention_multiplier if c.attention_multiplier is not None else \
            softmax_scale(c.rope, c.head_dim)
        self.bufs = BufferPool(self.device)
        self.gate_up_il = False      # set by load_weights when it stores gate / up interleaved
        self.native_layers = None    # decided at the first forward; False forces the per-op path
        self.w: dict[str, torch.Tensor] = {}
        self.layers: list[dict[str, torch.Tensor]] = []

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random N(0, std) weights of the configured shape; every rank draws the full tensor
        from the same generator and keeps its shard, so any TP degree sees the same model."""
        c = self.cfg
        H, D = c.hidden_size, c.head_dim
        # Small models draw on the CPU generator (bit-identical on any device, used by the
        # CPU-vs-GPU gates); big ones draw on the device to keep start-up short.
        n_params = c.num_layers * (2 * c.num_heads * D * H + 3 * c.intermediate_size * H)
        gdev = self.device if (self.device.type == "cuda" and n_params > 5e8) else torch.device("cpu")
        g = torch.Generator(device=gdev).manual_seed(seed)

        def full(shape):
            w = torch.empty(shape, dtype=torch.float32, device=gdev)
            w.normal_(0.0, std, generator=g)
            return w.to(self.dtype)

        emb = full((c.vocab_size, H))
        tensors = {"model.embed_tokens.weight": emb}
        for l in range(c.num_layers):
            p = f"model.layers.{l}."
            tensors[p + "self_attn.q_proj.weight"] = full((c.num_heads * D, H))
            tensors[p + "self_attn.k_proj.weight"] = full((c.num_kv_heads * D, H))
            tensors[p + "self_attn.v_proj.weight"] = full((c.num_kv_heads * D, H))
            tensors[p + "self_attn.o_proj.weight"] = full((H, c.num_heads * D))
            tensors[p + "mlp.gate_proj.weight"] = full((c.intermediate_size, H))
            tensors[p + "mlp.up_proj.weight"] = full((c.intermediate_size, H))
            tensors[p + "mlp.down_proj.weight"] = full((H, c.intermediate_size))
            ones = torch.ones(H, dtype=self.dtype) if not c.gemma_norm else torch.zeros(H, dtype=self.dtype)
            tensors[p + "input_layernorm.weight"] = ones.clone()
            tensors[p + "post_attention_layernorm.weight"] = ones.clone()
            if c.sandwich_norm:
                tensors[p + "pre_feedforward_layernorm.weight"] = ones.clone()
                tensors[p + "post_feedforward_layernorm.weight"] = ones.clone()
            if c.qk_norm:
                hd1 = torch.ones(D, dtype=self.dtype) if not c.gemma_norm else torch.zeros(D, dtype=self.dtype)
                tensors[p + "self_attn.q_norm.weight"] = hd1.clone()
                tensors[p + "self_attn.k_norm.weight"] = hd1.clone()
            if c.attention_bias:
                tensors[p + "self_attn.q_proj.bias"] = full((c.num_heads * D,))
                tensors[p + "self_attn.k_proj.bias"] = full((c.num_kv_heads * D,))
                tensors[p + "self_attn.v_proj.bias"] = full((c.num_kv_heads * D,))
        tensors["model.norm.weight"] = (torch.ones(H, dtype=self.dtype) if not c.gemma_norm
                                        else torch.zeros(H, dtype=self.dtype))
        if not c.tie_word_embeddings:
            tensors["lm_head.weight"] = full((c.vocab_size, H))
        self.load_weights(tensors.items())

    def load_weights(self, named_tensors) -> None:
        """Accepts HF-named full (unsharded) tensors; merges q|k|v and gate|up and keeps this
        rank's shard. Pre-fused ``qkv_proj`` / ``gate_up_proj`` (Phi-3) are split first."""
        c, D = self.cfg, self.cfg.head_dim
        tp, r = self.tp, self.rank
        staged: dict[str, torch.Tensor] = {}
        for name, t in named_tensors:
            if name.endswith("qkv_proj.weight"):
                base = name[: -len("qkv_proj.weight")]
                nq, nk = c.num_heads * D, c.num_kv_heads * D
                staged[base + "q_proj.weight"] = t[:nq]
                staged[base + "k_proj.weight"] = t[nq:nq + nk]
                staged[base + "v_proj.weight"] = t[nq + nk:]
            elif name.endswith("gate_up_proj.weight"):
                base = name[: -len("gate_up_proj.weight")]
                staged[base + "gate_proj.weight"] = t[: c.intermediate_size]
                staged[base + "up_proj.weight"] = t[c.intermediate_size:]
            else:
                staged[name] = t
        dev, dt = self.device, self.dtype

        def put(t):
            return t.to(dt).contiguous().to(dev)

        def kv_shard(w):  # rows = kv heads * D
            if self.kv_rep > 1:
                h = r // self.kv_rep
                return w[h * D:(h + 1) * D]
            return shard_rows(w, r, tp)

        emb = staged["model.embed_tokens.weight"]
        pad = self.vocab_shard * tp - c.vocab_size
        if pad:
            emb = torch.cat([emb, torch.zeros(pad, emb.shape[1], dtype=emb.dtype,
                                              device=emb.device)], 0)
        self.w["embed"] = put(emb[self.vocab_start:self.vocab_start + self.vocab_shard])
        if (tp > 1 and self.par.fused_collectives and self.device.type == "cuda"
                and emb.numel() * 2 <= (4 << 30)):
            # fused tensor parallel: every rank keeps the whole embedding table (a few GB at most)
            # and looks its tokens up locally instead of all-reducing [tokens, hidden] every step
            # (1.0 ms of an 11.5 ms step at 8 GPUs). The lm_head stays sharded over the vocabulary.
            self.w["embed_full"] = put(emb)
        if c.tie_word_embeddings or "lm_head.weight" not in staged:
            self.w["lm_head"] = self.w["embed"]
        else:
            lm = staged["lm_head.weight"]
            if pad:
                lm = torch.cat([lm, torch.zeros(pad, lm.shape[1], dtype=lm.dtype,
                                                device=lm.device)], 0)
            self.w["lm_head"] = put(lm[self.vocab_start:self.vocab_start + self.vocab_shard])
        self.w["final_norm"] = put(staged["model.norm.weight"])
        self.layers = []
        # On the GPU the merged gate / up projection is stored in blocks of [128 gate | 128 up]
        # rows, so that the GEMM epilogue can apply the gated activation (see ops.gemm_gated).
        self.gate_up_il = (self.device.type == "cuda" and self.dtype == torch.bfloat16 and
                           self.inter % 128 == 0 and not self.cfg.mlp_bias)
        for l in range(c.num_layers):
            p = f"model.layers.{l}."
            L: dict[str, torch.Tensor] = {}
            q = shard_rows(staged[p + "self_attn.q_proj.weight"], r, tp)
            k = kv_shard(staged[p + "self_attn.k_proj.weight"])
            v = kv_shard(staged[p + "self_attn.v_proj.weight"])
            L["qkv"] = put(torch.cat([q, k, v], 0))
            if c.attention_bias and (p + "self_attn.q_proj.bias") in staged:
                L["qkv_bias"] = put(torch.cat([
                    shard_rows(staged[p + "self_attn.q_proj.bias"][:, None], r, tp)[:, 0],
                    kv_shard(staged[p + "self_attn.k_proj.bias"][:, None])[:, 0],
                    kv_shard(staged[p + "self_attn.v_proj.bias"][:, None])[:, 0]], 0))
            L["o"] = put(shard_cols(staged[p + "self_attn.o_proj.weight"], r, tp))
            g = shard_rows(staged[p + "mlp.gate_proj.weight"], r, tp)
            u = shard_rows(staged[p + "mlp.up_proj.weight"], r, tp)
            if self.gate_up_il:
                from ..ops import interleave_gate_up
                L["gate_up"] = put(interleave_gate_up(g, u))
            else:
                L["gate_up"] = put(torch.cat([g, u], 0))
            L["down"] = put(shard_cols(staged[p + "mlp.down_proj.weight"], r, tp))
            L["ln1"] = put(staged[p + "input_layernorm.weight"])
            L["ln2"] = put(staged[p + "post_attention_layernorm.weight"])
            if c.sandwich_norm:
                L["ln_pre_ff"] = put(staged[p + "pre_feedforward_layernorm.weight"])
                L["ln_post_ff"] = put(staged[p + "post_feedforward_layernorm.weight"])
            if c.qk_norm and (p + "self_attn.q_norm.weight") in staged:
                L["q_norm"] = put(staged[p + "self_attn.q_norm.weight"])
                L["k_norm"] = put(staged[p + "self_attn.k_norm.weight"])
            self.layers.append(L)

    QUANT_KEYS = ("qkv", "o", "gate_up", "down", "in_proj", "out")

    def quantize_weights(self, method: str = "nvfp4") -> None:
        """Replaces the linear-layer weights by NVFP4 ``QuantWeight``s, or by ``Fp8Weight``s for
        ``"fp8"`` (values are rounded once here, on whatever device holds them, so CPU oracle and
        GPU see the same numbers)."""
        if method in ("q8_0", "q4_0"):
            # CPU backend: GGUF block formats, GEMMs on the packed weights
            from .backend import BlockQuantWeight
            for L in self.layers:
                for k in self.QUANT_KEYS:
                    w = L.get(k)
                    if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 32 == 0:
                        L[k] = BlockQuantWeight.from_dense(w, method)
            self.quantized = method
            return
        if method == "fp8":
            # W8A8: e4m3 weights with per-channel scales, activations quantised per call
            from .backend import Fp8Weight
            self.native_layers = None
            for L in self.layers:
                for k in self.QUANT_KEYS:
                    w = L.get(k)
                    if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 16 == 0 and w.shape[0] % 8 == 0:
                        L[k] = Fp8Weight.from_dense(w)
            self.quantized = method
            return
        if method != "nvfp4":
            raise ValueError(f"unsupported weight quantisation {method!r}")
        from .backend import QuantWeight
        self.native_layers = None
        for L in self.layers:
            for k in self.QUANT_KEYS:
                w = L.get(k)
                if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 64 == 0:
                    L[k] = QuantWeight.from_dense(w)
        self.quantized = method

    def _layer_window(self, l: int) -> int:
        """Attention span of layer ``l`` as the kernels take it: > 0 a sliding window, < 0
        chunked-local attention with chunks of that many tokens (a query sees its own chunk,
        reference ``ChunkedLocalAttentionSpec``), 0 the whole context."""
        c = self.cfg
        lt = c.layer_types[l] if c.layer_types else None
        if c.attention_chunk_size and lt == "chunked_attention":
            return -c.attention_chunk_size
        if c.sliding_window and (lt is None or lt == "sliding_attention"):
            return c.sliding_window
        return 0

    # ------------------------------------------------------------------ KV cache
    def kv_cache_groups(self, block_size: int):
        """[(layer indices, spec dict)] -- one group for full attention; sliding-window and
        chunked-local layers form further groups when the model mixes them."""
        c = self.cfg
        full, sliding, chunked = [], [], []
        for l in range(c.num_layers):
            w = self._layer_window(l)
            (chunked if w < 0 else sliding if (w > 0 and c.layer_types) else full).append(l)
        groups = []
        spec = dict(kind="full", block_size=block_size, num_kv_heads=self.hkv, head_size=self.D,
                    dtype_bytes=2)
        if full:
            groups.append((full, dict(spec)))
        if sliding:
            s = dict(spec)
            s.update(kind="sliding", sliding_window=c.sliding_window)
            groups.append((sliding, s))
        if chunked:
            s = dict(spec)
            s.update(kind="chunked", attention_chunk_size=c.attention_chunk_size)
            groups.append((chunked, s))
        return groups

    def alloc_kv_cache(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.kv_caches = [torch.zeros((num_blocks, 2, block_size, self.hkv, self.D),
                                      dtype=self.dtype, device=self.device)
                          for _ in range(self.cfg.num_layers)]
        self.layer_group = [0] * self.cfg.num_layers
        for gi, (layers, _) in enumerate(self.kv_cache_groups(block_size)):
            for l in layers:
                self.layer_group[l] = gi
        return self.kv_caches

    def kv_bytes_per_block(self, block_size: int) -> int:
        return self.cfg.num_layers * 2 * block_size * self.hkv * self.D * 2

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for t in list(self.w.values()) + [t for L in self.layers for t in L.values()]:
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n

    def reserve_buffers(self, max_tokens: int, max_reqs: int) -> None:
        c = self.cfg
        qkv_w = (self.hq + 2 * self.hkv) * self.D
        for name, cols in (("hidden", c.hidden_size), ("resid", c.hidden_size),
                           ("normed", c.hidden_size), ("qkv", qkv_w), ("attn", self.hq * self.D),
                           ("gate_up", 2 * self.inter), ("act", self.inter)):
            self.bufs.reserve(name, max_tokens, cols)
        self.bufs.reserve("last", max_reqs, c.hidden_size)
        self.bufs.reserve("logits", max_reqs, self.vocab_shard, torch.float32)
        self.bufs.reserve("argmax_cand", max_reqs, 2, torch.int32)

    # ------------------------------------------------------------------ forward
    # ------------------------------------------------------------------ fused TP forward
    def fused_tp_supported(self) -> bool:
        if getattr(self, "quantized", None):
            return False
        c = self.cfg
        return (self.tp > 1 and self.par.fused_collectives and self.device.type == "cuda"
                and not c.sandwich_norm and not c.post_norm and not c.attention_bias
                and c.residual_multiplier == 1.0 and c.hidden_size % 8 == 0)

    def enable_fused_tp(self, max_tokens: int) -> None:
        from ..parallel.tp_fused import OneShotAllReduce, TpFusedContext
        self.tpf = TpFusedContext(self.comm, self.device, self.cfg.hidden_size, max_tokens)
        # decode-sized steps: one-shot all-reduce + norm between plain small-M GEMMs instead of the
        # scatter / reduce / gather chain (B200_TP_ONESHOT_MAX=0 keeps every step on the chain)
        self.oneshot_max = min(int(os.environ.get("B200_TP_ONESHOT_MAX", "256")), max_tokens)
        self.tpf.oneshot = None
        if self.oneshot_max > 0 and type(self).forward is DenseModel.forward:
            self.tpf.oneshot = OneShotAllReduce(self.comm, self.device, self.cfg.hidden_size,
                                                self.oneshot_max)
        # with a "greedy_out" buffer in the step context the forward returns None and leaves the
        # argmax ids there (see the end of _forward_tp_fused)
        self.samples_greedy = self.cfg.final_logit_softcap <= 0

    def _forward_tp_fused(self, ctx: StepContext) -> torch.Tensor:
        """Sequence-parallel forward: every o_proj / down_proj is GEMM + reduce-scatter (scatter
        epilogue), followed by reduce + residual + RMSNorm + all-gather on the row shard, and
        every qkv / gate_up GEMM waits for its gathered rows tile by tile."""
        c, be, T, tpf = self.cfg, self.be, ctx.num_tokens, self.tpf
        if tpf.oneshot is not None and T <= self.oneshot_max:
            return self._forward_tp_oneshot(ctx)
        H, eps = c.hidden_size, c.rms_norm_eps
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, H)
        qkv = self.bufs.get("qkv", T, (self.hq + 2 * self.hkv) * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        gate_up = self.bufs.get("gate_up", T, 2 * self.inter)
        act = self.bufs.get("act", T, self.inter)
        self._tp_embed(ctx, T, hidden)
        tpf.first_norm(hidden, self.layers[0]["ln1"], eps, c.gemma_norm)
        pos = ctx.positions[:T]
        n_layers = len(self.layers)
        layers = self.layers
        if self.native_layers is None:
            self.native_layers = self._native_tp_ok()
        if self.native_layers and not nvtx.ENABLED:
            s = self._native_step(ctx, T, qkv, attn, gate_up, act, act_kind)
            if s is not None:
                from ..ops.layer import dense_layers_tp
                dense_layers_tp(self._native_weights(), s, tpf.native_ctx(self.w["final_norm"]))
                layers = []                    # every block already ran
        for l, L in enumerate(layers):
            grp = self.layer_group[l]
            window = self._layer_window(l)
            tpf.gemm_gather(T, L["qkv"], qkv)
            be.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                       head_dim=self.D, rot_dim=self.rot, neox=c.rope.neox,
                       q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=eps,
                       gemma=c.gemma_norm, slot_mapping=ctx.slot_mapping[grp][:T],
                       kv_cache=self.kv_caches[l], block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, grp,
                         num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                         block_size=self.block_size, scale=self.scale, out=attn,
                         softcap=c.attn_logit_softcap, window=window)
            exp = tpf.gemm_scatter(attn, L["o"])
            tpf.reduce_norm_gather(T, exp, L["ln2"], eps, c.gemma_norm)
            if self.gate_up_il and T > 256 and (2 * self.inter) % 256 == 0:
                tpf.gemm_gather(T, L["gate_up"], act, act_fuse=act_kind + 1)
            else:
                tpf.gemm_gather(T, L["gate_up"], gate_up)
                be.act_and_mul(gate_up, act_kind, out=act, interleaved=self.gate_up_il)
            exp = tpf.gemm_scatter(act, L["down"])
            nw = self.layers[l + 1]["ln1"] if l + 1 < n_layers else self.w["final_norm"]
            tpf.reduce_norm_gather(T, exp, nw, eps, c.gemma_norm)
        return self._tp_fused_logits(ctx, T)

    def _tp_embed(self, ctx: StepContext, T: int, hidden: torch.Tensor) -> None:
        """Token embeddings of the step on every rank: a local look-up in the replicated table, or the
        vocabulary-parallel look-up + NCCL all-reduce when the table is sharded. (The collective is
        not needed to order the passes of the fused chain: every pass ends in the all-gather of
        ``_tp_logits_tail``, which no rank enters before its last reduce kernel has been issued.)"""
        c = self.cfg
        full = self.w.get("embed_full")
        if full is not None:
            self.be.embedding(ctx.input_ids[:T], full, out=hidden, vocab_start=0,
                              vocab_total=full.shape[0], scale=c.embed_scale)
            return
        self.be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden, vocab_start=self.vocab_start,
                          vocab_total=c.vocab_size, scale=c.embed_scale)
        self.comm.all_reduce(hidden)

    def _forward_tp_oneshot(self, ctx: StepContext):
        """Decode-sized steps under tensor parallelism: every projection is a plain small-batch GEMM
        on this rank's shard; o_proj / down_proj write their partial rows into a peer-readable buffer
        and ONE kernel per site reads all ranks' partials, adds the residual and applies the next
        RMSNorm (``OneShotAllReduce``). Same arithmetic on every rank, so all ranks hold the same
        activations bit for bit. Two sites per block keep the buffer parity of a forward pass fixed."""
        c, be, T, osr = self.cfg, self.be, ctx.num_tokens, self.tpf.oneshot
        H, eps = c.hidden_size, c.rms_norm_eps
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, H)
        resid = self.bufs.get("resid", T, H)
        normed = self.bufs.get("normed", T, H)
        qkv = self.bufs.get("qkv", T, (self.hq + 2 * self.hkv) * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        gate_up = self.bufs.get("gate_up", T, 2 * self.inter)
        act = self.bufs.get("act", T, self.inter)
        self._tp_embed(ctx, T, hidden)
        resid.copy_(hidden)
        x = be.rmsnorm(hidden, self.layers[0]["ln1"], eps, out=normed, gemma=c.gemma_norm)
        osr.begin_forward()
        pos = ctx.positions[:T]
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            grp = self.layer_group[l]
            window = self._layer_window(l)
            be.gemm(x, L["qkv"], out=qkv)
            be.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                       head_dim=self.D, rot_dim=self.rot, neox=c.rope.neox,
                       q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=eps,
                       gemma=c.gemma_norm, slot_mapping=ctx.slot_mapping[grp][:T],
                       kv_cache=self.kv_caches[l], block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, grp,
                         num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                         block_size=self.block_size, scale=self.scale, out=attn,
                         softcap=c.attn_logit_softcap, window=window)
            be.gemm(attn, L["o"], out=osr.partial_out(T))
            x = osr.allreduce_norm(T, L["ln2"], eps, c.gemma_norm, resid, normed)
            if self.gate_up_il:
                a = be.gemm_gated(x, L["gate_up"], act_kind, out=act, scratch=gate_up)
            else:
                be.gemm(x, L["gate_up"], out=gate_up)
                a = be.act_and_mul(gate_up, act_kind, out=act)
            be.gemm(a, L["down"], out=osr.partial_out(T))
            nw = self.layers[l + 1]["ln1"] if l + 1 < n_layers else self.w["final_norm"]
            x = osr.allreduce_norm(T, nw, eps, c.gemma_norm, resid, normed)
        # `normed` holds the final norm of every row
        if ctx.decode_only_full_logits:
            n, last = T, normed
        else:
            n = ctx.num_logits
            last = be.gather_rows(normed, ctx.logits_indices[:n], out=self.bufs.get("last", n, H))
        logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
        be.gemm(last, self.w["lm_head"], out=logits, out_dtype=torch.float32)
        return self._tp_logits_tail(ctx, logits, n)

    def _tp_fused_logits(self, ctx: StepContext, T: int):
        """lm_head over the gathered final-norm rows. With a ``greedy_out`` buffer in the step
        context the argmax ids are left there and None is returned; otherwise fp32 logits
        ``[num_logits, vocab]`` (all-gathered over the vocabulary shards)."""
        c, be, tpf, H = self.cfg, self.be, self.tpf, self.cfg.hidden_size
        if ctx.decode_only_full_logits:
            n = T
            logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
            tpf.gemm_gather(T, self.w["lm_head"], logits)
        else:
            n = ctx.num_logits
            last = tpf.gather_rows(T, ctx.logits_indices[:n], self.bufs.get("last", n, H))
            logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
            be.gemm(last, self.w["lm_head"], out=logits, out_dtype=torch.float32)
        return self._tp_logits_tail(ctx, logits, n)

    def _tp_logits_tail(self, ctx: StepContext, logits: torch.Tensor, n: int):
        """This rank's vocabulary shard of the logits -> argmax ids (greedy steps) or full logits."""
        c = self.cfg
        greedy_out = ctx.extra.get("greedy_out")
        if greedy_out is not None and c.final_logit_softcap <= 0:
            # Vocabulary-parallel greedy sampling: every rank reduces its shard to one candidate
            # per row and only those 8-byte pairs cross the link, not [n, vocab] fp32 logits
            # (a positive logits scale does not change the argmax).
            from .. import ops
            cand = self.bufs.get("argmax_cand", n, 2, torch.int32)
            valid = max(0, min(self.vocab_shard, c.vocab_size - self.vocab_start))
            ops.argmax_candidates(logits, valid, self.vocab_start, cand)
            allc = self.comm.all_gather(cand, dim=0)
            ops.argmax_combine(allc, n, self.tp, c.vocab_size, greedy_out[:n])
            return None
        logits = self.comm.all_gather(logits, dim=-1)
        if logits.shape[1] != c.vocab_size:
            logits = logits[:, : c.vocab_size]
        if c.logits_scaling != 1.0:
            logits = logits / c.logits_scaling
        if c.final_logit_softcap > 0:
            logits = c.final_logit_softcap * torch.tanh(logits / c.final_logit_softcap)
        return logits

    # ------------------------------------------------------------------ native layer entry
    def _native_layers_ok(self) -> bool:
        """The plain pre-norm configuration on one GPU: its blocks run through the native
        per-layer entry (one call per layer instead of ~10 launches sequenced from Python)."""
        c = self.cfg
        if self.device.type != "cuda" or self.tp > 1 or type(self).forward is not DenseModel.forward:
            return False
        if os.environ.get("B200_NATIVE_LAYERS", "1") == "0":      # debugging: keep the per-op path
            return False
        if (c.post_norm or c.sandwich_norm or c.attention_bias or c.mlp_bias or c.sliding_window
                or c.attention_chunk_size or c.residual_multiplier != 1.0 or len(set(self.layer_group)) != 1):
            return False
        from .backend import Fp8Weight, QuantWeight
        if any(isinstance(v, QuantWeight) for L in self.layers for v in L.values()):
            return False
        # fp8: the native block takes all four projections in e4m3 with per-channel scales and
        # quantises the activations per token; anything else (static scales, a mix) keeps the per-op path
        n8 = [sum(isinstance(L.get(k), Fp8Weight) and L[k].input_scale is None and L[k].w_scale.numel() > 1
                  for k in ("qkv", "o", "gate_up", "down")) for L in self.layers]
        return all(n == 0 for n in n8) or all(n == 4 for n in n8)

    def _native_weights(self):
        ws = getattr(self, "_native_w", None)
        if ws is None or len(ws) != len(self.layers) or ws[0].kv_cache != self.kv_caches[0].data_ptr() \
                or ws[0].qkv != self.layers[0]["qkv"].data_ptr():
            from ..ops.layer import DenseLayerWeights
            ws = []
            for l, L in enumerate(self.layers):
                w = DenseLayerWeights()
                w.ln1, w.qkv, w.o, w.ln2 = L["ln1"].data_ptr(), L["qkv"].data_ptr(), L["o"].data_ptr(), L["ln2"].data_ptr()
                w.q_norm = L["q_norm"].data_ptr() if L.get("q_norm") is not None else None
                w.k_norm = L["k_norm"].data_ptr() if L.get("k_norm") is not None else None
                w.gate_up, w.down = L["gate_up"].data_ptr(), L["down"].data_ptr()
                w.kv_cache = self.kv_caches[l].data_ptr()
                if hasattr(L["qkv"], "w8"):
                    w.fp8 = 1
                    w.qkv_scale, w.o_scale = L["qkv"].w_scale.data_ptr(), L["o"].w_scale.data_ptr()
                    w.gate_up_scale, w.down_scale = L["gate_up"].w_scale.data_ptr(), L["down"].w_scale.data_ptr()
                ws.append(w)
            self._native_w = ws
        return ws

    def _native_step(self, ctx, T, qkv, attn, gate_up, act, act_kind, hidden=None, resid=None, normed=None):
        """The shapes, step metadata and activation buffers of one forward as the native layer
        entries take them; None when this step needs the per-op path (split-KV buffers absent)."""
        from .. import ops
        from ..ops.layer import DenseStep
        c = self.cfg
        grp = self.layer_group[0]
        G = self.hq // self.hkv
        nd = ctx.num_decodes
        splits, tmp = ctx.decode_splits, ctx.extra.get("decode_tmp")
        use_tc = ops._decode_uses_tc(self.D, G, self.block_size)
        bt = ctx.block_table[grp]
        if nd > 0 and splits <= 0:
            splits = ops.attn_decode_splits(nd, self.hkv, G, self.D, bt.shape[1] * self.block_size,
                                            self.block_size if use_tc else 0)
        if nd > 0 and splits > 1 and tmp is None:
            return None                       # the per-op path allocates the split buffers
        s = DenseStep()
        s.T, s.H, s.Hq, s.Hkv, s.D, s.rot, s.inter, s.block_size = (T, c.hidden_size, self.hq, self.hkv, self.D,
                                                                  self.rot, self.inter, self.block_size)
        s.neox, s.gemma, s.act_kind, s.gate_up_interleaved = int(c.rope.neox), int(c.gemma_norm), act_kind, \
            int(self.gate_up_il)
        s.eps, s.scale, s.softcap, s.window = c.rms_norm_eps, self.scale, c.attn_logit_softcap or 0.0, 0
        s.num_blocks = self.kv_caches[0].shape[0]
        s.positions, s.cos_sin = ctx.positions.data_ptr(), self.rope_table.data_ptr()
        s.slot_mapping = ctx.slot_mapping[grp].data_ptr()
        s.block_table, s.max_blocks, s.seq_lens = bt.data_ptr(), bt.stride(0), ctx.seq_lens.data_ptr()
        s.num_decodes, s.decode_splits, s.decode_tc = nd, max(1, splits), int(use_tc)
        if tmp is not None:
            s.decode_tmp_o, s.decode_tmp_lse = tmp[0].data_ptr(), tmp[1].data_ptr()
        s.num_prefills, s.num_tiles, s.num_prefill_tokens = ctx.num_prefills, ctx.num_tiles, T - nd
        if ctx.num_prefills > 0:
            s.prefill_q_start, s.tile_req, s.tile_q0 = (ctx.prefill_q_start.data_ptr(), ctx.tile_req.data_ptr(),
                                                        ctx.tile_q0.data_ptr())
        if hidden is not None:
            s.hidden, s.resid, s.normed = hidden.data_ptr(), resid.data_ptr(), normed.data_ptr()
        s.qkv_buf, s.attn, s.gate_up_buf, s.act = qkv.data_ptr(), attn.data_ptr(), gate_up.data_ptr(), act.data_ptr()
        ws = ops.workspace(self.device, ops.GEMM_WS_BYTES)
        s.gemm_ws, s.gemm_ws_bytes = ws.data_ptr(), ws.numel()
        if hasattr(self.layers[0]["qkv"], "w8"):
            widest = max(c.hidden_size, self.hq * self.D, self.inter)
            s.fp8_act = ops.workspace(self.device, T * widest, "fp8_act").data_ptr()
            s.fp8_scales = ops.workspace(self.device, T * 4, "fp8_row_scales").data_ptr()
        return s

    def _run_native_layers(self, ctx, T, hidden, resid, normed, qkv, attn, gate_up, act, act_kind) -> bool:
        from ..ops.layer import dense_layer
        s = self._native_step(ctx, T, qkv, attn, gate_up, act, act_kind, hidden, resid, normed)
        if s is None:
            return False
        for l, w in enumerate(self._native_weights()):
            s.first_layer = int(l == 0)
            dense_layer(w, s)
        return True

    def _native_tp_ok(self) -> bool:
        """The fused tensor-parallel stack has a native entry for the plain pre-norm block with one
        KV-cache group (the same configurations as the one-GPU native entry)."""
        c = self.cfg
        if os.environ.get("B200_NATIVE_LAYERS", "1") == "0" or type(self)._forward_tp_fused is not \
                DenseModel._forward_tp_fused:
            return False
        return not (c.mlp_bias or c.sliding_window or c.attention_chunk_size
                    or len(set(self.layer_group)) != 1)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Returns fp32 logits ``[num_logits, vocab]`` for the rows in ``ctx.logits_indices``."""
        if getattr(self, "tpf", None) is not None:
            return self._forward_tp_fused(ctx)
        c, be, T = self.cfg, self.be, ctx.num_tokens
        H = c.hidden_size
        eps = c.rms_norm_eps
        act_kind = ACT_KIND.get(c.hidden_act, 0)
        hidden = self.bufs.get("hidden", T, H)
        resid = self.bufs.get("resid", T, H)
        normed = self.bufs.get("normed", T, H)
        qkv = self.bufs.get("qkv", T, (self.hq + 2 * self.hkv) * self.D)
        attn = self.bufs.get("attn", T, self.hq * self.D)
        gate_up = self.bufs.get("gate_up", T, 2 * self.inter)
        act = self.bufs.get("act", T, self.inter)

        be_emb = be.embedding(ctx.input_ids[:T], self.w["embed"], out=hidden,
                              vocab_start=self.vocab_start, vocab_total=c.vocab_size,
                              scale=c.embed_scale)
        if be_emb is not hidden:
            hidden.copy_(be_emb)
        if self.tp > 1:
            self.comm.all_reduce(hidden)
        pos = ctx.positions[:T]
        first = True
        layers = self.layers
        if self.native_layers is None:
            self.native_layers = self._native_layers_ok()
        if self.native_layers and T > 0 and not nvtx.ENABLED and \
                self._run_native_layers(ctx, T, hidden, resid, normed, qkv, attn, gate_up, act, act_kind):
            layers = []                        # every block already ran
        for l, L in enumerate(layers):
            if nvtx.ENABLED:          # one flat marker per layer (ranges would need a pop at every exit)
                torch.cuda.nvtx.mark(f"layer {l}")
            grp = self.layer_group[l]
            window = self._layer_window(l)
            # ---- attention block
            if c.post_norm:
                if first:
                    resid.copy_(hidden)
                be.gemm(resid, L["qkv"], bias=L.get("qkv_bias"), out=qkv)
            else:
                if first:
                    resid.copy_(hidden)
                # the norm hands its rows to the projection (as quantised activations when the
                # weights take them)
                be.norm_gemm(hidden, L["ln1"], eps, L["qkv"], qkv, residual=None if first else resid,
                             gemma=c.gemma_norm, normed=normed, bias=L.get("qkv_bias"))
            first = False
            be.rope_kv(qkv, pos, self.rope_table, num_q_heads=self.hq, num_kv_heads=self.hkv,
                       head_dim=self.D, rot_dim=self.rot, neox=c.rope.neox,
                       q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), eps=eps,
                       gemma=c.gemma_norm, slot_mapping=ctx.slot_mapping[grp][:T],
                       kv_cache=self.kv_caches[l], block_size=self.block_size)
            be.attention(qkv[:, : self.hq * self.D], self.kv_caches[l], ctx, grp,
                         num_q_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.D,
                         block_size=self.block_size, scale=self.scale, out=attn,
                         softcap=c.attn_logit_softcap, window=window)
            be.gemm(attn, L["o"], out=hidden)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
            if c.post_norm:
                # OLMo-2: stream = stream + norm(attn(stream)); the stream lives in `resid`
                t = be.rmsnorm(hidden, L["ln2"], eps, out=normed)
                x_mlp = self._add_into(resid, t)
            else:
                if c.sandwich_norm:
                    hidden = be.rmsnorm(hidden, L["ln2"], eps, out=hidden, gemma=c.gemma_norm)
                    x_mlp = be.rmsnorm(hidden, L["ln_pre_ff"], eps, residual=resid, out=normed,
                                       gemma=c.gemma_norm)
                else:
                    if c.residual_multiplier != 1.0:
                        hidden = be.mul_scalar(hidden, c.residual_multiplier)
                    x_mlp = None           # ln2 runs with the gate / up projection below
            # ---- MLP block
            plain_w = isinstance(L["gate_up"], torch.Tensor)
            if x_mlp is None and (plain_w and self.gate_up_il):
                x_mlp = be.rmsnorm(hidden, L["ln2"], eps, residual=resid, out=normed, gemma=c.gemma_norm)
            if x_mlp is None:
                be.norm_gemm(hidden, L["ln2"], eps, L["gate_up"], gate_up, residual=resid, gemma=c.gemma_norm,
                             normed=normed)
                hidden = self.bufs.get("hidden", T, H)
                be.act_gemm(gate_up, act_kind, L["down"], hidden, act=act, interleaved=self.gate_up_il)
            else:
                if self.gate_up_il:
                    a = be.gemm_gated(x_mlp, L["gate_up"], act_kind, out=act, scratch=gate_up)
                else:
                    be.gemm(x_mlp, L["gate_up"], out=gate_up)
                    a = be.act_and_mul(gate_up, act_kind, out=act)
                hidden = self.bufs.get("hidden", T, H)
                be.gemm(a, L["down"], out=hidden)
            if self.tp > 1:
                self.comm.all_reduce(hidden)
            if c.post_norm:
                t = be.rmsnorm(hidden, L["ln_post_ff"] if "ln_post_ff" in L else L["ln1"], eps,
                               out=normed)
                self._add_into(resid, t)
            elif c.sandwich_norm:
                hidden = be.rmsnorm(hidden, L["ln_post_ff"], eps, out=hidden, gemma=c.gemma_norm)
            elif c.residual_multiplier != 1.0:
                hidden = be.mul_scalar(hidden, c.residual_multiplier)
        # ---- final norm on the rows that sample, lm_head
        if c.post_norm:
            final_in, res = resid, None
        else:
            final_in, res = hidden, resid
        if ctx.decode_only_full_logits:
            n = T
            last = be.rmsnorm(final_in, self.w["final_norm"], eps, residual=res, out=normed,
                              gemma=c.gemma_norm)
        else:
            n = ctx.num_logits
            full = be.rmsnorm(final_in, self.w["final_norm"], eps, residual=res, out=normed,
                              gemma=c.gemma_norm)
            last = be.gather_rows(full, ctx.logits_indices[:n], out=self.bufs.get("last", n, H))
        logits = self.bufs.get("logits", n, self.vocab_shard, torch.float32)
        be.gemm(last, self.w["lm_head"], out=logits, out_dtype=torch.float32)
        if self.tp > 1:
            logits = self.comm.all_gather(logits, dim=-1)
        if logits.shape[1] != c.vocab_size:
            logits = logits[:, : c.vocab_size]
        if c.logits_scaling != 1.0:
            logits = logits / c.logits_scaling
        if c.final_logit_softcap > 0:
            logits = c.final_logit_softcap * torch.tanh(logits / c.final_logit_softcap)
        return logits

    def _add_into(self, resid, t):
        """Post-norm residual: resid += t; returns the stream."""
        resid.copy_(self.be.add(resid, t))
        return resid
