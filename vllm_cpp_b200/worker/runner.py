"""Model runner: turns a SchedulerOutput into one packed host->device copy, a forward pass
(CUDA graph replay for decode-only batches) and sampled token ids.

The step loop, the scheduler and the input preparation (``InputBatch.prepare``) are C++;
this class owns the device side: KV-cache tensors, the packed step buffer (pinned host +
device copy), CUDA graphs keyed by padded decode batch size, and the sampler pipeline.

Reference: ``src/vllm/v1/worker/gpu/runner.cpp:373`` (initialize_kv_cache), ``:669-880``
(execute_model), ``:1051`` (sample_tokens), ``:1164`` (sample_tokens_async), decode graphs
``qwen3_5.cpp:5898-5960`` and ``include/vllm/model_executor/models/decode_graph_sizes.h``.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..utils import nvtx

from .. import _engine as E
from ..models.base import StepContext

_DT = {"input_ids": (torch.int64, 8), "positions": (torch.int64, 8), "slot_mapping": (torch.int64, 8),
       "query_start": (torch.int32, 4), "seq_lens": (torch.int32, 4), "block_table": (torch.int32, 4),
       "logits_indices": (torch.int32, 4), "tile_req": (torch.int32, 4), "tile_q0": (torch.int32, 4),
       "prefill_q_start": (torch.int32, 4), "state_slots": (torch.int32, 4),
       "temperature": (torch.float32, 4), "top_p": (torch.float32, 4), "min_p": (torch.float32, 4),
       "top_k": (torch.int32, 4), "seeds": (torch.int64, 8), "steps": (torch.int64, 8),
       "rep_pen": (torch.float32, 4), "freq_pen": (torch.float32, 4), "pres_pen": (torch.float32, 4),
       "splice_dst": (torch.int32, 4), "splice_src": (torch.int32, 4),
       "sample_rows": (torch.int32, 4)}


# StepInfo fields a rank needs to run a step it did not prepare itself
STEP_INFO_FIELDS = ("num_reqs", "num_tokens", "num_decodes", "num_prefills", "num_prefill_tokens",
                    "num_tiles", "max_query_len", "max_seq_len", "num_logits", "num_splice", "all_greedy",
                    "any_penalties", "any_top_k_top_p", "any_min_p", "any_logprobs", "any_logit_edits",
                    "req_ids", "produces_token", "max_logprobs", "num_draft", "logits_row0")


def _plain(v):
    return list(v) if isinstance(v, (list, tuple)) else v


def decode_graph_sizes(max_num_seqs: int) -> list[int]:
    """Padded decode batch sizes that get a captured graph: 1,2,4,8,16,24,...,max."""
    sizes = [s for s in (1, 2, 4, 8) if s <= max_num_seqs]
    s = 16
    while s < max_num_seqs:
        sizes.append(s)
        s += 8 if s < 64 else (16 if s < 256 else 32)
    if max_num_seqs not in sizes:
        sizes.append(max_num_seqs)
    return sorted(set(sizes))


class ModelRunner(E.ModelRunnerBase):
    def __init__(self, model, *, block_size: int, num_blocks: int, max_num_seqs: int,
                 max_num_batched_tokens: int, max_model_len: int, enable_cuda_graphs: bool = True,
                 async_mode: bool = False, speculative_config=None, step_channel=None):
        super().__init__()
        # Multi-rank serving: the rank that owns the scheduler publishes every step (the packed
        # step buffer and what the sampler needs) on this channel; the other ranks run
        # ``serve_steps`` and never see a request. None: this rank schedules for itself.
        self.step_channel = step_channel
        # Speculative decoding, n-gram (prompt lookup) drafts verified by argmax comparison:
        # a request scheduled with k drafts runs k + 1 query tokens, gets k + 1 logits rows and
        # keeps the longest prefix of drafts that the target agrees with plus one more token.
        # "mtp": the drafts come from the model's multi-token-prediction head instead
        # (models/gdn_mtp.py); "draft_model": from a second, smaller model (models/draft.py). Both
        # are verified the same way.
        self.spec = speculative_config if (speculative_config is not None and
                                           speculative_config.method in ("ngram", "mtp", "draft_model")) else None
        self.max_spec = self.spec.num_speculative_tokens if self.spec else 0
        self.mtp = None
        self.drafter = None                              # a separate draft model (models/draft.py)
        self.mtp_proposed: dict[str, list[int]] = {}     # every draft the head proposed, per request
        self._last_ctx = None
        self._drafts: dict[str, list[int]] = {}
        self._scheduled_spec: dict[str, list[int]] = {}
        self.spec_stats = {"drafted": 0, "accepted": 0}
        self.model = model
        self.device = model.device
        self.is_cuda = self.device.type == "cuda"
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max(max_num_batched_tokens, max_num_seqs)
        self.max_model_len = max_model_len
        self.async_mode = async_mode
        self.groups = model.kv_cache_groups(block_size)
        self.num_groups = len(self.groups)
        self.max_blocks = (max_model_len + block_size - 1) // block_size + 1
        self.layout = E.StepLayout.make(self.max_tokens, max_num_seqs, self.max_blocks,
                                        self.num_groups, self.max_spec)
        self.off = self.layout.offsets()
        nbytes = self.layout.total_bytes
        # two pinned staging buffers: with a step in flight its copy may not have run yet when
        # the next step is prepared
        self.host_bufs = [torch.zeros(nbytes, dtype=torch.uint8, pin_memory=self.is_cuda)
                          for _ in range(2 if async_mode else 1)]
        self.host_buf = self.host_bufs[0]
        self._step_no = 0
        self.dev_buf = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self.batch = E.InputBatch(max_num_seqs, max_model_len, self.max_tokens,
                                  [g[1]["block_size"] for g in self.groups])
        model.alloc_kv_cache(num_blocks, block_size)
        model.reserve_buffers(self.max_tokens, max_num_seqs)
        if getattr(model, "fused_tp_supported", None) and model.fused_tp_supported():
            model.enable_fused_tp(self.max_tokens)
        self.views = self._make_views(self.dev_buf)
        self.host_views_all = [self._make_views(b) for b in self.host_bufs]
        self.host_views = self.host_views_all[0]
        max_logits = self.layout.max_logits
        self.sampled = torch.zeros(max_logits, dtype=torch.int64, device=self.device)
        self.sampled_host = torch.zeros(max_logits, dtype=torch.int64,
                                        pin_memory=self.is_cuda)
        self.last_sampled = torch.zeros(max_num_seqs, dtype=torch.int64, device=self.device)
        self.graphs: dict[int, tuple] = {}
        self._model_samples_greedy = bool(getattr(model, "samples_greedy", False))
        self.enable_graphs = enable_cuda_graphs and self.is_cuda
        self.graph_sizes = decode_graph_sizes(max_num_seqs) if self.enable_graphs else []
        self._info = None
        self._logits = None
        self._eos: dict[str, int] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.num_kernel_steps = 0
        self.launches = 0
        self.time_steps = False          # record CUDA events around each step's GPU work
        self.step_events: list = []
        if self.is_cuda:
            from .. import ops
            self.ops = ops
            self.copy_stream = torch.cuda.Stream(device=self.device)
            # the kernels' status word rides on every step's device->host copy of the sampled ids
            from ..ops import _lib
            self._status_dev = _lib.status_word(self.device)
            self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            Hq, Hkv, D = model.hq, model.hkv, model.D
            self._decode_tmp: dict[int, tuple] = {}
            self._Hq, self._Hkv, self._D = Hq, Hkv, D

    # ------------------------------------------------------------------ helpers
    def _make_views(self, buf: torch.Tensor) -> dict:
        L, o = self.layout, self.off
        v = {}

        def view(name, count):
            dt, sz = _DT[name]
            return buf[o[name]: o[name] + count * sz].view(dt)

        T, R, B, G = L.max_tokens, L.max_reqs, L.max_blocks, L.num_groups
        v["input_ids"] = view("input_ids", T)
        v["positions"] = view("positions", T)
        sm = view("slot_mapping", T * G).view(G, T)
        v["slot_mapping"] = [sm[g] for g in range(G)]
        v["query_start"] = view("query_start", R + 1)
        v["seq_lens"] = view("seq_lens", R)
        bt = view("block_table", G * R * B).view(G, R, B)
        v["block_table"] = [bt[g] for g in range(G)]
        v["logits_indices"] = view("logits_indices", L.max_logits)
        v["tile_req"] = view("tile_req", L.max_tiles)
        v["tile_q0"] = view("tile_q0", L.max_tiles)
        v["prefill_q_start"] = view("prefill_q_start", R + 1)
        v["state_slots"] = view("state_slots", R)
        for k in ("temperature", "top_p", "min_p", "top_k", "seeds", "steps", "rep_pen", "freq_pen",
                  "pres_pen", "splice_dst", "splice_src"):
            v[k] = view(k, R)
        v["sample_rows"] = view("sample_rows", L.max_logits)
        return v

    def kv_cache_config(self) -> "E.KVCacheConfig":
        groups = []
        for layers, spec in self.groups:
            kind = {"full": E.KVSpecKind.FULL_ATTENTION, "sliding": E.KVSpecKind.SLIDING_WINDOW,
                    "mla": E.KVSpecKind.MLA, "mamba": E.KVSpecKind.MAMBA,
                    "chunked": E.KVSpecKind.CHUNKED_LOCAL}[spec["kind"]]
            kw = {k: v for k, v in spec.items() if k != "kind"}
            groups.append(E.KVCacheGroupSpec([f"layers.{l}" for l in layers],
                                             E.KVCacheSpec(kind=kind, **kw)))
        return E.KVCacheConfig(self.num_blocks, groups)

    def set_eos(self, req_id: str, eos: Optional[int]) -> None:
        self._eos[req_id] = -1 if eos is None else int(eos)

    def take_draft_token_ids(self):
        """Drafts proposed after the last sampling step (consumed by the scheduler)."""
        if not self._drafts:
            return None
        d = E.DraftTokenIds()
        d.req_ids = list(self._drafts.keys())
        d.draft_token_ids = [self._drafts[r] for r in d.req_ids]
        self._drafts = {}
        return d

    def supports_async(self) -> bool:
        if self.spec is not None:
            return False        # draft verification reads the sampled ids on the host every step
        return self.is_cuda

    def _decode_splits(self, batch: int) -> tuple[int, tuple | None]:
        if not self.is_cuda:
            return 1, None
        key = batch
        if key not in self._decode_tmp:
            s = self.ops.attn_decode_splits(batch, self._Hkv, self._Hq // self._Hkv, self._D,
                                            self.max_model_len, self.block_size)
            tmp = None
            if s > 1:
                tmp = (torch.empty((batch, self._Hq, s, self._D), dtype=torch.float32,
                                   device=self.device),
                       torch.empty((batch, self._Hq, s), dtype=torch.float32, device=self.device))
            self._decode_tmp[key] = (s, tmp)
        return self._decode_tmp[key]

    def _context(self, info, padded: int | None = None) -> StepContext:
        v = self.views
        T = padded if padded is not None else info.num_tokens
        nd = padded if padded is not None else info.num_decodes
        splits, tmp = self._decode_splits(nd) if nd > 0 else (1, None)
        ctx = StepContext(
            num_tokens=T, num_reqs=padded if padded is not None else info.num_reqs,
            num_decodes=nd, num_prefills=0 if padded is not None else info.num_prefills,
            num_prefill_tokens=0 if padded is not None else info.num_prefill_tokens,
            num_tiles=0 if padded is not None else info.num_tiles,
            num_logits=T if padded is not None else info.num_logits,
            input_ids=v["input_ids"], positions=v["positions"], slot_mapping=v["slot_mapping"],
            query_start=v["query_start"], seq_lens=v["seq_lens"], block_table=v["block_table"],
            logits_indices=v["logits_indices"], tile_req=v["tile_req"], tile_q0=v["tile_q0"],
            prefill_q_start=v["prefill_q_start"], state_slots=v["state_slots"],
            decode_splits=splits, max_seq_len=info.max_seq_len if info else 0,
            max_query_len=info.max_query_len if info else 1,
            decode_only_full_logits=padded is not None)
        ctx.extra["decode_tmp"] = tmp
        if padded is None:
            ctx.extra["host"] = self.host_views   # this step's pinned host copies
        if not self.is_cuda:
            # CPU oracle path wants exact-length views
            R = ctx.num_reqs
            ctx.query_start = v["query_start"][: R + 1]
            ctx.seq_lens = v["seq_lens"][:R]
            ctx.block_table = [b[:R] for b in v["block_table"]]
        return ctx

    # ------------------------------------------------------------------ CUDA graphs
    def _pad_size(self, n: int) -> int | None:
        for s in self.graph_sizes:
            if s >= n:
                return s
        return None

    def _capture(self, size: int):
        """Capture forward + greedy argmax for a decode-only batch padded to ``size`` rows."""
        info_stub = type("S", (), {"max_seq_len": 0, "max_query_len": 1})()
        ctx = self._context(info_stub, padded=size)
        # The warm-up runs below execute the model for real, so they must not see a live step's
        # inputs: KV writes would be harmless repeats, but a recurrent layer would advance the
        # state of live requests once per warm-up run. Every row becomes a pad row first (no KV
        # slot, no state slot, empty context); the caller copies the step's inputs in afterwards.
        v = self.views
        for k in ("input_ids", "positions", "seq_lens"):
            v[k].zero_()
        v["state_slots"].fill_(-1)
        for g_ in range(self.num_groups):
            v["slot_mapping"][g_].fill_(-1)
        # warm-up run on a side stream (allocations, tensor maps, lazy module state)
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        if self._model_samples_greedy:
            ctx.extra["greedy_out"] = self.sampled
        with torch.cuda.stream(s):
            for _ in range(2):
                logits = self.model.forward(ctx)
                if logits is not None:
                    self.ops.argmax(logits, out=self.sampled[:size])
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        from ..ops import _lib
        g = torch.cuda.CUDAGraph()
        n0 = _lib.LAUNCHES[0]
        with torch.cuda.graph(g):
            logits = self.model.forward(ctx)
            if logits is not None:
                self.ops.argmax(logits, out=self.sampled[:size])
        self.graphs[size] = (g, logits, _lib.LAUNCHES[0] - n0)
        return self.graphs[size]

    def warmup_graphs(self, sizes: list[int] | None = None) -> None:
        """Capture the decode graphs up front (pad rows: slot -1, seq_len 0, token 0)."""
        if not self.enable_graphs:
            return
        hv = self.host_views
        for k in ("input_ids", "positions", "seq_lens"):
            hv[k].zero_()
        hv["state_slots"].fill_(-1)
        for g in range(self.num_groups):
            hv["slot_mapping"][g].fill_(-1)
            hv["block_table"][g].zero_()
        self.dev_buf.copy_(self.host_buf, non_blocking=True)
        for s in (sizes or self.graph_sizes):
            if s not in self.graphs:
                self._capture(s)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ step
    offload = None   # KVOffloadWorker when KV offloading is configured

    def execute_model(self, so) -> None:
        self.batch.update_states(so)
        if self.offload is not None:
            self.offload.run_step_plan()
        if so.total_num_scheduled_tokens == 0:
            self._info = None
            return
        self._step_no += 1
        k = self._step_no % len(self.host_bufs)
        self.host_buf, self.host_views = self.host_bufs[k], self.host_views_all[k]
        info = self.batch.prepare(so, self.layout, self.host_buf.data_ptr(), self.async_mode)
        self._info = info
        self._scheduled_spec = dict(so.scheduled_spec_decode_tokens) if self.spec else {}
        R, T = info.num_reqs, info.num_tokens
        decode_only = info.num_prefills == 0 and info.num_decodes == R
        # plain greedy step: nothing edits the logits, the sampled id is the row's argmax
        plain_greedy = (info.all_greedy and not info.any_penalties and not info.any_logprobs
                        and not info.any_logit_edits and not so.structured_output_request_ids
                        and self.spec is None)
        pad = self._pad_size(R) if (decode_only and self.enable_graphs and plain_greedy) else None
        if pad is not None and pad > R:
            hv = self.host_views
            hv["input_ids"][R:pad].zero_()
            hv["positions"][R:pad].zero_()
            hv["seq_lens"][R:pad].zero_()
            hv["state_slots"][R:pad].fill_(-1)     # a stale slot here would update a live request's state
            for g in range(self.num_groups):
                hv["slot_mapping"][g][R:pad].fill_(-1)
        if self.step_channel is not None:
            # the other ranks run this step from the same packed buffer; they never see requests
            self.step_channel.broadcast_object(
                {"kind": "step", "pad": pad, "plain": plain_greedy,
                 "info": {f: _plain(getattr(info, f)) for f in STEP_INFO_FIELDS},
                 "buf": self.host_buf.numpy().tobytes()})
        if self.spec is not None and hasattr(self.model, "snapshot_state"):
            # requests that verify drafts in this step: their recurrent state is saved first
            slots = [int(self.host_views["state_slots"][r]) for r in range(R) if info.num_draft[r] > 0]
            self.model.snapshot_state(slots)
        self._launch_step(info, pad, plain_greedy)

    def _launch_step(self, info, pad, plain_greedy) -> None:
        """Host->device copy of the packed step buffer, forward pass (graph replay for padded
        decode-only batches). Runs on every rank; ``info`` is the StepInfo or its plain copy."""
        R, T = info.num_reqs, info.num_tokens
        self._step_plain = plain_greedy
        # one packed host->device copy per step
        if self.time_steps and self.is_cuda:
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
            self.step_events.append([e0, None])
        nbytes = self.layout.total_bytes
        if pad is not None and pad not in self.graphs:
            self._capture(pad)                 # before this step's inputs reach the device buffer
        if self.is_cuda:
            self.dev_buf.copy_(self.host_buf, non_blocking=True)
        else:
            self.dev_buf.copy_(self.host_buf)
        self.h2d_bytes += nbytes
        if info.num_splice and self.is_cuda:
            v = self.views
            from ..ops import _lib
            _lib.check(_lib.lib().b200_splice_sampled(
                v["input_ids"].data_ptr(), v["splice_dst"].data_ptr(), v["splice_src"].data_ptr(),
                self.last_sampled.data_ptr(), info.num_splice, _lib.stream_ptr()), "splice")
        if pad is not None:
            g = self.graphs[pad]
            g[0].replay()
            from ..ops import _lib as _l
            if _l.SYNC_CHECK:
                _l.sync_check(f"graph replay, padded batch {pad}, {R} requests")
            _l.LAUNCHES[0] += g[2]  # launcher calls folded into the replayed graph
            self._logits = g[1][:R] if g[1] is not None else None
            self._graph_sampled = True
        else:
            ctx = self._context(info)
            self._last_ctx = ctx
            if plain_greedy and self._model_samples_greedy:
                # the model writes the argmax ids itself (tensor parallel: candidates per vocabulary
                # shard are exchanged instead of the logits)
                ctx.extra["greedy_out"] = self.sampled
            with nvtx.range(f"forward T={T} R={R}"):
                self._logits = self.model.forward(ctx)
            self._graph_sampled = self._logits is None
        self.num_kernel_steps += 1
        if getattr(self.model, "eplb", None) is not None:
            self.model.eplb_end_step()         # closes the load window of the step; rebalances on schedule

    def _sample_device(self, info, grammar) -> torch.Tensor:
        """Runs the sampler pipeline on the logits of this step; returns int64 ids [num_logits]."""
        n = info.num_logits
        logits = self._logits
        v = self.views
        if self._graph_sampled:
            return self.sampled[:n]
        edits = self._pending_edits
        if edits is None:
            edits = self._host_sampler_edits(info, grammar)
            if self.step_channel is not None and not self._step_plain:
                self.step_channel.broadcast_object({"kind": "sample", "edits": edits})
        if not self.is_cuda:
            from ..sample import cpu_sampler
            return cpu_sampler.sample(self, info, self._logits, edits)
        ops = self.ops
        # row-compacted per-request scalars (rows that sample are a subset of the batch)
        rows = [i for i, p in enumerate(info.produces_token) if p]
        idx = None
        if n != info.num_reqs or len(rows) != info.num_reqs:
            # logits row -> batch row (a request verifying drafts owns several rows)
            idx = v["sample_rows"][:n].to(torch.int64)

        def per_row(name):
            t = v[name][: info.num_reqs]
            return t if idx is None else t[idx].contiguous()

        dev = self.device
        if edits.get("grammar"):
            row_ids, bitmask, words = edits["grammar"]
            mask = torch.tensor(bitmask, dtype=torch.int32, device=dev).view(len(row_ids), words)
            ops.apply_bitmask(logits, mask, torch.tensor(row_ids, dtype=torch.int32, device=dev))
        if edits.get("bias"):
            br, btk, bv = edits["bias"]
            ops.apply_logit_bias(logits, torch.tensor(br, dtype=torch.int32, device=dev),
                                 torch.tensor(btk, dtype=torch.int32, device=dev),
                                 torch.tensor(bv, dtype=torch.float32, device=dev))
        if edits.get("ban"):
            nr, nt = edits["ban"]
            ops.apply_token_mask(logits, torch.tensor(nr, dtype=torch.int32, device=dev),
                                 torch.tensor(nt, dtype=torch.int32, device=dev))
        if edits.get("penalties"):
            pr, pt, pc = edits["penalties"]
            ops.apply_penalties(logits, torch.tensor(pr, dtype=torch.int32, device=dev),
                                torch.tensor(pt, dtype=torch.int32, device=dev),
                                torch.tensor(pc, dtype=torch.int32, device=dev),
                                per_row("rep_pen"), per_row("freq_pen"), per_row("pres_pen"))
        greedy = ops.argmax(logits, out=self.sampled[:n])
        if info.all_greedy:
            return greedy
        temp = per_row("temperature")
        ops.apply_temperature(logits, temp)
        if info.any_min_p:
            ops.apply_min_p(logits, per_row("min_p"))
        if info.any_top_k_top_p:
            ops.apply_top_k_top_p(logits, per_row("top_k"), per_row("top_p"))
        probs = ops.softmax(logits)
        rnd = ops.random_sample(probs, per_row("seeds"), per_row("steps"))
        out = ops.merge_greedy_random(greedy.clone(), rnd, temp, out=self.sampled[:n])
        return out

    _pending_edits = None    # a worker rank: the sampler inputs the scheduling rank sent

    def _host_sampler_edits(self, info, grammar) -> dict:
        """Everything the sampler takes from host-side request state, as plain lists: grammar
        bitmask rows, logit bias, banned tokens, penalty counts. Computed on the rank that owns
        the requests; the other ranks receive it with the step."""
        edits: dict = {}
        rows = [i for i, p in enumerate(info.produces_token) if p]
        if grammar is not None and grammar.structured_output_request_ids:
            rid = {info.req_ids[j]: info.logits_row0[j] for j in rows}
            edits["grammar"] = ([rid.get(r, -1) for r in grammar.structured_output_request_ids],
                                list(grammar.bitmask), grammar.words_per_row)
        if info.any_logit_edits:
            br, btk, bv, nr, nt = self.batch.logit_edits(info, self._eos)
            if br:
                edits["bias"] = (list(br), list(btk), list(bv))
            if nr:
                edits["ban"] = (list(nr), list(nt))
        if info.any_penalties:
            pr, pt, pc = self.batch.penalty_entries(info)
            if pr:
                edits["penalties"] = (list(pr), list(pt), list(pc))
        return edits

    # ------------------------------------------------------------------ worker ranks
    def serve_steps(self) -> None:
        """Loop of a rank that owns no scheduler: run every step the scheduling rank publishes
        (same packed buffer, same sampler inputs, so every rank samples the same ids and keeps
        them on its device for the next step's input splice) until it says stop."""
        import types
        ch = self.step_channel
        try:
            while True:
                msg = ch.broadcast_object(None)
                if msg["kind"] == "stop":
                    return
                if msg["kind"] != "step":
                    raise RuntimeError(f"worker rank: unexpected message {msg['kind']!r}")
                info = types.SimpleNamespace(**msg["info"])
                self._step_no += 1
                k = self._step_no % len(self.host_bufs)
                self.host_buf, self.host_views = self.host_bufs[k], self.host_views_all[k]
                self.host_buf.numpy()[:] = np.frombuffer(msg["buf"], dtype=np.uint8)
                self._info = info
                self._launch_step(info, msg["pad"], msg["plain"])
                n = info.num_logits
                if n == 0:
                    continue
                if not msg["plain"]:
                    m2 = ch.broadcast_object(None)
                    if m2["kind"] != "sample":
                        raise RuntimeError("worker rank: expected the sampler inputs of the step")
                    self._pending_edits = m2["edits"]
                try:
                    ids = self._sample_device(info, None)
                finally:
                    self._pending_edits = None
                if self.async_mode and self.is_cuda:
                    from ..ops import _lib
                    ids = ids.clone()
                    _lib.check(_lib.lib().b200_scatter_sampled(
                        self.last_sampled.data_ptr(), self.views["sample_rows"].data_ptr(), ids.data_ptr(), n,
                        _lib.stream_ptr()), "scatter")
        except BaseException:
            if hasattr(ch, "abort"):
                ch.abort()          # the other ranks' next collective raises instead of waiting
            raise

    def stop_workers(self) -> None:
        if self.step_channel is not None:
            self.step_channel.broadcast_object({"kind": "stop"})

    def _logprobs_rows(self, info, ids: torch.Tensor):
        if not info.any_logprobs:
            return None
        lp = torch.log_softmax(self._raw_logits.float(), -1) if hasattr(self, "_raw_logits") else \
            torch.log_softmax(self._logits.float(), -1)
        out = []
        row = 0
        for r, p in enumerate(info.produces_token):
            if not p:
                out.append([])
                continue
            k = info.max_logprobs[r]
            if k < 0:
                out.append([])
            else:
                tok = int(ids[row])
                lr = E.LogprobsRow()
                vals, idxs = torch.topk(lp[row], k) if k > 0 else (torch.empty(0), torch.empty(0))
                lr.token_ids = [tok] + [int(i) for i in idxs]
                lr.logprobs = [float(lp[row, tok])] + [float(x) for x in vals]
                rank = int((lp[row] > lp[row, tok]).sum()) + 1
                lr.ranks = [rank] + list(range(1, k + 1))
                out.append([lr])
            row += 1 + info.num_draft[r]
        return out

    STATUS_NAMES = {1: "an mbarrier wait inside a kernel pipeline ran out",
                    2: "a wait on another GPU's progress ran out (a peer rank is late or gone)",
                    3: "a kernel rejected its arguments", 4: "misaligned shared memory"}

    def _check_status(self, value: int) -> None:
        """A kernel that gave up a bounded wait skipped its work: what was sampled in this step
        is not to be trusted and peers may be out of step. The engine stops serving."""
        if value != 0:
            raise E.EngineDeadError(f"GPU kernel status {value}: {self.STATUS_NAMES.get(value, 'unknown error')}; "
                                    "the step's output was discarded")

    def _mark_step_end(self) -> None:
        if self.time_steps and self.is_cuda and self.step_events and self.step_events[-1][1] is None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.step_events[-1][1] = e1

    def device_step_ms(self) -> float:
        """Sum of per-step device time (first copy to last sampling kernel) since the last call."""
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in self.step_events if b is not None)
        self.step_events = []
        return ms

    def _build_output(self, info, ids_host) -> "E.ModelRunnerOutput":
        out = E.ModelRunnerOutput()
        out.req_ids = list(info.req_ids)
        toks = []
        rollback: list = []
        recompute: dict = {}
        row = 0
        for r, p in enumerate(info.produces_token):
            if p:
                k = info.num_draft[r]
                rid = info.req_ids[r]
                if k:
                    # rows row .. row + k hold the target's choice after each draft prefix
                    drafts = self._scheduled_spec.get(rid, [])[:k]
                    acc = 0
                    while acc < k and acc < len(drafts) and int(ids_host[row + acc]) == drafts[acc]:
                        acc += 1
                    new = [int(ids_host[row + i]) for i in range(acc + 1)]
                    self.spec_stats["drafted"] += k
                    self.spec_stats["accepted"] += acc
                    if acc < k and hasattr(self.model, "restore_state"):
                        # the recurrent state has run past the kept tokens: back to the saved
                        # state, and the kept tokens of this step run again with the next one
                        rollback.append(int(self.host_views["state_slots"][r]))
                        recompute[rid] = acc + 1
                else:
                    new = [int(ids_host[row])]
                toks.append(new)
                self.batch.append_sampled(rid, new)
                row += k + 1
            else:
                toks.append([])
        out.sampled_token_ids = toks
        if rollback:
            self.model.restore_state(rollback)
            out.num_recompute = recompute          # (assigned whole: the binding copies containers)
        if self.mtp is not None:
            self._propose_mtp(info, toks)
        elif self.drafter is not None:
            self._propose_draft_model(info, toks)
        elif self.spec is not None:
            for r, p in enumerate(info.produces_token):
                rid = info.req_ids[r]
                if p:
                    # an entry for every request that sampled (empty = no drafts next step)
                    self._drafts[rid] = self.batch.propose_ngram(
                        rid, self.spec.prompt_lookup_min, self.spec.prompt_lookup_max,
                        self.max_spec) if self.batch.plain_greedy(rid) else []
        return out

    def attach_mtp(self, mtp) -> None:
        """The multi-token-prediction drafter of the model (its blocks get a KV cache over the same
        block numbers as the trunk's, and activation buffers of the step's size)."""
        mtp.alloc(self.num_blocks, self.block_size, self.max_tokens, self.max_num_seqs)
        mtp.bind_block_table(self.max_blocks)
        self.mtp = mtp

    def _propose_mtp(self, info, toks) -> None:
        """Runs the draft head over the rows of the step that just finished. ``toks``: per request
        the tokens it kept in this step (accepted drafts plus the trunk's own choice), empty for a
        request that only prefilled. Every row's "next token" is the following query token, and
        for the last row a request keeps, the token the trunk chose; rows past it are rejected
        drafts whose cache entries the next pass over those positions rewrites."""
        T, R = info.num_tokens, info.num_reqs
        hv = self.host_views
        ids = hv["input_ids"][:T]
        qs = hv["query_start"][: R + 1].tolist()
        nxt = torch.zeros(T, dtype=torch.int64)
        if T > 1:
            nxt[: T - 1] = ids[1:T]
        rows, rids = [], []
        for r in range(R):
            e = qs[r + 1]
            rid = info.req_ids[r]
            new = toks[r]
            if not new:
                # a prompt chunk that stops short of the prompt's end: the next prompt token is known
                pos = int(hv["positions"][e - 1])
                known = self.batch.token_ids(rid)
                nxt[e - 1] = known[pos + 1] if pos + 1 < len(known) else 0
                continue
            base = e - 1 - info.num_draft[r]         # row of the last token the request had
            for j, t in enumerate(new):
                nxt[base + j] = t
            if self.batch.plain_greedy(rid):
                rows.append(base + len(new) - 1)
                rids.append(rid)
            else:
                self._drafts[rid] = []
        m = self.mtp
        m.next_ids[:T].copy_(nxt)
        n = len(rows)
        if n:
            m.rows[:n].copy_(torch.tensor(rows, dtype=torch.int32))
        # the head runs even when no request wants a draft: its cache must cover every position
        logits = m.forward(self._last_ctx, m.next_ids, self.model.last_full, m.rows[:max(n, 1)])
        if not n:
            return
        draft = logits[:n].argmax(-1)
        chains = [[int(d)] for d in draft.tolist()]
        if self.max_spec > 1:
            self._extend_mtp_drafts(info, rows, rids, draft, chains)
        for rid, ch in zip(rids, chains):
            self._drafts[rid] = ch
            if len(self.mtp_proposed) > 256:          # a debugging aid, not a log: keep it small
                self.mtp_proposed.clear()
            self.mtp_proposed.setdefault(rid, []).extend(ch)

    def _extend_mtp_drafts(self, info, rows, rids, draft, chains) -> None:
        """Drafts two to k: the head continues from its own output. Step i feeds (the head's hidden
        state of step i - 1, draft i) at position p + i, one row per request, as a decode-only
        batch over the same block tables (the scheduler reserved those slots as look-ahead); the
        cache entries it writes there are replaced when the trunk reaches those positions."""
        m, hv, n = self.mtp, self.host_views, len(rows)
        R = info.num_reqs
        qs = hv["query_start"][: R + 1].tolist()
        req_of_row = {}
        for r in range(R):
            for row in range(qs[r], qs[r + 1]):
                req_of_row[row] = r
        reqs = [req_of_row[row] for row in rows]
        pos0 = torch.tensor([int(hv["positions"][row]) for row in rows], dtype=torch.int64)
        bt_host = torch.stack([hv["block_table"][0][r] for r in reqs], 0)          # [n, max_blocks]
        hidden = m.inner.last_full[torch.tensor(rows, dtype=torch.long, device=self.device)].clone()
        ids = draft.to(torch.int64)
        for i in range(1, self.max_spec):
            pos = pos0 + i
            if int(pos.max()) + 1 >= self.max_model_len:
                break
            m.next_ids[:n].copy_(ids)
            ctx = self._draft_decode_ctx(m, n, pos, bt_host)
            logits = m.forward(ctx, m.next_ids, hidden, m.rows[:n])
            ids = logits[:n].argmax(-1).to(torch.int64)
            for ch, d in zip(chains, ids.tolist()):
                ch.append(int(d))
            hidden = m.inner.last_full[:n].clone()

    def _draft_decode_ctx(self, m, n: int, pos: torch.Tensor, bt_host: torch.Tensor):
        """A decode-only step of ``n`` rows (one per request) at positions ``pos`` over the block
        tables ``bt_host`` [n, max_blocks], written into the drafter's own input buffers
        (``m.d_*``, ``m.next_ids`` already holds the token ids)."""
        from ..models.base import StepContext
        bs = self.block_size
        blk = torch.gather(bt_host.long(), 1, (pos // bs).unsqueeze(1)).squeeze(1)
        m.d_bt[:n].copy_(bt_host)
        m.d_qs[: n + 1].copy_(torch.arange(n + 1, dtype=torch.int32))
        m.rows[:n].copy_(torch.arange(n, dtype=torch.int32))
        m.d_pos[:n].copy_(pos)
        m.d_slots[:n].copy_(blk * bs + pos % bs)
        m.d_seq[:n].copy_((pos + 1).to(torch.int32))
        splits, tmp = self._decode_splits(n) if self.is_cuda else (1, None)
        ctx = StepContext(
            num_tokens=n, num_reqs=n, num_decodes=n, num_prefills=0, num_prefill_tokens=0, num_tiles=0,
            num_logits=n, input_ids=m.next_ids, positions=m.d_pos, slot_mapping=[m.d_slots],
            query_start=m.d_qs if self.is_cuda else m.d_qs[: n + 1],
            seq_lens=m.d_seq if self.is_cuda else m.d_seq[:n],
            block_table=[m.d_bt if self.is_cuda else m.d_bt[:n]], logits_indices=m.rows,
            tile_req=self.views["tile_req"], tile_q0=self.views["tile_q0"],
            prefill_q_start=self.views["prefill_q_start"], state_slots=self.views["state_slots"],
            decode_splits=splits, max_seq_len=int(pos.max()) + 1, max_query_len=1)
        ctx.extra["decode_tmp"] = tmp
        return ctx

    # ---- a separate draft model
    def attach_draft_model(self, drafter) -> None:
        """``drafter``: models/draft.py DraftModel. Its KV cache uses the target's block numbers."""
        if self.num_groups != 1:
            raise ValueError("draft-model speculation needs a target with one KV cache group")
        drafter.alloc(self.num_blocks, self.block_size, self.max_tokens, self.max_num_seqs, self.max_blocks)
        self.drafter = drafter

    def _propose_draft_model(self, info, toks) -> None:
        """After the target's step: the draft model runs the same rows (cache fill), then k
        decode-only passes from the token each request just got. ``toks`` as in _propose_mtp."""
        d, hv = self.drafter, self.host_views
        R = info.num_reqs
        d.fill(self._last_ctx)
        qs = hv["query_start"][: R + 1].tolist()
        reqs, rids, first, pos_last = [], [], [], []
        for r in range(R):
            new, rid = toks[r], info.req_ids[r]
            if not new:
                continue
            if not self.batch.plain_greedy(rid):
                self._drafts[rid] = []
                continue
            base = qs[r + 1] - 1 - info.num_draft[r]          # row of the last token the request had
            reqs.append(r)
            rids.append(rid)
            first.append(new[-1])
            pos_last.append(int(hv["positions"][base + len(new) - 1]))
        n = len(reqs)
        if not n:
            return
        bt_host = torch.stack([hv["block_table"][0][r] for r in reqs], 0)
        ids = torch.tensor(first, dtype=torch.int64)
        pos0 = torch.tensor(pos_last, dtype=torch.int64) + 1       # where the new token sits
        chains = [[] for _ in range(n)]
        for i in range(self.max_spec):
            pos = pos0 + i
            if int(pos.max()) + 1 >= self.max_model_len:
                break
            d.next_ids[:n].copy_(ids)
            logits = d.decode(self._draft_decode_ctx(d, n, pos, bt_host))
            ids = logits[:n].argmax(-1).to(torch.int64).cpu()
            for ch, t in zip(chains, ids.tolist()):
                ch.append(int(t))
        for rid, ch in zip(rids, chains):
            self._drafts[rid] = ch

    def sample_tokens(self, grammar) -> "E.ModelRunnerOutput":
        info = self._info
        n = info.num_logits
        if n == 0:
            return self._build_output(info, [])
        if info.any_logprobs:
            self._raw_logits = self._logits.clone()
        ids = self._sample_device(info, grammar)
        self._mark_step_end()
        if self.is_cuda:
            self.sampled_host[:n].copy_(ids[:n], non_blocking=True)
            self._status_host.copy_(self._status_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self._check_status(int(self._status_host[0]))
            host = self.sampled_host[:n].tolist()
            self.d2h_bytes += 4
        else:
            host = ids[:n].tolist()
        self.d2h_bytes += n * 8
        out = self._build_output(info, host)
        lps = self._logprobs_rows(info, host)
        if lps is not None:
            out.logprobs = lps
        return out

    def sample_tokens_async(self, grammar):
        """Sampled ids stay on the device for the next step's input splice; the returned
        handle blocks only on the copy-stream event of the device->host copy."""
        info = self._info
        n = info.num_logits
        if n == 0 or not self.is_cuda:
            out = self.sample_tokens(grammar)
            return lambda: out
        ids = self._sample_device(info, grammar).clone()  # the next step reuses the buffer
        self._mark_step_end()
        # scatter into the per-batch-row table read by the next step's splice kernel
        row_of = self.views["sample_rows"]
        from ..ops import _lib
        _lib.check(_lib.lib().b200_scatter_sampled(self.last_sampled.data_ptr(), row_of.data_ptr(),
                                                   ids.data_ptr(), n, _lib.stream_ptr()), "scatter")
        ev = torch.cuda.Event()
        host = torch.empty(n, dtype=torch.int64, pin_memory=True)
        status = torch.empty(1, dtype=torch.int32, pin_memory=True)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(ready)
            host.copy_(ids[:n], non_blocking=True)
            status.copy_(self._status_dev, non_blocking=True)
            ev.record(self.copy_stream)
        self.d2h_bytes += n * 8 + 4

        def get():
            ev.synchronize()
            self._check_status(int(status[0]))
            return self._build_output(info, host.tolist())

        return get
