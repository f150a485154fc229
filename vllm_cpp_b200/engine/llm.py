"""The public Python API: ``LLM`` (offline, synchronous step loop) on top of the C++ engine
core, a model from the registry and a ``ModelRunner``.

Assembly order follows the reference's ``LoadedEngine`` (``src/vllm/entrypoints/
model_loader.cpp:273-366``): config -> model/weights -> KV sizing -> runner -> scheduler
config (token budget per family, prefix caching unless hybrid, async when the runner
supports it) -> engine core. ``LLMEngine``-style calls: ``add_request / step / generate /
abort_request`` (``src/vllm/v1/engine/llm_engine.cpp:22-83``).
"""
from __future__ import annotations

import os

import itertools
import time
from dataclasses import dataclass, field
from typing import Iterable, Optional, Sequence

import torch

from .. import _engine as E
from ..config import EngineArgs, ModelConfig, ParallelConfig, load_model_config
from ..models import registry
from ..worker.runner import ModelRunner

SamplingParams = E.SamplingParams


@dataclass
class CompletionOutput:
    index: int = 0
    text: str = ""
    token_ids: list = field(default_factory=list)
    logprobs: Optional[list] = None
    finish_reason: Optional[str] = None
    stop_reason: Optional[object] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list
    outputs: list
    finished: bool = False
    num_cached_tokens: int = 0
    prompt: Optional[str] = None
    metrics: dict = field(default_factory=dict)
    detok: object = None          # incremental detokenizer (stop strings, UTF-8 hold-back)
    delta: bool = False
    delta_text: Optional[str] = None


class LLM:
    def __init__(self, args: EngineArgs | None = None, comm=None, **kw):
        """``comm``: a communicator to use instead of the one built from ``args.parallel``
        (host-mock ranks in tests)."""
        if args is None:
            args = EngineArgs(**kw)
        self.args = args
        cfg = args.model_config
        self.tokenizer = None
        tensors = None
        if cfg is None:
            if args.model is None:
                raise ValueError("either model or model_config is required")
            from ..loader import load_model_dir
            cfg, tensors, self.tokenizer = load_model_dir(args.model, args.tokenizer)
        self.cfg = cfg
        par = args.parallel
        self.comm = comm if comm is not None else self._make_comm(par)
        device = torch.device(args.device)
        if device.type == "cuda":
            torch.cuda.set_device(par.local_rank)
            device = torch.device("cuda", par.local_rank)
        self.device = device
        max_len = args.max_model_len or cfg.max_position_embeddings
        self.max_model_len = max_len
        _, cls = registry.resolve(cfg.architecture)
        self.model = cls(cfg, device=device, parallel=par, comm=self.comm, max_position=max_len)
        if torch.device(device).type == "cpu" and args.cpu_backend == "native":
            from ..models.backend import CpuNativeBackend
            self.model.be = CpuNativeBackend(device)
        mtp_tensors: dict = {}
        if tensors is not None:
            want_mtp = args.speculative_config is not None and args.speculative_config.method == "mtp"

            def trunk_only(it):
                # the draft head's tensors ride in the same checkpoint; they are set aside here
                for name, t in it:
                    if name.startswith(("mtp.", "model.mtp.")):
                        if want_mtp:
                            mtp_tensors[name] = t
                        continue
                    yield name, t
            self.model.load_weights(trunk_only(tensors))
        else:
            self.model.init_random(args.seed)
        if getattr(cfg, "quant", None) == "nvfp4" and getattr(args, "quantize", True) \
                and hasattr(self.model, "quantize_weights"):
            self.model.quantize_weights("nvfp4")
        if getattr(cfg, "quant", None) == "fp8" and getattr(args, "quantize", True) \
                and hasattr(self.model, "quantize_weights") and os.environ.get("B200_FP8_WEIGHTS", "fp8") == "fp8":
            # fp8 checkpoints run W8A8 on the fp8 tensor cores (B200_FP8_WEIGHTS=bf16: expanded weights)
            self.model.quantize_weights("fp8")
        if args.cpu_weight_quant and torch.device(device).type == "cpu" \
                and hasattr(self.model, "quantize_weights"):
            self.model.quantize_weights(args.cpu_weight_quant)
        if par.enable_eplb and hasattr(self.model, "enable_eplb") and getattr(cfg, "num_experts", 0):
            from ..parallel.eplb import EplbConfig
            self.model.enable_eplb(EplbConfig(
                num_redundant_experts=par.eplb_redundant_experts, interval=par.eplb_interval,
                window=par.eplb_window, num_groups=max(1, getattr(cfg, "n_group", 1) or 1)))
        budget = args.resolve_max_num_batched_tokens(cfg)
        spec = args.speculative_config
        # a draft model is loaded before the cache is sized: its weights and its share of every
        # KV block come out of the same memory
        drafter = self._load_draft_model(spec, args, par, max_len) \
            if spec is not None and spec.method == "draft_model" else None
        self._draft_kv_bytes = drafter.model.kv_bytes_per_block(args.block_size) if drafter else 0
        num_blocks = args.num_blocks or self._size_kv_cache(args, budget, max_len)
        if par.tensor_parallel_size > 1:
            # every rank must size its cache alike: the scheduler counts one set of blocks
            num_blocks = min(self.comm.all_gather_object(int(num_blocks)))
        self.is_driver = par.rank == 0 or not par.driver_worker
        channel = self._make_step_channel(par) if (par.driver_worker and par.tensor_parallel_size > 1) else None
        use_async = args.async_scheduling if args.async_scheduling is not None else False
        if spec is not None and spec.method in ("ngram", "mtp", "draft_model"):
            use_async = False       # drafts are verified on the host between steps
        if spec is not None and spec.method == "mtp":
            if not hasattr(self.model, "is_gdn") or par.tensor_parallel_size > 1:
                raise ValueError("method 'mtp' needs a model with a multi-token-prediction head "
                                 "(the Qwen3.5 / 3.6 / Qwen3-Next hybrids) on one rank")
        self.runner = ModelRunner(self.model, block_size=args.block_size, num_blocks=num_blocks,
                                  max_num_seqs=args.max_num_seqs, max_num_batched_tokens=budget,
                                  max_model_len=max_len, enable_cuda_graphs=args.enable_cuda_graphs,
                                  async_mode=use_async, speculative_config=spec, step_channel=channel)
        if spec is not None and spec.method == "mtp":
            from ..models.gdn_mtp import Qwen35MTP
            mtp = Qwen35MTP(self.model, getattr(cfg, "mtp_num_hidden_layers", 1) or 1)
            if mtp_tensors:
                mtp.load_weights(iter(mtp_tensors.items()))
            else:
                mtp.init_random(args.seed)
            self.runner.attach_mtp(mtp)
        if drafter is not None:
            self.runner.attach_draft_model(drafter)
        sc = E.SchedulerConfig(max_num_batched_tokens=budget, max_num_seqs=args.max_num_seqs,
                               max_model_len=max_len, policy=args.scheduling_policy,
                               async_scheduling=use_async,
                               enable_prefix_caching=args.resolve_prefix_caching(cfg))
        if self.runner.max_spec:
            sc.num_lookahead_tokens = self.runner.max_spec
        self.scheduler_config = sc
        self.structured = None
        if self.tokenizer is not None and hasattr(E, "StructuredOutputManager"):
            tk = self.tokenizer
            tb = [b"" if tk.is_special(i) else tk.token_bytes(i) for i in range(tk.vocab_size)]
            eos = [e for e in {cfg.eos_token_id, tk.eos_id} if e is not None and e >= 0]
            self.structured = E.StructuredOutputManager(tb, cfg.vocab_size, eos)
        self.offload = None
        if args.kv_transfer_config and args.kv_transfer_config.get("kv_connector") == "LMCacheConnector":
            from ..worker.lmcache import LMCacheConnector, LMCacheStore
            ktc = args.kv_transfer_config
            caches = self.model.kv_caches
            caches = list(caches.values()) if isinstance(caches, dict) else list(caches)
            store = LMCacheStore(ktc["url"], ktc.get("model_name", f"{cfg.architecture}:{cfg.hidden_size}x{cfg.num_layers}"),
                                 caches, args.block_size, chunk_size=int(ktc.get("chunk_size", 256)),
                                 world_size=par.tensor_parallel_size, worker_id=par.rank,
                                 hash_algo=ktc.get("hash_algo", "blake3"))
            self.offload = LMCacheConnector(store)
            self.runner.offload = self.offload
        elif args.kv_transfer_config:
            from ..worker.offload import KVOffloadWorker
            caches = self.model.kv_caches
            caches = list(caches.values()) if isinstance(caches, dict) else list(caches)
            self.offload = KVOffloadWorker(caches, args.block_size, args.kv_transfer_config,
                                           model_id=f"{cfg.architecture}:{cfg.hidden_size}x{cfg.num_layers}")
            self.runner.offload = self.offload
        self.core = E.EngineCore(sc, self.runner.kv_cache_config(), self.runner,
                                 2 if use_async else 1, self.structured,
                                 self.offload.connector if self.offload else None)
        self.use_async = use_async
        self._counter = itertools.count()
        self._states: dict[str, RequestOutput] = {}
        self.eos_token_id = cfg.eos_token_id
        self.step_times: list = []

    # ------------------------------------------------------------------ set-up helpers
    def _load_draft_model(self, spec, args, par, max_len):
        """The second model of ``method="draft_model"``: same device, backend and max length as the
        target; its weights come from ``spec.draft_model`` (a directory or .gguf file) or, for a
        ``draft_model_config``, from a seeded random init."""
        from ..models.draft import DraftModel
        if par.tensor_parallel_size > 1:
            raise ValueError("method 'draft_model' runs on one rank")
        tensors = None
        dcfg = spec.draft_model_config
        if dcfg is None:
            from ..loader import load_model_dir
            dcfg, tensors, _ = load_model_dir(spec.draft_model, args.tokenizer or args.model)
        _, cls = registry.resolve(dcfg.architecture)
        draft = cls(dcfg, device=self.device, parallel=par, comm=self.comm, max_position=max_len)
        if type(draft.be) is not type(self.model.be):
            draft.be = type(self.model.be)(self.device)
        if tensors is not None:
            draft.load_weights(tensors)
        else:
            draft.init_random(args.seed if spec.draft_seed is None else spec.draft_seed)
        return DraftModel(draft, self.model)

    @staticmethod
    def _make_comm(par: ParallelConfig):
        from ..parallel.comm import SingleComm, TorchComm
        if par.tensor_parallel_size <= 1:
            return SingleComm()
        return TorchComm()

    def _make_step_channel(self, par: ParallelConfig):
        """What the scheduling rank publishes steps on: a host-side (gloo) group beside the NCCL
        one, so that control messages never queue behind GPU work; a communicator handed in by
        the caller (thread ranks in tests) serves as its own channel."""
        from ..parallel.comm import TorchComm
        if isinstance(self.comm, TorchComm):
            import torch.distributed as dist
            return TorchComm(dist.new_group(backend="gloo"))
        return self.comm

    def serve_as_worker(self) -> None:
        """Rank > 0 of a ``driver_worker`` engine: run the steps rank 0 publishes until it stops."""
        if self.is_driver:
            raise RuntimeError("serve_as_worker() is for the ranks that own no scheduler")
        self.runner.serve_steps()

    workers = None     # parallel.launch.WorkerGroup when this process started the other ranks

    def shutdown(self) -> None:
        """Ends the worker ranks' loops (driver_worker engines); harmless otherwise."""
        if self.is_driver and self.runner.step_channel is not None:
            if self.workers is None or self.workers.failed is None:
                self.runner.stop_workers()
            self.runner.step_channel = None
        if self.workers is not None:
            self.workers.shutdown()
            self.workers = None

    def _size_kv_cache(self, args: EngineArgs, budget: int, max_len: int) -> int:
        per_block = self.model.kv_bytes_per_block(args.block_size) + getattr(self, "_draft_kv_bytes", 0)
        if self.device.type != "cuda":
            want = args.max_num_seqs * ((max_len + args.block_size - 1) // args.block_size) + 1
            return max(16, min(want, 4096))
        torch.cuda.synchronize()
        free, total = torch.cuda.mem_get_info(self.device)
        # leave room for activations of a full-budget step
        c = self.cfg
        act = budget * (4 * c.hidden_size + 3 * max(c.intermediate_size, 1)) * 2 * 2
        usable = free - (1.0 - args.gpu_memory_utilization) * total - act - (2 << 30)
        n = int(usable // per_block)
        cap = args.max_num_seqs * ((max_len + args.block_size - 1) // args.block_size) + 16
        return max(16, min(n, cap))

    # ------------------------------------------------------------------ LLMEngine surface
    def add_request(self, prompt_token_ids: Sequence[int], params: "E.SamplingParams",
                    request_id: Optional[str] = None, priority: int = 0,
                    prompt: Optional[str] = None) -> str:
        if not self.is_driver:
            raise RuntimeError("this rank owns no scheduler: requests go to rank 0")
        rid = request_id or f"req-{next(self._counter)}"
        toks = list(prompt_token_ids)
        if len(toks) >= self.max_model_len:
            raise ValueError(f"prompt ({len(toks)} tokens) is longer than max_model_len "
                             f"({self.max_model_len})")
        req = E.EngineCoreRequest(rid, toks, params, self.eos_token_id, time.monotonic(), priority)
        self.runner.set_eos(rid, self.eos_token_id)
        if self.structured is not None and params.structured_outputs is not None \
                and params.structured_outputs.any():
            self.structured.validate(params.structured_outputs)    # raises on a bad constraint
        self.core.add_request(req)
        st = RequestOutput(rid, toks, [CompletionOutput()], prompt=prompt)
        if self.tokenizer is not None and params.detokenize:
            st.detok = E.IncrementalDetokenizer(self.tokenizer, toks, params.skip_special_tokens,
                                                list(params.stop), params.include_stop_str_in_output,
                                                params.min_tokens)
        st.delta = params.output_kind == E.OutputKind.DELTA
        self._states[rid] = st
        return rid

    def abort_request(self, request_id: str) -> None:
        self.core.abort_requests([request_id])
        self._states.pop(request_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.core.has_work()

    def step(self) -> list[RequestOutput]:
        """One engine step; returns the requests that produced tokens (finished ones are
        flagged and dropped from the live table)."""
        if self.workers is not None and self.workers.failed:
            # a rank is gone: the next collective could never complete
            raise E.EngineDeadError(f"tensor-parallel worker lost: {self.workers.failed}")
        outs, _ = self.core.step_with_batch_queue() if self.use_async else self.core.step()
        done = []
        for o in outs.outputs:
            st = self._states.get(o.request_id)
            if st is None:
                continue
            c = st.outputs[0]
            c.token_ids.extend(o.new_token_ids)
            st.num_cached_tokens = o.num_cached_tokens
            stop_hit = None
            if st.detok is not None and o.new_token_ids:
                # the last token of a request that stopped on EOS / a stop token is not text
                stop_terminated = (o.finished() and E.finish_reason_str(o.finish_reason) == "stop"
                                   and (o.stop_reason is None or o.stop_reason.is_token))
                stop_hit = st.detok.update(list(o.new_token_ids), bool(stop_terminated))
                if stop_hit is not None and not o.finished():
                    # a stop string ends the request here: drop it from the engine
                    self.core.abort_requests([o.request_id])
                    c.finish_reason, c.stop_reason = "stop", stop_hit
                    st.finished = True
                    self._states.pop(o.request_id, None)
                finished_now = st.finished or o.finished()
                piece = st.detok.get_next_output_text(finished_now, st.delta)
                c.text = piece if st.delta else piece
                st.delta_text = piece if st.delta else None
            if st.finished:
                done.append(st)
                continue
            if o.new_logprobs:
                c.logprobs = (c.logprobs or []) + list(o.new_logprobs)
            if o.finished():
                c.finish_reason = E.finish_reason_str(o.finish_reason)
                if o.stop_reason is not None:
                    c.stop_reason = o.stop_reason.token if o.stop_reason.is_token else o.stop_reason.text
                st.finished = True
                self._states.pop(o.request_id, None)
            done.append(st)
        return done

    def generate(self, prompts: Iterable, sampling_params=None, use_tqdm: bool = False):
        """Runs a batch to completion. ``prompts``: token-id lists, strings (needs a tokenizer)
        or dicts with ``prompt_token_ids``. Returns RequestOutputs in input order."""
        prompts = list(prompts)
        if sampling_params is None:
            sampling_params = E.SamplingParams()
        if not isinstance(sampling_params, (list, tuple)):
            sampling_params = [sampling_params] * len(prompts)
        order = []
        for p, sp in zip(prompts, sampling_params):
            text = None
            if isinstance(p, str):
                if self.tokenizer is None:
                    raise ValueError("string prompts need a tokenizer")
                text, p = p, self.tokenizer.encode(p)
            elif isinstance(p, dict):
                p = p["prompt_token_ids"]
            order.append(self.add_request(p, sp, prompt=text))
        results: dict[str, RequestOutput] = {}
        while self.has_unfinished_requests():
            for st in self.step():
                if st.finished:
                    results[st.request_id] = st
        outs = [results[r] for r in order if r in results]
        if self.tokenizer is not None:
            for o in outs:
                for c in o.outputs:
                    if o.detok is None:
                        c.text = self.tokenizer.decode(c.token_ids)
        return outs

    def stats(self):
        return self.core.scheduler().make_stats()

    def step_stats(self) -> dict:
        """Counters of the last step: queue depths, KV usage, scheduled tokens, the host time
        spent scheduling / updating and the device time of the step (when the runner records
        CUDA events, ``runner.time_steps``)."""
        st = self.core.scheduler().make_stats()
        c = self.core
        d = {"num_running": st.num_running_reqs, "num_waiting": st.num_waiting_reqs,
             "kv_cache_usage": st.kv_cache_usage, "scheduled_tokens": st.step_scheduled_tokens,
             "prefix_cache_queries": st.prefix_cache_queries, "prefix_cache_hits": st.prefix_cache_hits,
             "num_preempted": st.num_preempted,
             "schedule_ms": getattr(c, "last_schedule_ms", 0.0), "execute_ms": getattr(c, "last_execute_ms", 0.0),
             "update_ms": getattr(c, "last_update_ms", 0.0),
             "h2d_bytes": self.runner.h2d_bytes, "d2h_bytes": self.runner.d2h_bytes,
             "kernel_launches": self.runner.launches}
        if self.runner.spec is not None:
            d.update({"spec_" + k: v for k, v in self.runner.spec_stats.items()})
        return d
