"""Python half of the C interface (``include/vllm.h``): the C layer embeds the interpreter and
calls these functions with plain dicts / strings; everything heavy stays in the engine.

Reference: ``src/capi/vllm_c.cpp:404-855``, ``src/capi/chat_prompt.cpp``.
"""
from __future__ import annotations

import json
import time
import uuid

from . import _engine as E


class EngineHandle:
    def __init__(self, params: dict):
        from .config import EngineArgs, ParallelConfig
        from .entrypoints.api_server import ServerState
        from .parallel.launch import launch_engine
        par = ParallelConfig(tensor_parallel_size=max(1, params.get("tensor_parallel_size") or 1),
                             enable_expert_parallel=bool(params.get("enable_expert_parallel")))
        args = EngineArgs(model=params["model_path"], tokenizer=params.get("tokenizer_config_path") or None,
                          block_size=params.get("block_size") or 32, num_blocks=params.get("num_blocks") or 256,
                          max_model_len=params.get("max_model_len") or 0, max_num_seqs=params.get("max_num_seqs") or 8,
                          device=params.get("device") or "cuda", parallel=par)
        self.llm, _ = launch_engine(args)
        tool = params.get("tool_parser") or "auto"
        reason = params.get("reasoning_parser")
        self.state = ServerState(self.llm, params["model_path"], tool_parser=tool,
                                 reasoning_parser=None if reason == "none" else (reason or "auto"))
        if self.state.tool_parser is None:
            self.state.tool_parser = "hermes"
        if reason == "none":
            self.state.reasoning_parser = None
        self.engine = self.state.engine

    def close(self):
        self.engine.shutdown()


def load(params: dict) -> EngineHandle:
    return EngineHandle(params)


def _sampling(p: dict):
    if not p.get("repetition_penalty", 0) > 0:
        raise ValueError("repetition_penalty must be > 0 (use vllm_sampling_params_default)")
    kw = dict(temperature=p["temperature"], top_p=p["top_p"], top_k=max(0, p["top_k"]), min_p=p["min_p"],
              max_tokens=p["max_tokens"], presence_penalty=p["presence_penalty"],
              frequency_penalty=p["frequency_penalty"], repetition_penalty=p["repetition_penalty"],
              min_tokens=p["min_tokens"], ignore_eos=p["ignore_eos"])
    if p.get("has_seed"):
        kw["seed"] = int(p["seed"])
    if p.get("stop"):
        kw["stop"] = list(p["stop"])
    sp = E.SamplingParams(**kw)
    sp.output_kind = E.OutputKind.DELTA
    so = E.StructuredOutputsParams()
    if p.get("structured_json"):
        so.json = p["structured_json"]
    if p.get("structured_regex"):
        so.regex = p["structured_regex"]
    if p.get("structured_choice"):
        so.choice = list(p["structured_choice"])
    if p.get("structured_grammar"):
        so.grammar = p["structured_grammar"]
    if p.get("structured_json_object"):
        so.json_object = True
    if so.count() > 1:
        raise ValueError("at most one structured-output constraint may be set")
    if so.any():
        sp.structured_outputs = so
    return sp


def submit(h: EngineHandle, prompt: str, params: dict):
    """-> (request id, prompt token count)."""
    if h.llm.tokenizer is None:
        raise ValueError("the model has no tokenizer")
    ids = h.llm.tokenizer.encode(prompt)
    sp = _sampling(params)
    room = h.llm.max_model_len - len(ids)
    if room < 1:
        raise ValueError(f"the prompt has {len(ids)} tokens but the context is {h.llm.max_model_len}")
    if sp.max_tokens > room:
        sp.max_tokens = room
    return h.engine.submit(ids, sp), len(ids)


def stream(h: EngineHandle, rid: str):
    """Yields (delta text, finished, finish_reason, completion tokens so far, error)."""
    n = 0
    for item in h.engine.stream(rid):
        n += len(item.token_ids)
        yield item.text, bool(item.finished), item.finish_reason or "", n, item.error or ""


def abort(h: EngineHandle, rid: str) -> None:
    h.engine.abort(rid)


class _Capture:
    """Stands in for the HTTP handler so that the chat route's logic is reused verbatim."""

    def __init__(self, state):
        from .entrypoints import api_server
        self.state = state
        self.chunks, self.result, self.status = [], None, 200
        self._h = api_server.Handler.__new__(api_server.Handler)
        self._h.state = state
        self._h._send_json = self._send_json
        self._h._sse_begin = lambda: None
        self._h._sse = self._sse
        self.on_chunk = None

    def _send_json(self, status, obj):
        self.status, self.result = status, obj

    def _sse(self, obj):
        text = obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)
        if self.on_chunk is not None and self.on_chunk(text) is False:
            raise BrokenPipeError("client stopped the stream")


def chat(h: EngineHandle, request_json: str) -> str:
    from .entrypoints.api_server import ApiError
    body = json.loads(request_json)
    body["stream"] = False
    cap = _Capture(h.state)
    try:
        cap._h._chat(body)
    except ApiError as e:
        raise ValueError(e.message)
    return json.dumps(cap.result, ensure_ascii=False)


def chat_stream(h: EngineHandle, request_json: str, on_chunk) -> None:
    """``on_chunk(text) -> bool`` gets every chunk JSON and finally "[DONE]"."""
    from .entrypoints.api_server import ApiError
    body = json.loads(request_json)
    body["stream"] = True
    cap = _Capture(h.state)
    cap.on_chunk = on_chunk
    try:
        cap._h._chat(body)
    except ApiError as e:
        raise ValueError(e.message)


def version() -> str:
    from . import __version__
    return __version__
