"""OpenAI-compatible HTTP server.

Routes: POST /v1/completions, POST /v1/chat/completions (JSON or SSE ``data: {...}`` ...
``data: [DONE]``), GET /v1/models, GET /health, GET /version, GET /metrics, POST /tokenize,
POST /detokenize. Errors use ``{"error": {"message", "type", "code"}}``. A client that goes
away mid-stream aborts its request.

Reference: ``examples/server/main.cpp:79-203`` (flags), ``src/vllm/entrypoints/openai/
{api_server,protocol,serving_chat,serving_completion}.cpp``.

The HTTP layer is the standard library's threading server: one thread per connection, all of
them feeding the single engine thread of ``AsyncLLM``.
"""
from __future__ import annotations

import argparse
import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from .. import __version__ as VERSION
from .. import _engine as E
from .async_llm import AsyncLLM
from .chat_template import ChatTemplate
from .reasoning_parsers import ReasoningParser, detect_reasoning_parser
from .tool_parsers import ToolParser, detect_tool_parser


class ApiError(Exception):
    def __init__(self, status: int, message: str, type_: str = "invalid_request_error", code=None):
        super().__init__(message)
        self.status, self.message, self.type, self.code = status, message, type_, code

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.type, "code": self.code or self.status}}


# ------------------------------------------------------------------------------ protocol
def sampling_params_from_request(req: dict, default_max_tokens: int, chat: bool) -> "E.SamplingParams":
    """OpenAI request fields (+ the vLLM extras) -> SamplingParams; validates ranges."""
    def num(key, default, lo=None, hi=None, cast=float):
        v = req.get(key)
        if v is None:
            return default
        try:
            v = cast(v)
        except (TypeError, ValueError):
            raise ApiError(400, f"{key} must be a number")
        if (lo is not None and v < lo) or (hi is not None and v > hi):
            raise ApiError(400, f"{key} must be in [{lo}, {hi}]")
        return v

    kw = dict(
        temperature=num("temperature", 1.0, 0.0, None),
        top_p=num("top_p", 1.0, 0.0, 1.0),
        top_k=num("top_k", 0, -1, None, int),
        min_p=num("min_p", 0.0, 0.0, 1.0),
        presence_penalty=num("presence_penalty", 0.0, -2.0, 2.0),
        frequency_penalty=num("frequency_penalty", 0.0, -2.0, 2.0),
        repetition_penalty=num("repetition_penalty", 1.0, 0.0, None),
        min_tokens=num("min_tokens", 0, 0, None, int),
        ignore_eos=bool(req.get("ignore_eos", False)),
        skip_special_tokens=bool(req.get("skip_special_tokens", True)),
        include_stop_str_in_output=bool(req.get("include_stop_str_in_output", False)),
    )
    if kw["top_k"] < 0:
        kw["top_k"] = 0
    mt = req.get("max_completion_tokens") if chat else None
    if mt is None:
        mt = req.get("max_tokens")
    kw["max_tokens"] = int(mt) if mt is not None else default_max_tokens
    if kw["max_tokens"] < 1:
        raise ApiError(400, "max_tokens must be at least 1")
    if req.get("seed") is not None:
        kw["seed"] = int(req["seed"])
    stop = req.get("stop")
    if stop:
        kw["stop"] = [stop] if isinstance(stop, str) else [str(s) for s in stop]
    if req.get("stop_token_ids"):
        kw["stop_token_ids"] = [int(t) for t in req["stop_token_ids"]]
    if req.get("logit_bias"):
        kw["logit_bias"] = {int(k): float(v) for k, v in req["logit_bias"].items()}
    lp = req.get("top_logprobs") if chat else req.get("logprobs")
    if chat and req.get("logprobs") and lp is None:
        lp = 0
    if lp is not None and lp is not False:
        kw["logprobs"] = int(lp)
    sp = E.SamplingParams(**kw)
    sp.output_kind = E.OutputKind.DELTA
    so = structured_outputs_from_request(req)
    if so is not None:
        sp.structured_outputs = so
    return sp


def structured_outputs_from_request(req: dict):
    so = E.StructuredOutputsParams()
    rf = req.get("response_format") or {}
    ext = req.get("structured_outputs") or {}
    if rf.get("type") == "json_object":
        so.json_object = True
    elif rf.get("type") == "json_schema":
        schema = (rf.get("json_schema") or {}).get("schema", rf.get("json_schema"))
        so.json = json.dumps(schema)
    for key, attr in (("guided_json", "json"), ("guided_regex", "regex"), ("guided_choice", "choice"),
                      ("guided_grammar", "grammar")):
        v = req.get(key, ext.get(attr))
        if v is not None:
            setattr(so, attr, json.dumps(v) if attr == "json" and not isinstance(v, str) else v)
    if ext.get("structural_tag"):
        so.structural_tag = ext["structural_tag"] if isinstance(ext["structural_tag"], str) \
            else json.dumps(ext["structural_tag"])
    if so.count() > 1:
        raise ApiError(400, "only one structured-output constraint may be given")
    return so if so.any() else None


def _usage(prompt: int, completion: int, cached: int = 0) -> dict:
    u = {"prompt_tokens": prompt, "completion_tokens": completion, "total_tokens": prompt + completion}
    if cached:
        u["prompt_tokens_details"] = {"cached_tokens": cached}
    return u


def _logprobs_chat(rows, tokenizer) -> Optional[dict]:
    if not rows:
        return None
    content = []
    for r in rows:
        ids, lps = list(r.token_ids), list(r.logprobs)
        def ent(i):
            t = tokenizer.decode([ids[i]], False) if tokenizer else str(ids[i])
            return {"token": t, "logprob": lps[i], "bytes": list(t.encode("utf-8"))}
        e = ent(0)
        e["top_logprobs"] = [ent(i) for i in range(1, len(ids))]
        content.append(e)
    return {"content": content}


class Metrics:
    """Counters and latency sums of the Prometheus endpoint."""

    def __init__(self):
        self.lock = threading.Lock()
        self.c = dict(requests_total=0, requests_failed=0, prompt_tokens_total=0, generation_tokens_total=0,
                      ttft_seconds_sum=0.0, ttft_seconds_count=0, e2e_seconds_sum=0.0, e2e_seconds_count=0)

    def add(self, **kw):
        with self.lock:
            for k, v in kw.items():
                self.c[k] += v

    def render(self, running: int, waiting: int) -> str:
        with self.lock:
            lines = [f"vllm:num_requests_running {running}", f"vllm:num_requests_waiting {waiting}"]
            lines += [f"vllm:{k} {v}" for k, v in self.c.items()]
        return "\n".join(lines) + "\n"


class ServerState:
    def __init__(self, llm, served_model_name: str, tool_parser: Optional[str] = None,
                 reasoning_parser: Optional[str] = None, chat_template: Optional[str] = None,
                 default_max_tokens: int = 256, api_key: Optional[str] = None, replicas: Optional[list] = None):
        self.llm = llm
        if replicas:
            from .async_llm import DataParallelEngine
            self.engine = DataParallelEngine([llm] + list(replicas))
        else:
            self.engine = AsyncLLM(llm)
        self.tokenizer = llm.tokenizer
        self.model_name = served_model_name
        self.default_max_tokens = default_max_tokens
        self.api_key = api_key
        tpl = chat_template or (self.tokenizer.chat_template if self.tokenizer is not None else "") or None
        self.template = ChatTemplate(tpl)
        if not self.template.probe():
            self.template = ChatTemplate(None)
        self.tool_parser = tool_parser if tool_parser not in (None, "auto") else detect_tool_parser(tpl or "")
        self.reasoning_parser = reasoning_parser if reasoning_parser not in (None, "auto") \
            else detect_reasoning_parser(tpl or "")
        self.metrics = Metrics()
        self.created = int(time.time())

    def tokenize(self, text: str, add_special: bool = True) -> list[int]:
        if self.tokenizer is None:
            raise ApiError(400, "this server has no tokenizer: send token ids")
        return self.tokenizer.encode(text, add_special)


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    state: ServerState = None     # set on the server class

    # ------------------------------------------------------------------ plumbing
    def log_message(self, fmt, *args):   # quiet
        pass

    def _send_json(self, status: int, obj) -> None:
        data = json.dumps(obj, ensure_ascii=False).encode("utf-8")
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def _send_text(self, status: int, text: str, ctype="text/plain; version=0.0.4") -> None:
        data = text.encode("utf-8")
        self.send_response(status)
        self.send_header("Content-Type", ctype)
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def _read_json(self) -> dict:
        n = int(self.headers.get("Content-Length") or 0)
        raw = self.rfile.read(n) if n else b""
        try:
            obj = json.loads(raw.decode("utf-8") or "{}")
        except ValueError as e:
            raise ApiError(400, f"invalid JSON body: {e}")
        if not isinstance(obj, dict):
            raise ApiError(400, "the request body must be a JSON object")
        return obj

    def _check_auth(self) -> None:
        key = self.state.api_key
        if key and self.headers.get("Authorization") != f"Bearer {key}":
            raise ApiError(401, "invalid API key", "authentication_error")

    def _sse_begin(self) -> None:
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Connection", "close")
        self.end_headers()
        self.close_connection = True

    def _sse(self, obj) -> None:
        payload = obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)
        self.wfile.write(f"data: {payload}\n\n".encode("utf-8"))
        self.wfile.flush()

    # ------------------------------------------------------------------ routes
    def do_GET(self):
        st = self.state
        try:
            path = self.path.split("?", 1)[0]
            if path == "/health":
                if st.engine.errored:
                    raise ApiError(503, f"engine is dead: {st.engine.errored}", "internal_error")
                self._send_json(200, {"status": "ok"})
            elif path == "/version":
                self._send_json(200, {"version": VERSION})
            elif path == "/v1/models":
                self._check_auth()
                self._send_json(200, {"object": "list", "data": [{
                    "id": st.model_name, "object": "model", "created": st.created, "owned_by": "vllm_cpp_b200",
                    "max_model_len": st.llm.max_model_len}]})
            elif path == "/metrics":
                s = st.llm.stats() if hasattr(st.llm, "stats") else None
                self._send_text(200, st.metrics.render(getattr(s, "num_running_reqs", 0),
                                                       getattr(s, "num_waiting_reqs", 0)))
            else:
                raise ApiError(404, f"no route {path}", "not_found")
        except ApiError as e:
            self._send_json(e.status, e.body())

    def do_POST(self):
        st = self.state
        try:
            self._check_auth()
            path = self.path.split("?", 1)[0]
            body = self._read_json()
            if path == "/v1/completions":
                self._completions(body)
            elif path == "/v1/chat/completions":
                self._chat(body)
            elif path == "/tokenize":
                ids = st.tokenize(body.get("prompt", ""), bool(body.get("add_special_tokens", True)))
                self._send_json(200, {"tokens": ids, "count": len(ids), "max_model_len": st.llm.max_model_len})
            elif path == "/detokenize":
                if st.tokenizer is None:
                    raise ApiError(400, "this server has no tokenizer")
                self._send_json(200, {"prompt": st.tokenizer.decode([int(t) for t in body.get("tokens", [])], False)})
            else:
                raise ApiError(404, f"no route {path}", "not_found")
        except ApiError as e:
            st.metrics.add(requests_failed=1)
            try:
                self._send_json(e.status, e.body())
            except OSError:
                pass
        except (BrokenPipeError, ConnectionResetError):
            pass
        except Exception as e:    # never let a handler thread die silently
            st.metrics.add(requests_failed=1)
            try:
                self._send_json(500, ApiError(500, f"{type(e).__name__}: {e}", "internal_error").body())
            except OSError:
                pass

    # ------------------------------------------------------------------ completions
    def _prompt_ids(self, prompt) -> list[list[int]]:
        st = self.state
        if isinstance(prompt, str):
            return [st.tokenize(prompt)]
        if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            return [list(prompt)]
        if isinstance(prompt, list) and prompt:
            return [st.tokenize(p) if isinstance(p, str) else [int(t) for t in p] for p in prompt]
        raise ApiError(400, "prompt must be a string, a list of strings or token ids")

    def _submit(self, ids: list[int], sp) -> str:
        st = self.state
        if len(ids) + 1 > st.llm.max_model_len:
            raise ApiError(400, f"the prompt has {len(ids)} tokens but the context is {st.llm.max_model_len}")
        room = st.llm.max_model_len - len(ids)
        if sp.max_tokens > room:
            sp.max_tokens = room
        try:
            return st.engine.submit(ids, sp)
        except ValueError as e:
            raise ApiError(400, str(e))
        except RuntimeError as e:
            raise ApiError(503, str(e), "internal_error")

    def _completions(self, body: dict) -> None:
        st = self.state
        if "prompt" not in body:
            raise ApiError(400, "prompt is required")
        prompts = self._prompt_ids(body["prompt"])
        n = int(body.get("n") or 1)
        stream = bool(body.get("stream"))
        echo = bool(body.get("echo"))
        rid = "cmpl-" + uuid.uuid4().hex
        t0 = time.monotonic()
        jobs = []
        for pi, ids in enumerate(prompts):
            for k in range(n):
                sp = sampling_params_from_request(body, st.default_max_tokens, chat=False)
                if n > 1 and body.get("seed") is not None:
                    sp.seed = int(body["seed"]) + k
                jobs.append((pi * n + k, ids, self._submit(ids, sp)))
        st.metrics.add(requests_total=1, prompt_tokens_total=sum(len(j[1]) for j in jobs))
        created = int(time.time())
        if stream:
            self._sse_begin()
            total_completion = 0
            try:
                # streams are drained one after another; each keeps generating meanwhile
                for index, ids, req_id in jobs:
                    first = True
                    for item in st.engine.stream(req_id):
                        if item.error:
                            self._sse({"error": {"message": item.error, "type": "internal_error", "code": 500}})
                            break
                        if first:
                            st.metrics.add(ttft_seconds_sum=item.t - t0, ttft_seconds_count=1)
                            first = False
                        total_completion += len(item.token_ids)
                        text = (st.tokenizer.decode(ids, True) if (echo and total_completion == len(item.token_ids)
                                                                   and st.tokenizer) else "") + item.text
                        self._sse({"id": rid, "object": "text_completion", "created": created, "model": st.model_name,
                                   "choices": [{"index": index, "text": text, "logprobs": None,
                                                "finish_reason": item.finish_reason if item.finished else None}]})
                if (body.get("stream_options") or {}).get("include_usage"):
                    self._sse({"id": rid, "object": "text_completion", "created": created, "model": st.model_name,
                               "choices": [], "usage": _usage(sum(len(j[1]) for j in jobs), total_completion)})
                self._sse("[DONE]")
            except (BrokenPipeError, ConnectionResetError, OSError):
                for _, _, req_id in jobs:
                    st.engine.abort(req_id)
            st.metrics.add(generation_tokens_total=total_completion, e2e_seconds_sum=time.monotonic() - t0,
                           e2e_seconds_count=1)
            return
        choices, completion, cached = [], 0, 0
        for index, ids, req_id in jobs:
            text, toks, last = [], [], None
            for item in st.engine.stream(req_id):
                if item.error:
                    raise ApiError(500, item.error, "internal_error")
                text.append(item.text)
                toks.extend(item.token_ids)
                last = item
            completion += len(toks)
            cached += last.num_cached_tokens if last else 0
            out = "".join(text)
            if echo and st.tokenizer:
                out = st.tokenizer.decode(ids, True) + out
            choices.append({"index": index, "text": out, "logprobs": None,
                            "finish_reason": last.finish_reason if last else None,
                            "stop_reason": last.stop_reason if last else None, "token_ids": toks
                            if body.get("return_token_ids") else None})
        st.metrics.add(generation_tokens_total=completion, e2e_seconds_sum=time.monotonic() - t0, e2e_seconds_count=1)
        self._send_json(200, {"id": rid, "object": "text_completion", "created": created, "model": st.model_name,
                              "choices": choices, "usage": _usage(sum(len(j[1]) for j in jobs), completion, cached)})

    # ------------------------------------------------------------------ chat
    def _chat(self, body: dict) -> None:
        st = self.state
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise ApiError(400, "messages must be a non-empty list")
        tools = body.get("tools") or None
        tool_choice = body.get("tool_choice", "auto" if tools else "none")
        if tool_choice == "none":
            tools_for_prompt = None
        else:
            tools_for_prompt = tools
        try:
            prompt = st.template.render(msgs, tools=tools_for_prompt,
                                        add_generation_prompt=bool(body.get("add_generation_prompt", True)),
                                        **(body.get("chat_template_kwargs") or {}))
        except Exception as e:
            raise ApiError(400, f"chat template error: {e}")
        ids = st.tokenize(prompt, add_special=False) if st.tokenizer is not None else None
        if ids is None:
            raise ApiError(400, "chat needs a tokenizer")
        sp = sampling_params_from_request(body, st.default_max_tokens, chat=True)
        parser_name = st.tool_parser if tools_for_prompt else None
        forced = tool_choice == "required" or isinstance(tool_choice, dict)
        if tools_for_prompt and parser_name and sp.structured_outputs is None and forced:
            chosen = tools
            if isinstance(tool_choice, dict):
                want = (tool_choice.get("function") or {}).get("name")
                chosen = [t for t in tools if t.get("function", t).get("name") == want]
            tag = ToolParser(parser_name).structural_tag(chosen)
            if tag:
                so = E.StructuredOutputsParams()
                so.structural_tag = tag
                sp.structured_outputs = so
        stream = bool(body.get("stream"))
        rid = "chatcmpl-" + uuid.uuid4().hex
        created = int(time.time())
        t0 = time.monotonic()
        req_id = self._submit(ids, sp)
        st.metrics.add(requests_total=1, prompt_tokens_total=len(ids))
        reasoning = ReasoningParser(st.reasoning_parser, st.template.ends_in_reasoning()) \
            if st.reasoning_parser else None
        tool_parser = ToolParser(parser_name) if parser_name else None
        base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": st.model_name}

        def split(piece: str, final: bool) -> list[dict]:
            """text -> deltas through the reasoning parser, then the tool parser."""
            stage1 = reasoning.feed(piece, final) if reasoning else ([{"content": piece}] if piece or final else [])
            out = []
            for d in stage1:
                if "content" in d and tool_parser:
                    out.extend(tool_parser.feed(d["content"], False))
                else:
                    out.append(d)
            if final and tool_parser:
                out.extend(tool_parser.feed("", True))
            return out

        if stream:
            self._sse_begin()
            n_out, saw_tool, first = 0, False, True
            try:
                self._sse(dict(base, choices=[{"index": 0, "delta": {"role": "assistant", "content": ""},
                                               "finish_reason": None}]))
                for item in st.engine.stream(req_id):
                    if item.error:
                        self._sse({"error": {"message": item.error, "type": "internal_error", "code": 500}})
                        break
                    if first and item.token_ids:
                        st.metrics.add(ttft_seconds_sum=item.t - t0, ttft_seconds_count=1)
                        first = False
                    n_out += len(item.token_ids)
                    for d in split(item.text, item.finished):
                        if "tool_call" in d:
                            saw_tool = True
                            tc = d["tool_call"]
                            fn = {k: tc[k] for k in ("name", "arguments") if k in tc}
                            entry = {"index": tc["index"], "function": fn}
                            if "id" in tc:
                                entry.update(id=tc["id"], type="function")
                            delta = {"tool_calls": [entry]}
                        else:
                            delta = d
                        self._sse(dict(base, choices=[{"index": 0, "delta": delta, "finish_reason": None}]))
                    if item.finished:
                        fr = "tool_calls" if (saw_tool and item.finish_reason == "stop") else item.finish_reason
                        self._sse(dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": fr}]))
                if (body.get("stream_options") or {}).get("include_usage"):
                    self._sse(dict(base, choices=[], usage=_usage(len(ids), n_out)))
                self._sse("[DONE]")
            except (BrokenPipeError, ConnectionResetError, OSError):
                st.engine.abort(req_id)
            st.metrics.add(generation_tokens_total=n_out, e2e_seconds_sum=time.monotonic() - t0, e2e_seconds_count=1)
            return
        text, toks, last, lps = [], [], None, []
        for item in st.engine.stream(req_id):
            if item.error:
                raise ApiError(500, item.error, "internal_error")
            text.append(item.text)
            toks.extend(item.token_ids)
            lps.extend(item.logprobs or [])
            last = item
        full = "".join(text)
        reasoning_content = None
        if reasoning:
            reasoning_content, full = reasoning.extract(full)
            full = full or ""
        calls = []
        content = full
        if tool_parser:
            content, calls = tool_parser.extract(full)
        msg = {"role": "assistant", "content": content}
        if reasoning_content is not None:
            msg["reasoning_content"] = reasoning_content
        if calls:
            msg["tool_calls"] = [{"id": c.id, "type": "function",
                                  "function": {"name": c.name, "arguments": c.arguments}} for c in calls]
        fr = "tool_calls" if (calls and last and last.finish_reason == "stop") else (last.finish_reason if last else None)
        st.metrics.add(generation_tokens_total=len(toks), e2e_seconds_sum=time.monotonic() - t0, e2e_seconds_count=1)
        self._send_json(200, {"id": rid, "object": "chat.completion", "created": created, "model": st.model_name,
                              "choices": [{"index": 0, "message": msg, "finish_reason": fr,
                                           "logprobs": _logprobs_chat(lps, st.tokenizer) if body.get("logprobs") else None}],
                              "usage": _usage(len(ids), len(toks), last.num_cached_tokens if last else 0)})


def make_server(state: ServerState, host: str = "0.0.0.0", port: int = 8000) -> ThreadingHTTPServer:
    handler = type("BoundHandler", (Handler,), {"state": state})
    srv = ThreadingHTTPServer((host, port), handler)
    srv.daemon_threads = True
    return srv


def build_arg_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("vllm_cpp_b200 OpenAI-compatible server")
    ap.add_argument("--model", required=True, help="model directory or .gguf file")
    ap.add_argument("--tokenizer-config", dest="tokenizer", default=None)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--enable-prefix-caching", action="store_true", default=None)
    ap.add_argument("--no-enable-prefix-caching", dest="enable_prefix_caching", action="store_false")
    ap.add_argument("--async-scheduling", action="store_true", default=None)
    ap.add_argument("--tool-call-parser", default="auto")
    ap.add_argument("--reasoning-parser", default="auto")
    ap.add_argument("--chat-template", default=None, help="path of a Jinja chat template")
    ap.add_argument("--default-max-tokens", type=int, default=256)
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--tensor-parallel-size", type=int, default=1,
                    help="ranks (one process per GPU); this process is rank 0 and starts the others")
    ap.add_argument("--data-parallel-size", type=int, default=1,
                    help="engine replicas (one per GPU) behind this server; a request goes to the least loaded one")
    ap.add_argument("--enable-expert-parallel", action="store_true",
                    help="MoE models: experts are split over the ranks instead of sharded")
    ap.add_argument("--no-warmup", action="store_true",
                    help="skip the pre-serve warm-up (decode graphs are then captured by the first steps that need them)")
    ap.add_argument("--speculative-config", default=None,
                    help='JSON, e.g. {"method": "ngram", "num_speculative_tokens": 3, "prompt_lookup_max": 4} '
                         'or {"method": "mtp", "num_speculative_tokens": 1} '
                         'or {"method": "draft_model", "draft_model": "<directory>", "num_speculative_tokens": 3}')
    ap.add_argument("--enable-eplb", action="store_true",
                    help="expert parallel: rebalance the expert placement from observed loads")
    ap.add_argument("--eplb-redundant-experts", type=int, default=0,
                    help="physical expert slots beyond one per expert (hot experts get replicas)")
    ap.add_argument("--eplb-interval", type=int, default=3000, help="engine steps between rebalances")
    ap.add_argument("--eplb-window", type=int, default=1000, help="engine steps of load history used")
    return ap


def main(argv=None) -> int:
    from ..config import EngineArgs, ParallelConfig
    from ..parallel.launch import launch_engine
    a = build_arg_parser().parse_args(argv)
    kw = dict(model=a.model, tokenizer=a.tokenizer, device=a.device, block_size=a.block_size,
              max_num_seqs=a.max_num_seqs, max_model_len=a.max_model_len,
              max_num_batched_tokens=a.max_num_batched_tokens,
              gpu_memory_utilization=a.gpu_memory_utilization, async_scheduling=a.async_scheduling,
              enable_prefix_caching=a.enable_prefix_caching)
    if a.speculative_config:
        import json as _json
        from ..spec_decode import SpeculativeConfig
        try:
            kw["speculative_config"] = SpeculativeConfig(**_json.loads(a.speculative_config))
        except (TypeError, ValueError) as e:
            raise SystemExit(f"--speculative-config: {e}")
    kw["parallel"] = ParallelConfig(tensor_parallel_size=max(1, a.tensor_parallel_size),
                                    enable_expert_parallel=a.enable_expert_parallel,
                                    enable_eplb=a.enable_eplb, eplb_redundant_experts=a.eplb_redundant_experts,
                                    eplb_interval=a.eplb_interval, eplb_window=a.eplb_window)
    llm, _workers = launch_engine(EngineArgs(**{k: v for k, v in kw.items() if v is not None}))
    if not a.no_warmup and llm.runner.is_cuda and a.tensor_parallel_size <= 1:
        # capture the decode graphs of every padded batch size before the first request arrives
        # (tensor-parallel engines capture in lockstep inside their first steps instead)
        llm.runner.warmup_graphs()
    replicas = []
    if a.data_parallel_size > 1:
        if a.tensor_parallel_size > 1:
            raise SystemExit("--data-parallel-size with --tensor-parallel-size > 1 is not supported")
        from ..engine import LLM
        for r in range(1, a.data_parallel_size):
            kr = dict(kw)
            if (a.device or "cuda").startswith("cuda"):
                kr["device"] = f"cuda:{r}"
            replicas.append(LLM(EngineArgs(**{k: v for k, v in kr.items() if v is not None})))
    tpl = open(a.chat_template).read() if a.chat_template else None
    state = ServerState(llm, a.served_model_name or a.model, a.tool_call_parser, a.reasoning_parser, tpl,
                        a.default_max_tokens, a.api_key, replicas=replicas)
    srv = make_server(state, a.host, a.port)
    print(f"serving {state.model_name} on http://{a.host}:{a.port} (tool parser: {state.tool_parser}, "
          f"reasoning parser: {state.reasoning_parser})", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        state.engine.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
