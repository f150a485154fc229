"""Asynchronous engine: one background thread drives ``LLM.step()`` while any number of
callers submit requests and read their outputs from per-request queues (streaming or final).

Reference: ``src/vllm/v1/engine/async_llm.cpp`` (AsyncLLM: input thread, output thread,
per-request collectors, abort on client disconnect).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Iterator, Optional

from ..engine.llm import LLM, RequestOutput


@dataclass
class StreamItem:
    text: str = ""                 # new text since the last item
    token_ids: list = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    stop_reason: object = None
    logprobs: Optional[list] = None
    error: Optional[str] = None
    num_prompt_tokens: int = 0
    num_cached_tokens: int = 0
    t: float = 0.0


class AsyncLLM:
    def __init__(self, llm: LLM):
        self.llm = llm
        self._lock = threading.Lock()                 # guards the engine (add / abort / step)
        self._queues: dict[str, queue.Queue] = {}
        self._sent: dict[str, int] = {}               # tokens / text already delivered
        self._sent_text: dict[str, int] = {}
        self._wake = threading.Event()
        self._stop = False
        self.errored: Optional[str] = None
        self._thread = threading.Thread(target=self._loop, name="engine-loop", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ client side
    def submit(self, prompt_token_ids, params, request_id: Optional[str] = None, prompt=None) -> str:
        if self.errored:
            raise RuntimeError(f"engine is dead: {self.errored}")
        with self._lock:
            rid = self.llm.add_request(prompt_token_ids, params, request_id=request_id, prompt=prompt)
            self._queues[rid] = queue.Queue()
            self._sent[rid] = 0
            self._sent_text[rid] = 0
        self._wake.set()
        return rid

    def abort(self, request_id: str) -> None:
        with self._lock:
            if request_id in self._queues:
                self.llm.abort_request(request_id)
                q = self._queues.pop(request_id)
                self._sent.pop(request_id, None)
                self._sent_text.pop(request_id, None)
                q.put(StreamItem(finished=True, finish_reason="abort", t=time.monotonic()))

    def stream(self, request_id: str, timeout: Optional[float] = None) -> Iterator[StreamItem]:
        q = self._queues.get(request_id)
        if q is None:
            return
        while True:
            item = q.get(timeout=timeout)
            yield item
            if item.finished or item.error:
                return

    def generate(self, prompt_token_ids, params, request_id=None) -> StreamItem:
        """Blocking: the concatenation of the stream."""
        rid = self.submit(prompt_token_ids, params, request_id)
        text, toks, last = [], [], None
        for item in self.stream(rid):
            text.append(item.text)
            toks.extend(item.token_ids)
            last = item
        last.text, last.token_ids = "".join(text), toks
        return last

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        self._thread.join(timeout=10)
        if hasattr(self.llm, "shutdown"):
            self.llm.shutdown()          # ends the worker ranks of a multi-rank engine

    # ------------------------------------------------------------------ engine thread
    def _deliver(self, st: RequestOutput) -> None:
        rid = st.request_id
        q = self._queues.get(rid)
        if q is None:
            return
        c = st.outputs[0]
        n0 = self._sent.get(rid, 0)
        new_toks = c.token_ids[n0:]
        self._sent[rid] = len(c.token_ids)
        if st.detok is not None:
            if st.delta:
                piece = st.delta_text or ""
            else:
                t0 = self._sent_text.get(rid, 0)
                piece = c.text[t0:]
                self._sent_text[rid] = len(c.text)
        else:
            piece = ""
        item = StreamItem(text=piece, token_ids=list(new_toks), finished=st.finished,
                          finish_reason=c.finish_reason, stop_reason=c.stop_reason,
                          logprobs=c.logprobs[n0:] if c.logprobs else None,
                          num_prompt_tokens=len(st.prompt_token_ids),
                          num_cached_tokens=st.num_cached_tokens, t=time.monotonic())
        q.put(item)
        if st.finished:
            self._queues.pop(rid, None)
            self._sent.pop(rid, None)
            self._sent_text.pop(rid, None)

    def _loop(self) -> None:
        try:
            while not self._stop:
                with self._lock:
                    busy = self.llm.has_unfinished_requests()
                    outs = self.llm.step() if busy else []
                    for st in outs:
                        self._deliver(st)
                if not busy:
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
        except Exception as e:  # engine death: fail every waiter instead of hanging them
            self.errored = f"{type(e).__name__}: {e}"
            with self._lock:
                for q in self._queues.values():
                    q.put(StreamItem(finished=True, error=self.errored, finish_reason="error"))
                self._queues.clear()


class DataParallelEngine:
    """N engine replicas (one ``AsyncLLM`` each, typically one per GPU) behind the interface of one:
    a request goes to the replica with the fewest requests in flight and stays there. The front end
    of data-parallel serving for models that fit on one GPU (reference: the data-parallel section
    of ``.agents/specs/tensor-parallelism.md``; the reference itself serves one engine)."""

    def __init__(self, llms: list):
        self.replicas = [AsyncLLM(l) for l in llms]
        self.llm = llms[0]
        self._lock = threading.Lock()
        self._where: dict[str, int] = {}
        self._inflight = [0] * len(self.replicas)
        self._next = 0
        self.routed = [0] * len(self.replicas)          # requests sent to each replica so far

    @property
    def errored(self) -> Optional[str]:
        for r in self.replicas:
            if r.errored:
                return r.errored
        return None

    def submit(self, prompt_token_ids, params, request_id: Optional[str] = None, prompt=None) -> str:
        with self._lock:
            i = min(range(len(self.replicas)), key=lambda j: (self._inflight[j], (j - self._next) % len(self.replicas)))
            self._next = (i + 1) % len(self.replicas)
            self._next_id = getattr(self, "_next_id", 0) + 1
            rid = request_id or f"dp{i}-req-{self._next_id}"
            self._inflight[i] += 1
            self.routed[i] += 1
            self._where[rid] = i
        try:
            return self.replicas[i].submit(prompt_token_ids, params, request_id=rid, prompt=prompt)
        except Exception:
            self._done(rid)
            raise

    def _done(self, rid: str) -> None:
        with self._lock:
            i = self._where.pop(rid, None)
            if i is not None:
                self._inflight[i] -= 1

    def stream(self, request_id: str, timeout: Optional[float] = None) -> Iterator[StreamItem]:
        i = self._where.get(request_id)
        if i is None:
            return
        try:
            for item in self.replicas[i].stream(request_id, timeout):
                yield item
        finally:
            self._done(request_id)

    def abort(self, request_id: str) -> None:
        i = self._where.get(request_id)
        if i is not None:
            self.replicas[i].abort(request_id)

    def generate(self, prompt_token_ids, params, request_id=None) -> StreamItem:
        rid = self.submit(prompt_token_ids, params, request_id)
        text, toks, last = [], [], None
        for item in self.stream(rid):
            text.append(item.text)
            toks.extend(item.token_ids)
            last = item
        last.text, last.token_ids = "".join(text), toks
        return last

    def shutdown(self) -> None:
        for r in self.replicas:
            r.shutdown()
