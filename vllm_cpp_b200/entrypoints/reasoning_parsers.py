"""Reasoning parsers: split a model's answer into ``reasoning_content`` and ``content``.

Dialects differ in the tags and in whether the opening tag is emitted by the model or already
injected by the chat template (then the answer starts inside the reasoning span).

Reference: ``src/vllm/entrypoints/openai/reasoning_parsers/`` (think_auto, basic, deepseek_r1,
mistral, minimax_m2, step3, olmo3; detection in ``detect.cpp:22-23``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class ReasoningDialect:
    start: str
    end: str
    implicit_start: bool      # the answer begins inside the reasoning span
    require_end: bool = False  # without an end tag everything is content (basic)


REASONING: dict[str, ReasoningDialect] = {
    "basic": ReasoningDialect("<think>", "</think>", False, True),
    "deepseek_r1": ReasoningDialect("<think>", "</think>", True),
    "think_auto": ReasoningDialect("<think>", "</think>", False),
    "mistral": ReasoningDialect("[THINK]", "[/THINK]", False),
    "minimax_m2": ReasoningDialect("<think>", "</think>", True),
    "step3": ReasoningDialect("<think>", "</think>", True),
    "olmo3": ReasoningDialect("<think>", "</think>", False),
}


def list_reasoning_parsers() -> list[str]:
    return sorted(REASONING)


def detect_reasoning_parser(chat_template: str) -> Optional[str]:
    t = chat_template or ""
    if "[THINK]" in t:
        return "mistral"
    if "<think>" in t or "</think>" in t:
        # templates that append "<think>\\n" to the generation prompt start inside the span
        tail = t[-400:]
        return "deepseek_r1" if "<think>" in tail and "add_generation_prompt" in t else "think_auto"
    return None


class ReasoningParser:
    def __init__(self, name: str, prompt_ends_in_reasoning: Optional[bool] = None):
        if name not in REASONING:
            raise ValueError(f"unknown reasoning parser {name!r}; known: {', '.join(list_reasoning_parsers())}")
        self.d = REASONING[name]
        self.name = name
        self.inside = self.d.implicit_start if prompt_ends_in_reasoning is None else prompt_ends_in_reasoning
        self._started = self.inside
        self._done = False
        self._buf = ""

    def extract(self, text: str) -> tuple[Optional[str], Optional[str]]:
        """-> (reasoning_content, content) of a complete answer."""
        d = self.d
        t = text
        if d.start in t:
            pre, _, rest = t.partition(d.start)
            if d.end in rest:
                r, _, c = rest.partition(d.end)
                return (r.strip("\n") or None), ((pre + c).strip("\n") or None)
            if d.require_end:
                return None, text
            return (rest.strip("\n") or None), (pre.strip("\n") or None)
        if d.end in t:
            r, _, c = t.partition(d.end)
            return (r.strip("\n") or None), (c.strip("\n") or None)
        if self.inside and not d.require_end:
            return (t.strip("\n") or None), None
        return None, text

    def feed(self, piece: str, final: bool = False) -> list[dict]:
        """Streaming deltas: {"reasoning_content": s} / {"content": s}; text that may be the
        beginning of a tag is held back until it is decided."""
        d = self.d
        self._buf += piece
        out = []

        def emit(kind, s):
            if s:
                if out and kind in out[-1]:
                    out[-1][kind] += s
                else:
                    out.append({kind: s})

        while self._buf:
            if self._done:
                emit("content", self._buf)
                self._buf = ""
                break
            if self.inside:
                k = self._buf.find(d.end)
                if k >= 0:
                    emit("reasoning_content", self._buf[:k])
                    self._buf = self._buf[k + len(d.end):].lstrip("\n")
                    self.inside, self._done = False, True
                    continue
                hold = _partial_suffix(self._buf, d.end) if not final else 0
                emit("reasoning_content", self._buf[: len(self._buf) - hold])
                self._buf = self._buf[len(self._buf) - hold:]
                break
            # outside, span not seen yet
            k = self._buf.find(d.start)
            if k >= 0 and not self._started:
                emit("content", self._buf[:k])
                self._buf = self._buf[k + len(d.start):].lstrip("\n")
                self.inside = self._started = True
                continue
            k = self._buf.find(d.end)
            if k >= 0 and not self._started:      # end tag without a start: all before it was reasoning
                emit("reasoning_content", self._buf[:k])
                self._buf = self._buf[k + len(d.end):].lstrip("\n")
                self._done = True
                continue
            hold = 0 if final else max(_partial_suffix(self._buf, d.start), _partial_suffix(self._buf, d.end))
            emit("content", self._buf[: len(self._buf) - hold])
            self._buf = self._buf[len(self._buf) - hold:]
            break
        return out


def _partial_suffix(text: str, tag: str) -> int:
    for k in range(min(len(tag) - 1, len(text)), 0, -1):
        if text.endswith(tag[:k]):
            return k
    return 0
