"""Tool-call parsers: model output text -> (plain content, tool calls), whole or streamed.

Every dialect is a row of ``DIALECTS``: the markers that open / close a tool-call region and
the payload syntax inside it. One engine handles them all; streaming re-parses the text seen
so far and emits only what is new (content that cannot be the beginning of a marker, a call's
name once, then its argument string as it grows), which is how OpenAI deltas are shaped.

Reference: ``src/vllm/entrypoints/openai/tool_parsers/abstract.cpp:94-252`` (the dialect
names), ``detect.cpp:57-82`` (template-marker auto-detection) and one file per dialect.
"""
from __future__ import annotations

import ast
import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class ToolCall:
    name: str
    arguments: str            # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])


@dataclass
class Dialect:
    kind: str                       # payload syntax, see _PAYLOAD
    start: tuple = ()               # any of these opens a region ("" = the whole text may be one)
    end: str = ""                   # closes a region ("" = runs to the end / is self-delimiting)
    name_key: tuple = ("name",)
    args_key: tuple = ("arguments", "parameters")
    strip_fences: bool = False      # payload may sit in ```json fences
    bare: bool = False              # no marker needed: the text itself may be the payload


def _d(kind, start=(), end="", **kw):
    return Dialect(kind, tuple([start] if isinstance(start, str) else start), end, **kw)


DS_BEGIN, DS_END = "<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>"

DIALECTS: dict[str, Dialect] = {
    "hermes": _d("json", "<tool_call>", "</tool_call>"),
    "qwen3": _d("json", "<tool_call>", "</tool_call>"),
    "qwen3_coder": _d("xml_function", "<tool_call>", "</tool_call>"),
    "qwen3_xml": _d("xml_function", "<tool_call>", "</tool_call>"),
    "mimo": _d("xml_function", "<tool_call>", "</tool_call>"),
    "step3p5": _d("xml_function", "<tool_call>", "</tool_call>"),
    "seed_oss": _d("xml_function", "<seed:tool_call>", "</seed:tool_call>"),
    "deepseek_v3": _d("deepseek_v3", DS_BEGIN, DS_END),
    "deepseek_v31": _d("deepseek_v31", DS_BEGIN, DS_END),
    "deepseek_v32": _d("xml_invoke", "<｜DSML｜function_calls>", "</｜DSML｜function_calls>"),
    "deepseek_v4": _d("xml_invoke", "<｜DSML｜function_calls>", "</｜DSML｜function_calls>"),
    "longcat": _d("json", "<longcat_tool_call>", "</longcat_tool_call>"),
    "mistral": _d("json", "[TOOL_CALLS]"),
    "granite": _d("json", ("<|tool_call|>", "<tool_call>")),
    "granite4": _d("json", "<tool_call>", "</tool_call>"),
    "granite-20b-fc": _d("json", "<function_call>"),
    "llama3_json": _d("json", ("<|python_tag|>",), bare=True),
    "llama4_json": _d("json", ("<|python_tag|>",), bare=True),
    "pythonic": _d("pythonic", (), bare=True),
    "llama4_pythonic": _d("pythonic", "<|python_start|>", "<|python_end|>", bare=True),
    "xlam": _d("json", ("<tool_call>", "[TOOL_CALLS]"), "</tool_call>", strip_fences=True, bare=True),
    "phi4_mini_json": _d("json", "functools"),
    "internlm": _d("json", "<|action_start|><|plugin|>", "<|action_end|>"),
    "jamba": _d("json", "<tool_calls>", "</tool_calls>"),
    "step3": _d("step3", "<｜tool_calls_begin｜>", "<｜tool_calls_end｜>"),
    "olmo3": _d("pythonic_lines", "<function_calls>", "</function_calls>"),
    "minicpm5": _d("json", "<|tool_call_start|>", "<|tool_call_end|>", strip_fences=True),
    "hy_v3": _d("json", "<tool_calls>", "</tool_calls>"),
    "hunyuan_a13b": _d("json", "<tool_calls>", "</tool_calls>"),
    "apertus": _d("json_fn_map", "<|tools_prefix|>", "<|tools_suffix|>"),
    "ernie45": _d("json", "<tool_call>", "</tool_call>"),
    "gigachat3": _d("json", ("<|function_call|>", "function call"), bare=False),
    "lfm2": _d("pythonic", "<|tool_call_start|>", "<|tool_call_end|>"),
    "poolside_v1": _d("json", "<tool_call>", "</tool_call>"),
    "functiongemma": _d("functiongemma", "<start_function_call>", "<end_function_call>"),
    "gemma4": _d("functiongemma", "<|tool_call>", "<tool_call|>"),
    "kimi_k2": _d("kimi", "<|tool_calls_section_begin|>", "<|tool_calls_section_end|>"),
    "glm45": _d("arg_key_value", "<tool_call>", "</tool_call>"),
    "glm47": _d("arg_key_value", "<tool_call>", "</tool_call>"),
    "minimax_m2": _d("xml_invoke", "<minimax:tool_call>", "</minimax:tool_call>"),
}

# chat-template marker -> dialect (first match wins; more specific markers first)
_DETECT = [
    ("<｜DSML｜", "deepseek_v32"), ("<｜tool▁call▁begin｜>function<｜tool▁sep｜>", "deepseek_v3"),
    ("<｜tool▁calls▁begin｜>", "deepseek_v31"), ("<|tool_calls_section_begin|>", "kimi_k2"),
    ("<minimax:tool_call>", "minimax_m2"), ("<seed:tool_call>", "seed_oss"),
    ("<longcat_tool_call>", "longcat"), ("<arg_key>", "glm45"), ("<function=", "qwen3_coder"),
    ("<start_function_call>", "functiongemma"), ("<|tools_prefix|>", "apertus"),
    ("<|action_start|>", "internlm"), ("<|python_start|>", "llama4_pythonic"),
    ("<|tool_call_start|>", "lfm2"), ("[TOOL_CALLS]", "mistral"), ("<|tool_call|>", "granite"),
    ("<function_calls>", "olmo3"), ("functools", "phi4_mini_json"), ("<tool_calls>", "hunyuan_a13b"),
    ("<|python_tag|>", "llama3_json"), ("<tool_call>", "hermes"),
]


def detect_tool_parser(chat_template: str) -> Optional[str]:
    for marker, name in _DETECT:
        if marker in (chat_template or ""):
            return name
    return None


def list_tool_parsers() -> list[str]:
    return sorted(DIALECTS)


# ------------------------------------------------------------------------------ payloads
def _dump(v) -> str:
    return json.dumps(v, ensure_ascii=False)


def _calls_from_json_value(v, d: Dialect) -> list[ToolCall]:
    items = v if isinstance(v, list) else [v]
    out = []
    for it in items:
        if not isinstance(it, dict):
            continue
        if "function" in it and isinstance(it["function"], dict):
            it = it["function"]
        name = next((it[k] for k in d.name_key if k in it), None)
        args = next((it[k] for k in d.args_key if k in it), {})
        if name is None:
            continue
        if isinstance(args, str):
            try:
                args = json.loads(args)
            except ValueError:
                pass
        out.append(ToolCall(str(name), args if isinstance(args, str) else _dump(args)))
    return out


def _json_values(text: str, partial: bool):
    """All top-level JSON values in ``text`` (separated by whitespace, ';' or ','); when
    ``partial`` the last, unfinished value is repaired by closing what is open."""
    dec = json.JSONDecoder()
    i, n, vals = 0, len(text), []
    while i < n:
        while i < n and text[i] in " \t\r\n;,":
            i += 1
        if i >= n:
            break
        if text[i] not in "{[":
            # name{...} form (mistral v11+): take the identifier as the name
            m = re.match(r"([A-Za-z_][\w.\-]*)\s*(?=\{)", text[i:])
            if not m:
                break
            try:
                v, e = dec.raw_decode(text, i + m.end())
                vals.append({"name": m.group(1), "arguments": v})
                i = e
                continue
            except ValueError:
                if partial:
                    rep = _repair(text[i + m.end():])
                    if rep is not None:
                        vals.append({"name": m.group(1), "arguments": rep})
                break
        try:
            v, e = dec.raw_decode(text, i)
            vals.append(v)
            i = e
        except ValueError:
            if partial:
                rep = _repair(text[i:])
                if rep is not None:
                    vals.append(rep)
            break
    flat = []
    for v in vals:
        flat.extend(v if isinstance(v, list) else [v])
    return flat


def _repair(s: str):
    """Best-effort parse of a JSON prefix: close open strings / arrays / objects."""
    stack, in_str, esc = [], False, False
    for ch in s:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
        elif ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append("}" if ch == "{" else "]")
        elif ch in "}]" and stack:
            stack.pop()
    t = s
    if in_str:
        t += '"'
    t = re.sub(r"[,:]\s*$", "", t.rstrip()) if not in_str else t
    for k in range(4):
        try:
            return json.loads(t + "".join(reversed(stack)))
        except ValueError:
            # drop a dangling key or half-written literal and retry
            t2 = re.sub(r',?\s*"[^"]*"?\s*:?\s*$', "", t) if k == 0 else re.sub(r"[^\[{,]*$", "", t)
            t2 = re.sub(r",\s*$", "", t2)
            if t2 == t:
                break
            t = t2
    return None


def _xml_value(raw: str):
    v = raw.strip("\n")
    try:
        return json.loads(v)
    except ValueError:
        return v


def _parse_xml_function(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<function=([^>\n]+)>(.*?)(?:</function>|\Z)", body, re.S):
        args = {}
        for pm in re.finditer(r"<parameter=([^>\n]+)>(.*?)(?:</parameter>|(?=<parameter=)|\Z)", m.group(2), re.S):
            args[pm.group(1).strip()] = _xml_value(pm.group(2))
        out.append(ToolCall(m.group(1).strip(), _dump(args)))
    return out


def _parse_xml_invoke(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<(?:｜DSML｜)?invoke name=\"([^\"]+)\">(.*?)(?:</(?:｜DSML｜)?invoke>|\Z)", body, re.S):
        args = {}
        for pm in re.finditer(r"<(?:｜DSML｜)?parameter name=\"([^\"]+)\"[^>]*>(.*?)(?:</(?:｜DSML｜)?parameter>|\Z)",
                              m.group(2), re.S):
            args[pm.group(1)] = _xml_value(pm.group(2))
        out.append(ToolCall(m.group(1), _dump(args)))
    return out


def _parse_arg_key_value(body: str, partial: bool) -> list[ToolCall]:
    head = body.lstrip()
    name = head.split("\n", 1)[0].split("<arg_key>", 1)[0].strip()
    if not name or (partial and "\n" not in head and "<arg_key>" not in head):
        return []          # the name may still be growing
    args = {}
    for m in re.finditer(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)(?:</arg_value>|\Z)", body, re.S):
        args[m.group(1).strip()] = _xml_value(m.group(2))
    return [ToolCall(name, _dump(args))]


def _py_value(node):
    return ast.literal_eval(node)


def _parse_pythonic(body: str, partial: bool) -> list[ToolCall]:
    src = body.strip()
    if not src:
        return []
    if not src.startswith("["):
        src = "[" + src + "]"
    try:
        tree = ast.parse(src, mode="eval")
    except SyntaxError:
        if not partial:
            return []
        # keep the calls that are already complete
        depth, last, in_s = 0, 0, None
        for i, ch in enumerate(src):
            if in_s:
                if ch == in_s and src[i - 1] != "\\":
                    in_s = None
            elif ch in "\"'":
                in_s = ch
            elif ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
                if depth == 1 and ch == ")":
                    last = i + 1
        if last == 0:
            return []
        try:
            tree = ast.parse(src[:last] + "]", mode="eval")
        except SyntaxError:
            return []
    calls = tree.body.elts if isinstance(tree.body, (ast.List, ast.Tuple)) else [tree.body]
    out = []
    for c in calls:
        if not isinstance(c, ast.Call):
            continue
        name = ast.unparse(c.func)
        try:
            args = {k.arg: _py_value(k.value) for k in c.keywords if k.arg}
        except (ValueError, SyntaxError):
            continue
        out.append(ToolCall(name, _dump(args)))
    return out


def _parse_pythonic_lines(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for line in body.strip().splitlines():
        out.extend(_parse_pythonic(line.strip(), partial))
    return out


def _parse_deepseek_v3(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>([^\n]+)\n```json\n(.*?)(?:\n```|\Z)", body, re.S):
        out.append(ToolCall(m.group(1).strip(), _finish_json(m.group(2), partial)))
    return out


def _parse_deepseek_v31(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)(?:<｜tool▁call▁end｜>|\Z)", body, re.S):
        out.append(ToolCall(m.group(1).strip(), _finish_json(m.group(2), partial)))
    return out


def _parse_step3(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<｜tool_call_begin｜>(?:function)?<｜tool_sep｜>(.*?)(?:<｜tool_call_end｜>|\Z)", body, re.S):
        out.extend(_parse_xml_invoke(m.group(1).replace("<steptml:", "<").replace("</steptml:", "</"), partial))
    return out


def _parse_kimi(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for m in re.finditer(r"<\|tool_call_begin\|>\s*([^\s<]+)\s*<\|tool_call_argument_begin\|>(.*?)(?:<\|tool_call_end\|>|\Z)",
                         body, re.S):
        ident = m.group(1)                       # functions.name:idx
        name = ident.split(":")[0].split(".", 1)[-1]
        out.append(ToolCall(name, _finish_json(m.group(2), partial), id=ident))
    return out


def _parse_functiongemma(body: str, partial: bool) -> list[ToolCall]:
    m = re.match(r"\s*call:([\w.\-]+)\s*\{(.*)\}?\s*$", body, re.S)
    if not m:
        return []
    args = {}
    for pm in re.finditer(r"([\w.\-]+)\s*:\s*(?:<escape>(.*?)<escape>|([^,}]+))", m.group(2), re.S):
        raw = pm.group(2) if pm.group(2) is not None else pm.group(3).strip()
        args[pm.group(1)] = raw if pm.group(2) is not None else _xml_value(raw)
    return [ToolCall(m.group(1), _dump(args))]


def _parse_json_fn_map(body: str, partial: bool) -> list[ToolCall]:
    out = []
    for it in _json_values(body, partial):
        if isinstance(it, dict):
            for k, v in it.items():
                out.append(ToolCall(k, _dump(v)))
    return out


def _finish_json(s: str, partial: bool) -> str:
    """Canonical JSON text of the first value in ``s``; trailing marker fragments are ignored
    and, when ``partial``, an unfinished value is closed provisionally."""
    s = s.strip()
    try:
        v, _ = json.JSONDecoder().raw_decode(s)
        return _dump(v)
    except ValueError:
        if partial:
            cut = s.rfind("<")
            if cut > max(s.rfind("}"), s.rfind('"'), s.rfind("]")):
                s = s[:cut]
            rep = _repair(s)
            if rep is not None:
                return _dump(rep)
        return s


_PAYLOAD = {
    "xml_function": _parse_xml_function, "xml_invoke": _parse_xml_invoke,
    "arg_key_value": _parse_arg_key_value, "pythonic": _parse_pythonic,
    "pythonic_lines": _parse_pythonic_lines, "deepseek_v3": _parse_deepseek_v3,
    "deepseek_v31": _parse_deepseek_v31, "step3": _parse_step3, "kimi": _parse_kimi,
    "functiongemma": _parse_functiongemma, "json_fn_map": _parse_json_fn_map,
}


class ToolParser:
    """One dialect bound to a request. ``extract`` parses a complete answer; ``feed`` takes the
    next piece of streamed text and returns the OpenAI-shaped deltas it completes."""

    def __init__(self, name: str):
        if name not in DIALECTS:
            raise ValueError(f"unknown tool parser {name!r}; known: {', '.join(list_tool_parsers())}")
        self.name = name
        self.d = DIALECTS[name]
        self._text = ""
        self._content_sent = 0
        self._calls_sent: list[dict] = []        # per call: {"name": bool, "args": chars sent}
        self._ids: list[str] = []

    # ------------------------------------------------------------------ whole text
    def _regions(self, text: str, partial: bool):
        """-> (content, [payload strings], tail_is_open)."""
        d = self.d
        content, payloads, pos, open_tail = [], [], 0, False
        starts = [s for s in d.start if s]
        while pos < len(text):
            nxt, mark = -1, ""
            for s in starts:
                k = text.find(s, pos)
                if k >= 0 and (nxt < 0 or k < nxt):
                    nxt, mark = k, s
            if nxt < 0:
                break
            content.append(text[pos:nxt])
            b = nxt + len(mark)
            if d.end:
                e = text.find(d.end, b)
                if e < 0:
                    payloads.append(text[b:])
                    open_tail = True
                    pos = len(text)
                    break
                payloads.append(text[b:e])
                pos = e + len(d.end)
            else:
                payloads.append(text[b:])
                open_tail = True
                pos = len(text)
        else:
            pass
        if pos < len(text):
            content.append(text[pos:])
        body = "".join(content)
        if not payloads and d.bare:
            stripped = body.strip()
            if d.strip_fences:
                stripped = re.sub(r"^```(?:json)?\s*", "", stripped)
            looks = stripped[:1] in ("{", "[") if d.kind != "pythonic" else re.match(r"\[?\s*[A-Za-z_][\w.]*\(", stripped)
            if looks:
                return "", [stripped], True
        return body, payloads, open_tail

    def _parse_payload(self, payload: str, partial: bool) -> list[ToolCall]:
        d = self.d
        p = payload
        if d.strip_fences:
            p = re.sub(r"^\s*```(?:json)?\s*|\s*```\s*$", "", p)
        if d.kind == "json":
            return _calls_from_json_value(_json_values(p.strip(), partial), d)
        return _PAYLOAD[d.kind](p, partial)

    def extract(self, text: str) -> tuple[Optional[str], list[ToolCall]]:
        content, payloads, _ = self._regions(text, False)
        calls = []
        for p in payloads:
            calls.extend(self._parse_payload(p, False))
        if not calls:
            return text, []
        content = content.strip()
        return (content or None), calls

    # ------------------------------------------------------------------ streaming
    def _holdback(self, content: str) -> int:
        """Characters at the end of ``content`` that may be the beginning of a start marker."""
        keep = 0
        for s in self.d.start:
            for k in range(min(len(s) - 1, len(content)), 0, -1):
                if content.endswith(s[:k]):
                    keep = max(keep, k)
                    break
        return keep

    def feed(self, piece: str, final: bool = False) -> list[dict]:
        """Deltas: {"content": str} or {"tool_call": {"index", "id"?, "name"?, "arguments"?}}."""
        self._text += piece
        content, payloads, open_tail = self._regions(self._text, not final)
        # payloads whose argument text is rebuilt from parsed pieces (XML-like, pythonic) only
        # grow monotonically once a call is complete: hold the open call's arguments back
        hold_last = (not final) and open_tail and self.d.kind not in ("json", "deepseek_v3", "deepseek_v31", "kimi")
        deltas = []
        calls = []
        for p in payloads:
            calls.extend(self._parse_payload(p, not final))
        if self.d.bare and not payloads and not final:
            # could still turn out to be a bare payload: hold everything while it looks like one
            s = self._text.lstrip()
            if self.d.strip_fences and "```".startswith(s[:3]) or s.startswith("```"):
                return deltas
            if s[:1] in ("{", "[") or (self.d.kind == "pythonic" and re.match(r"\[?\s*[A-Za-z_][\w.]*\(?$", s)):
                return deltas
        visible = content if final else content[: len(content) - self._holdback(content)]
        if len(visible) > self._content_sent:
            deltas.append({"content": visible[self._content_sent:]})
            self._content_sent = len(visible)
        for i, c in enumerate(calls):
            while len(self._calls_sent) <= i:
                self._calls_sent.append({"name": False, "args": 0})
                self._ids.append(c.id)
            st = self._calls_sent[i]
            is_last = i == len(calls) - 1
            if not st["name"]:
                if not final and is_last and self.d.kind == "json" and not self._name_complete(payloads, c.name):
                    continue          # the name string is still being written
                st["name"] = True
                deltas.append({"tool_call": {"index": i, "id": self._ids[i], "name": c.name, "arguments": ""}})
            if hold_last and is_last:
                continue
            args = c.arguments
            if not final and is_last:
                # the closing braces of a repaired prefix are guesses: do not stream them yet
                args = args.rstrip("}]\" ")
            sent = st.get("text", "")
            if len(args) > len(sent) and args.startswith(sent):
                deltas.append({"tool_call": {"index": i, "arguments": args[len(sent):]}})
                st["text"] = args
        return deltas

    @staticmethod
    def _name_complete(payloads: list, name: str) -> bool:
        if not name:
            return False
        q = re.escape(json.dumps(name, ensure_ascii=False))
        pat = re.compile(r'"(?:name|fn)"\s*:\s*' + q + r'\s*[,}]|' + re.escape(name) + r'\s*\{')
        return any(pat.search(p) for p in payloads)

    # ------------------------------------------------------------------ constrained decoding
    def structural_tag(self, tools: list[dict]) -> Optional[str]:
        """A lazy grammar (structural tag) that forces valid JSON arguments inside this dialect's
        tool-call markers, for the dialects whose payload is one JSON object per region."""
        d = self.d
        if d.kind != "json" or not d.start or not d.start[0] or not d.end:
            return None
        structures = []
        for t in tools:
            fn = t.get("function", t)
            structures.append({
                "begin": f'{d.start[0]}\n{{"name": "{fn["name"]}", "arguments": ',
                "schema": fn.get("parameters") or {"type": "object"},
                "end": f"}}\n{d.end}"})
        return json.dumps({"structures": structures, "triggers": [d.start[0]]})
