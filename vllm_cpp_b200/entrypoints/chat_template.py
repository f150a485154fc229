"""Chat templating: renders OpenAI-style messages (+ tools) to a prompt with the model's own
Jinja template, with a ChatML fallback and a Hermes-style tool preamble when the template
ignores ``tools``.

Reference: ``src/vllm/entrypoints/chat_template.cpp`` (probe render + Hermes-aware fallback;
the reference embeds the minja engine, here the sandboxed jinja2 environment is used).
"""
from __future__ import annotations

import datetime
import json
from typing import Optional

CHATML = ("{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
          "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")

_HERMES_TOOLS = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                 "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n{tools}\n</tools>\n\n"
                 "For each function call, return a json object with function name and arguments within "
                 "<tool_call></tool_call> XML tags:\n<tool_call>\n{{\"name\": <function-name>, \"arguments\": <args-json-object>}}\n</tool_call>")


def _env():
    import jinja2
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(msg):
        raise jinja2.exceptions.TemplateError(msg)

    def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                        extensions=["jinja2.ext.loopcontrols"])
    env.filters["tojson"] = tojson
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    return env


def _normalise(messages: list[dict]) -> list[dict]:
    out = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):          # content parts -> text
            m["content"] = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") == "text")
        elif c is None:
            m["content"] = ""
        for tc in m.get("tool_calls") or []:
            fn = tc.get("function", {})
            if isinstance(fn.get("arguments"), str):
                try:
                    fn["arguments"] = json.loads(fn["arguments"])
                except ValueError:
                    pass
        out.append(m)
    return out


class ChatTemplate:
    def __init__(self, template: Optional[str] = None, bos_token: str = "", eos_token: str = ""):
        self.source = template or CHATML
        self.is_fallback = template is None
        self.bos_token, self.eos_token = bos_token, eos_token
        self._tpl = _env().from_string(self.source)
        self._tools_aware = "tools" in self.source

    def render(self, messages: list[dict], tools: Optional[list] = None, add_generation_prompt: bool = True,
               **kwargs) -> str:
        msgs = _normalise(messages)
        if tools and not self._tools_aware:
            # the template would drop the tools silently: describe them in a system message
            block = _HERMES_TOOLS.format(tools="\n".join(json.dumps(t, ensure_ascii=False) for t in tools))
            if msgs and msgs[0]["role"] == "system":
                msgs[0] = dict(msgs[0], content=msgs[0]["content"] + "\n\n" + block)
            else:
                msgs.insert(0, {"role": "system", "content": block})
        return self._tpl.render(messages=msgs, tools=tools or None, add_generation_prompt=add_generation_prompt,
                                bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)

    def probe(self) -> bool:
        """A test render with a plain exchange: False means the template cannot be used."""
        try:
            self.render([{"role": "user", "content": "ping"}])
            return True
        except Exception:
            return False

    def ends_in_reasoning(self) -> bool:
        """Does the generation prompt leave the model inside a <think> span?"""
        try:
            p = self.render([{"role": "user", "content": "x"}])
        except Exception:
            return False
        tail = p[-32:]
        return "<think>" in tail and "</think>" not in tail
