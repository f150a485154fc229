"""Tool-call / reasoning parsers, chat templating and the OpenAI server (CPU, tiny model)."""
import http.client
import json
import threading

import pytest

from vllm_cpp_b200.entrypoints.chat_template import ChatTemplate
from vllm_cpp_b200.entrypoints.reasoning_parsers import ReasoningParser, detect_reasoning_parser, list_reasoning_parsers
from vllm_cpp_b200.entrypoints.tool_parsers import DIALECTS, ToolParser, detect_tool_parser, list_tool_parsers

ARGS = {"city": "Paris", "days": 3}
AJ = json.dumps(ARGS)

SAMPLES = {
    "hermes": 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": %s}\n</tool_call>' % AJ,
    "qwen3": '<tool_call>\n{"name": "get_weather", "arguments": %s}\n</tool_call>' % AJ,
    "qwen3_coder": '<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>',
    "seed_oss": '<seed:tool_call>\n<function=get_weather>\n<parameter=city>Paris</parameter>\n<parameter=days>3</parameter>\n</function>\n</seed:tool_call>',
    "deepseek_v3": '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n%s\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>' % AJ,
    "deepseek_v31": '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>get_weather<｜tool▁sep｜>%s<｜tool▁call▁end｜><｜tool▁calls▁end｜>' % AJ,
    "deepseek_v32": '<｜DSML｜function_calls>\n<｜DSML｜invoke name="get_weather">\n<｜DSML｜parameter name="city" string="true">Paris</｜DSML｜parameter>\n<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜function_calls>',
    "longcat": '<longcat_tool_call>{"name": "get_weather", "arguments": %s}</longcat_tool_call>' % AJ,
    "mistral": '[TOOL_CALLS][{"name": "get_weather", "arguments": %s}]' % AJ,
    "granite": '<|tool_call|>[{"name": "get_weather", "arguments": %s}]' % AJ,
    "granite-20b-fc": '<function_call> {"name": "get_weather", "arguments": %s}' % AJ,
    "llama3_json": '{"name": "get_weather", "parameters": %s}' % AJ,
    "llama4_json": '<|python_tag|>{"name": "get_weather", "parameters": %s}' % AJ,
    "pythonic": '[get_weather(city="Paris", days=3)]',
    "llama4_pythonic": '<|python_start|>[get_weather(city="Paris", days=3)]<|python_end|>',
    "xlam": '```json\n[{"name": "get_weather", "arguments": %s}]\n```' % AJ,
    "phi4_mini_json": 'functools[{"name": "get_weather", "arguments": %s}]' % AJ,
    "internlm": 'I will call.<|action_start|><|plugin|>\n{"name": "get_weather", "parameters": %s}<|action_end|>' % AJ,
    "jamba": '<tool_calls>[{"name": "get_weather", "arguments": %s}]</tool_calls>' % AJ,
    "hunyuan_a13b": '<tool_calls>[{"name": "get_weather", "arguments": %s}]</tool_calls>' % AJ,
    "olmo3": '<function_calls>\nget_weather(city="Paris", days=3)\n</function_calls>',
    "apertus": '<|tools_prefix|>[{"get_weather": %s}]<|tools_suffix|>' % AJ,
    "lfm2": '<|tool_call_start|>[get_weather(city="Paris", days=3)]<|tool_call_end|>',
    "functiongemma": '<start_function_call>call:get_weather{city:<escape>Paris<escape>,days:3}<end_function_call>',
    "kimi_k2": '<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>%s<|tool_call_end|><|tool_calls_section_end|>' % AJ,
    "glm45": '<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>',
    "minimax_m2": '<minimax:tool_call>\n<invoke name="get_weather">\n<parameter name="city">Paris</parameter>\n<parameter name="days">3</parameter>\n</invoke>\n</minimax:tool_call>',
    "step3": '<｜tool_calls_begin｜><｜tool_call_begin｜>function<｜tool_sep｜><steptml:invoke name="get_weather"><steptml:parameter name="city">Paris</steptml:parameter><steptml:parameter name="days">3</steptml:parameter></steptml:invoke><｜tool_call_end｜><｜tool_calls_end｜>',
}


def test_every_dialect_of_the_inventory_exists():
    names = set(list_tool_parsers())
    for n in ("hermes qwen3 qwen3_coder qwen3_xml mimo deepseek_v3 deepseek_v31 deepseek_v32 deepseek_v4 longcat "
              "mistral granite granite4 granite-20b-fc llama3_json llama4_json pythonic llama4_pythonic xlam "
              "phi4_mini_json internlm jamba step3 step3p5 olmo3 minicpm5 hy_v3 hunyuan_a13b apertus ernie45 "
              "gigachat3 lfm2 poolside_v1 functiongemma kimi_k2 glm45 glm47 minimax_m2 gemma4 seed_oss").split():
        assert n in names, n
    assert len(names) >= 39
    assert set(list_reasoning_parsers()) == {"think_auto", "basic", "deepseek_r1", "mistral", "minimax_m2", "step3", "olmo3"}


@pytest.mark.parametrize("name", sorted(SAMPLES))
def test_tool_parser_extract_and_stream(name):
    text = SAMPLES[name]
    content, calls = ToolParser(name).extract(text)
    assert len(calls) == 1, (name, content, calls)
    assert calls[0].name == "get_weather" and json.loads(calls[0].arguments) == ARGS
    if name in ("hermes", "internlm"):
        assert content and "<" not in content
    # streamed three characters at a time: the same call, and no marker text leaks as content
    p = ToolParser(name)
    got_name, args, shown = None, "", ""
    for i in range(0, len(text), 3):
        for d in p.feed(text[i:i + 3], final=False):
            if "content" in d:
                shown += d["content"]
            else:
                tc = d["tool_call"]
                got_name = tc.get("name", got_name)
                args += tc.get("arguments", "")
    for d in p.feed("", final=True):
        if "content" in d:
            shown += d["content"]
        else:
            args += d["tool_call"].get("arguments", "")
            got_name = d["tool_call"].get("name", got_name)
    assert got_name == "get_weather", name
    assert json.loads(args) == ARGS, (name, args)
    for s in DIALECTS[name].start:
        assert not s or s not in shown


def test_plain_text_passes_through_and_multiple_calls():
    p = ToolParser("hermes")
    assert p.extract("just an answer") == ("just an answer", [])
    two = ('<tool_call>{"name": "a", "arguments": {}}</tool_call>\n<tool_call>{"name": "b", "arguments": {"x": 1}}</tool_call>')
    _, calls = ToolParser("hermes").extract(two)
    assert [c.name for c in calls] == ["a", "b"]
    _, calls = ToolParser("pythonic").extract('[f(x=1), g(y="s", z=[1, 2])]')
    assert [c.name for c in calls] == ["f", "g"] and json.loads(calls[1].arguments) == {"y": "s", "z": [1, 2]}
    assert detect_tool_parser("...<tool_call>...") == "hermes"
    assert detect_tool_parser("{{ '[TOOL_CALLS]' }}") == "mistral"
    assert detect_tool_parser("<｜tool▁calls▁begin｜>") == "deepseek_v31"
    tag = json.loads(ToolParser("hermes").structural_tag([{"type": "function", "function": {
        "name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}}}}]))
    assert tag["triggers"] == ["<tool_call>"] and tag["structures"][0]["begin"].startswith("<tool_call>")


def test_reasoning_parsers():
    r, c = ReasoningParser("basic").extract("<think>step 1\nstep 2</think>\nanswer")
    assert (r, c) == ("step 1\nstep 2", "answer")
    assert ReasoningParser("basic").extract("no tags") == (None, "no tags")
    assert ReasoningParser("deepseek_r1").extract("thinking...</think>final") == ("thinking...", "final")
    assert ReasoningParser("deepseek_r1").extract("still thinking") == ("still thinking", None)
    assert ReasoningParser("mistral").extract("[THINK]hm[/THINK]ok") == ("hm", "ok")
    # streaming, two characters at a time
    for name, text, want in (("think_auto", "<think>abc</think>answer", ("abc", "answer")),
                             ("deepseek_r1", "abc</think>answer", ("abc", "answer")),
                             ("mistral", "pre[THINK]abc[/THINK]answer", ("abc", "preanswer"))):
        p = ReasoningParser(name)
        r = c = ""
        for i in range(0, len(text), 2):
            for d in p.feed(text[i:i + 2], final=i + 2 >= len(text)):
                r += d.get("reasoning_content", "")
                c += d.get("content", "")
        assert (r, c) == want, name
    assert detect_reasoning_parser("{{ '[THINK]' }}") == "mistral"
    assert detect_reasoning_parser("plain") is None


def test_chat_template():
    t = ChatTemplate(None)
    p = t.render([{"role": "system", "content": "be brief"}, {"role": "user", "content": [{"type": "text", "text": "hi"}]}])
    assert p == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]
    p = t.render([{"role": "user", "content": "hi"}], tools=tools)
    assert "<tools>" in p and '"name": "f"' in p           # tools are not dropped silently
    custom = ChatTemplate("{{ bos_token }}{% for m in messages %}[{{ m.role }}] {{ m.content }}\n{% endfor %}"
                          "{% if tools %}T={{ tools | tojson }}{% endif %}{% if add_generation_prompt %}<think>\n{% endif %}",
                          bos_token="<s>")
    assert custom.render([{"role": "user", "content": "x"}], tools=tools).startswith("<s>[user] x\nT=[{")
    assert custom.ends_in_reasoning() and not t.ends_in_reasoning()
    assert not ChatTemplate("{{ raise_exception('no') }}").probe()


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM
    from vllm_cpp_b200.entrypoints.api_server import ServerState, make_server
    cfg = synthetic_config("tiny-qwen3")
    d = loader.write_synthetic_checkpoint(str(tmp_path_factory.mktemp("m") / "ck"), cfg, seed=2)
    llm = LLM(EngineArgs(model=d, device="cpu", block_size=16, num_blocks=128, max_model_len=256,
                         max_num_seqs=8, max_num_batched_tokens=128))
    state = ServerState(llm, "tiny", tool_parser="hermes", default_max_tokens=8)
    srv = make_server(state, "127.0.0.1", 0)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    yield srv.server_address[1], state
    srv.shutdown()
    state.engine.shutdown()


def _req(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request(method, path, json.dumps(body) if body is not None else None, {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode("utf-8")
    c.close()
    return r.status, data


def test_server_routes(server):
    port, _ = server
    assert _req(port, "GET", "/health")[0] == 200
    st, body = _req(port, "GET", "/v1/models")
    assert st == 200 and json.loads(body)["data"][0]["id"] == "tiny"
    assert "version" in json.loads(_req(port, "GET", "/version")[1])
    st, body = _req(port, "POST", "/v1/completions", {"prompt": "The quick brown", "max_tokens": 6, "temperature": 0})
    o = json.loads(body)
    assert st == 200 and o["object"] == "text_completion" and o["usage"]["completion_tokens"] <= 6
    assert isinstance(o["choices"][0]["text"], str) and o["choices"][0]["finish_reason"] in ("length", "stop")
    # deterministic with temperature 0
    assert json.loads(_req(port, "POST", "/v1/completions", {"prompt": "The quick brown", "max_tokens": 6,
                                                            "temperature": 0})[1])["choices"][0]["text"] == o["choices"][0]["text"]
    st, body = _req(port, "POST", "/v1/completions", {"prompt": [[1, 2, 3], [4, 5]], "max_tokens": 3, "n": 2})
    assert st == 200 and len(json.loads(body)["choices"]) == 4
    st, body = _req(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hello"}],
                                                           "max_tokens": 5, "guided_choice": ["yes", "no"]})
    o = json.loads(body)
    assert st == 200 and o["choices"][0]["message"]["content"] in ("yes", "no")
    st, body = _req(port, "POST", "/tokenize", {"prompt": "hello world"})
    toks = json.loads(body)["tokens"]
    assert json.loads(_req(port, "POST", "/detokenize", {"tokens": toks})[1])["prompt"] == "hello world"
    assert "vllm:requests_total" in _req(port, "GET", "/metrics")[1]
    # errors
    st, body = _req(port, "POST", "/v1/completions", {"max_tokens": 3})
    assert st == 400 and json.loads(body)["error"]["type"] == "invalid_request_error"
    assert _req(port, "POST", "/v1/completions", {"prompt": "x", "temperature": -1})[0] == 400
    assert _req(port, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
    assert _req(port, "GET", "/nope")[0] == 404
    assert _req(port, "POST", "/v1/completions", {"prompt": "x", "guided_grammar": "root ::= oops"})[0] == 400


def test_server_streaming(server):
    port, _ = server
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request("POST", "/v1/chat/completions", json.dumps({
        "messages": [{"role": "user", "content": "count"}], "max_tokens": 6, "temperature": 0, "stream": True,
        "stream_options": {"include_usage": True}}), {"Content-Type": "application/json"})
    r = c.getresponse()
    assert r.status == 200 and r.getheader("Content-Type").startswith("text/event-stream")
    events = [l[6:] for l in r.read().decode("utf-8").split("\n\n") if l.startswith("data: ")]
    c.close()
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks if ch["choices"])
    fins = [ch["choices"][0]["finish_reason"] for ch in chunks if ch["choices"] and ch["choices"][0]["finish_reason"]]
    assert fins and fins[-1] in ("length", "stop")
    assert chunks[-1]["usage"]["completion_tokens"] <= 6
    # the non-streaming answer is the same text
    st, body = _req(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "count"}],
                                                           "max_tokens": 6, "temperature": 0})
    assert json.loads(body)["choices"][0]["message"]["content"] == text


def test_server_with_tensor_parallel_workers(tmp_path):
    """``--tensor-parallel-size 2``: this process is rank 0 (scheduler + HTTP), a child process is
    rank 1 and only runs the published steps. Same completions as the single-rank server, and a
    lost worker turns into EngineDeadError on the host instead of a hang. CPU ranks over gloo."""
    import time

    from vllm_cpp_b200 import _engine as E
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import EngineArgs, ParallelConfig, synthetic_config
    from vllm_cpp_b200.entrypoints.api_server import ServerState, make_server
    from vllm_cpp_b200.parallel.launch import launch_engine
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ck"), synthetic_config("tiny-qwen3"), seed=5)

    def serve(tp):
        args = EngineArgs(model=d, device="cpu", block_size=16, num_blocks=128, max_model_len=256, max_num_seqs=8,
                          max_num_batched_tokens=128, parallel=ParallelConfig(tensor_parallel_size=tp))
        llm, workers = launch_engine(args)
        state = ServerState(llm, "tiny", tool_parser="hermes", default_max_tokens=8)
        srv = make_server(state, "127.0.0.1", 0)
        threading.Thread(target=srv.serve_forever, daemon=True).start()
        return llm, workers, state, srv

    body = {"prompt": "The quick brown", "max_tokens": 8, "temperature": 0}
    llm1, _, st1, srv1 = serve(1)
    want = json.loads(_req(srv1.server_address[1], "POST", "/v1/completions", body)[1])["choices"][0]["text"]
    srv1.shutdown()
    st1.engine.shutdown()

    llm2, workers, st2, srv2 = serve(2)
    try:
        assert workers is not None and len(workers.procs) == 1
        code, out = _req(srv2.server_address[1], "POST", "/v1/completions", body)
        assert code == 200 and json.loads(out)["choices"][0]["text"] == want
        # a sampled request exercises the sampler-input message to the worker
        code, out = _req(srv2.server_address[1], "POST", "/v1/completions",
                         {"prompt": "abc", "max_tokens": 4, "temperature": 0.7, "seed": 3, "presence_penalty": 0.5})
        assert code == 200
        # the worker dies between steps: the host notices, the next step raises
        workers.procs[0].kill()
        t0 = time.time()
        while workers.failed is None and time.time() - t0 < 10:
            time.sleep(0.1)
        assert workers.failed and "rank 1" in workers.failed
        llm2.add_request([1, 2, 3], E.SamplingParams(max_tokens=2))
        with pytest.raises(E.EngineDeadError):
            llm2.step()
    finally:
        srv2.shutdown()
        st2.engine.shutdown()
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def test_data_parallel_replicas_behind_one_server(tmp_path):
    """Two engine replicas behind one server: concurrent requests are spread over both, every answer
    equals the single-engine answer, and a streamed request stays on its replica."""
    from concurrent.futures import ThreadPoolExecutor
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM
    from vllm_cpp_b200.entrypoints.api_server import ServerState, make_server
    cfg = synthetic_config("tiny-qwen3")
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ck"), cfg, seed=2)
    mk = lambda: LLM(EngineArgs(model=d, device="cpu", block_size=16, num_blocks=128, max_model_len=256,
                                max_num_seqs=8, max_num_batched_tokens=128))
    state = ServerState(mk(), "tiny", default_max_tokens=8, replicas=[mk()])
    srv = make_server(state, "127.0.0.1", 0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    port = srv.server_address[1]
    try:
        prompts = [f"prompt number {i} says" for i in range(8)]
        body = lambda p: {"prompt": p, "max_tokens": 6, "temperature": 0}
        with ThreadPoolExecutor(8) as ex:
            got = list(ex.map(lambda p: json.loads(_req(port, "POST", "/v1/completions", body(p))[1]), prompts))
        assert all(g["object"] == "text_completion" for g in got)
        assert min(state.engine.routed) >= 1 and sum(state.engine.routed) == 8
        # one at a time afterwards: same text whichever replica answers
        again = [json.loads(_req(port, "POST", "/v1/completions", body(p))[1]) for p in prompts[:3]]
        assert [g["choices"][0]["text"] for g in again] == [g["choices"][0]["text"] for g in got[:3]]
        assert state.engine._inflight == [0, 0] and not state.engine._where
        assert _req(port, "GET", "/health")[0] == 200
    finally:
        srv.shutdown()
        state.engine.shutdown()
