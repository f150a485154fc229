"""Structured output: GBNF parser + push-down matcher, JSON-schema / regex / choice front ends,
token bitmasks over a real tokenizer vocabulary, lazy structural tags, engine integration."""
import json
import random

import pytest

from vllm_cpp_b200 import _engine as E


def accepts(g, s):
    m = E.GrammarMatcher(g)
    return m.accept_string(s) and m.can_terminate()


def test_gbnf_basics():
    g = E.Grammar.from_gbnf('''
root ::= greeting " " name ("!" | "?")+
greeting ::= "hello" | "hi"   # comment
name ::= [A-Z] [a-z]{1,5}
''')
    assert accepts(g, "hello World!") and accepts(g, "hi Bob?!?")
    assert not accepts(g, "hello world!") and not accepts(g, "hi Bobbbbbbb!") and not accepts(g, "hi Bob")
    m = E.GrammarMatcher(g)
    assert m.accept_string("hi ") and not m.accept_string("x") and m.accept_string("Xy")   # failed accept keeps state
    assert not m.can_terminate() and m.accept_string("!") and m.can_terminate()
    with pytest.raises(RuntimeError):
        E.Grammar.from_gbnf("root ::= missing")
    with pytest.raises(RuntimeError):
        E.Grammar.from_gbnf('root ::= "unterminated')
    # unicode and escapes
    g = E.Grammar.from_gbnf('root ::= "caf\\u00e9 " [\\U0001F600-\\U0001F64F]+ [^a-z]')
    assert accepts(g, "café 😀😃X") and not accepts(g, "café 😀x")


def test_json_schema():
    schema = {"type": "object", "properties": {
        "name": {"type": "string"}, "age": {"type": "integer"},
        "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 2},
        "mode": {"const": "fast"}, "score": {"type": ["number", "null"]}},
        "required": ["name", "age"]}
    g = E.Grammar.from_json_schema(json.dumps(schema))
    ok = ['{"name": "x", "age": 3}', '{"name":"x","age":-12,"tags":["a","b"]}',
          '{ "name": "q\\"uote", "age": 0, "mode": "fast", "score": null }', '{"name":"x","age":1,"score":1.5e3}']
    bad = ['{"age": 3}', '{"name": "x", "age": 3.5}', '{"name":"x","age":1,"tags":["c"]}',
           '{"name":"x","age":1,"tags":["a","a","a"]}', '{"age": 1, "name": "x"}', '{"name":"x","age":1,"extra":1}']
    for s in ok:
        assert accepts(g, s), s
    for s in bad:
        assert not accepts(g, s), s
    # $ref + recursion + anyOf
    tree = {"$defs": {"node": {"type": "object", "properties": {
        "v": {"type": "integer"}, "kids": {"type": "array", "items": {"$ref": "#/$defs/node"}}},
        "required": ["v"]}}, "anyOf": [{"$ref": "#/$defs/node"}, {"type": "boolean"}]}
    g = E.Grammar.from_json_schema(json.dumps(tree))
    assert accepts(g, '{"v":1,"kids":[{"v":2},{"v":3,"kids":[]}]}') and accepts(g, "true")
    assert not accepts(g, '{"kids":[]}')
    assert accepts(E.Grammar.any_json_object(), '{"a": [1, {"b": null}], "c": "d"}')
    assert not accepts(E.Grammar.any_json_object(), '[1]')


def test_regex_and_choices():
    g = E.Grammar.from_regex(r"^\d{3}-\d{4}$")
    assert accepts(g, "555-1234") and not accepts(g, "55-1234") and not accepts(g, "555-12345")
    g = E.Grammar.from_regex(r"(yes|no)+[A-Fa-f0-9_]*\.txt")
    assert accepts(g, "yesnoyesAf_9.txt") and not accepts(g, "maybe.txt")
    g = E.Grammar.from_regex(r"[^\s,]+(, ?[^\s,]+){0,2}")
    assert accepts(g, "a,b, c") and not accepts(g, "a,b,c,d")
    g = E.Grammar.from_choices(["red", "green", 'say "hi"'])
    assert accepts(g, "green") and accepts(g, 'say "hi"') and not accepts(g, "gre")


@pytest.fixture(scope="module")
def vocab():
    from vllm_cpp_b200.loader import synthetic_tokenizer_json
    tok = E.Tokenizer.from_hf_json(synthetic_tokenizer_json(320))
    tb = [b"" if tok.is_special(i) else tok.token_bytes(i) for i in range(tok.vocab_size)]
    eos = tok.token_to_id("<|endoftext|>")
    return tok, tb, eos


def _params(**kw):
    p = E.StructuredOutputsParams()
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def _generate(mgr, st, tok, eos, rng, limit=400):
    out = []
    for _ in range(limit):
        allowed = mgr.allowed_tokens(st)
        assert allowed, "dead end"
        # prefer finishing when possible so that runs stay short
        t = eos if (eos in allowed and rng.random() < 0.3) else rng.choice(allowed)
        assert mgr.accept(st, t)
        if t == eos:
            break
        out.append(t)
    return tok.decode(out, False)


def test_token_masks_generate_valid_json(vocab):
    tok, tb, eos = vocab
    mgr = E.StructuredOutputManager(tb, 320, [eos])
    schema = {"type": "object", "properties": {"city": {"enum": ["Paris", "Rome"]},
                                               "pop": {"type": "integer"}}, "required": ["city", "pop"]}
    rng = random.Random(0)
    for _ in range(5):
        st = mgr.make_state(_params(json=json.dumps(schema)))
        assert not st.invalid
        text = _generate(mgr, st, tok, eos, rng)
        obj = json.loads(text)
        assert obj["city"] in ("Paris", "Rome") and isinstance(obj["pop"], int)
    st = mgr.make_state(_params(choice=["alpha", "beta"]))
    assert _generate(mgr, st, tok, eos, rng) in ("alpha", "beta")
    st = mgr.make_state(_params(regex=r"[a-c]{2}\d"))
    t = _generate(mgr, st, tok, eos, rng)
    assert len(t) == 3 and t[:2].strip("abc") == "" and t[2].isdigit()
    bad = mgr.make_state(_params(grammar="root ::= undefined-rule"))
    assert bad.invalid and "undefined-rule" in bad.error and mgr.allowed_tokens(bad) == [eos]
    # a token that does not fit is refused and leaves the state usable
    st = mgr.make_state(_params(choice=["alpha"]))
    wrong = tok.encode("z", False)[0]
    assert not mgr.accept(st, wrong)
    assert _generate(mgr, st, tok, eos, rng) == "alpha"


def test_lazy_structural_tag(vocab):
    tok, tb, eos = vocab
    mgr = E.StructuredOutputManager(tb, 320, [eos])
    tag = {"structures": [{"begin": "<tool_call>{\"name\": \"f\", \"arguments\": ",
                           "schema": {"type": "object", "properties": {"x": {"type": "integer"}}, "required": ["x"]},
                           "end": "}</tool_call>"}], "triggers": ["<tool_call>"]}
    st = mgr.make_state(_params(structural_tag=json.dumps(tag)))
    assert st.lazy and not st.constrained
    for t in tok.encode("free text, anything goes ", False):
        assert mgr.accept(st, t)
        assert len(mgr.allowed_tokens(st)) == 320          # unconstrained
    for t in tok.encode("<tool_call>", False):
        assert mgr.accept(st, t)
    assert st.constrained
    rng = random.Random(1)
    body = ""
    for _ in range(300):
        allowed = mgr.allowed_tokens(st)
        if not st.constrained:
            break
        t = rng.choice([a for a in allowed if a != eos] or allowed)
        assert mgr.accept(st, t)
        body += tok.decode([t], False)
    assert body.startswith('{"name": "f", "arguments": ') and body.endswith("}</tool_call>")
    args = json.loads(body[len('{"name": "f", "arguments": '):-len("}</tool_call>")])
    assert isinstance(args["x"], int)
    assert not st.constrained                                # back in free text


def test_engine_constrained_generation(tmp_path):
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-qwen3")
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ck"), cfg, seed=1)
    llm = LLM(EngineArgs(model=d, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                         max_num_seqs=4, max_num_batched_tokens=128))
    so = _params(regex=r"(cat|dog) \d\d")
    sp1 = SamplingParams(temperature=0.0, max_tokens=24, structured_outputs=so)
    sp2 = SamplingParams(temperature=1.0, seed=3, max_tokens=24, structured_outputs=_params(choice=["yes", "no"]))
    sp3 = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    outs = llm.generate(["Pick an animal:", "Answer:", "free"], [sp1, sp2, sp3])
    import re
    assert re.fullmatch(r"(cat|dog) \d\d", outs[0].outputs[0].text), outs[0].outputs[0].text
    assert outs[1].outputs[0].text in ("yes", "no")
    assert len(outs[2].outputs[0].token_ids) == 5
