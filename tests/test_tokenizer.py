"""The native tokenizer / detokenizer against Hugging Face `tokenizers` on tokenizers trained
here (no network): byte-exact pre-token splits, ids and decoded text for every regex family
and for the SentencePiece-style byte-fallback layout."""
import json
import random

import pytest

tokenizers = pytest.importorskip("tokenizers")
from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, processors, trainers  # noqa: E402

from vllm_cpp_b200 import _engine as E  # noqa: E402

GPT2 = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
LLAMA3 = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
QWEN2 = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
QWEN35 = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?[\p{L}\p{M}]+|\p{N}| ?[^\s\p{L}\p{M}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
DS3 = [r"\p{N}{1,3}", r"[一-龥぀-ゟ゠-ヿ]+",
       r"""[!"#$%&'()*+,\-./:;<=>?@\[\\\]^_`{|}~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""]

CORPUS = [
    "The quick brown fox jumps over the lazy dog. It's 2024, isn't it? I'LL say: we've 12345 apples!",
    "def f(x):\n    return x**2 + 3.14159  # comment\n\n\nclass A:\r\n\tpass",
    "Ünïcödé çhåracters: naïve café, Straße, Ελληνικά, русский язык, العربية, हिन्दी, 日本語のテキスト、中文字符。",
    "emoji 🙂🙃 👩‍👩‍👧‍👦 flags 🇺🇳, math ∑∫√∞ ≠ ≤, currency €£¥₹, combining e\u0301 a\u0308\u0323",
    "   leading spaces,  double  spaces   and trailing   ",
    "tabs\tand\nnewlines\n\n  mixed \n \n\t\n end",
    "numbers 1 22 333 4444 55555 666666 1,000,000 3.5e-7 ０１２ ⅓ Ⅷ",
    "URL https://example.com/a_b?c=d&e=f#g and e-mail someone@example.org",
    "<|im_start|>user\nHello<|im_end|>\n<|im_start|>assistant\n",
    "한국어 텍스트와 English mixed 中英文 mixed123text",
    "don't DON'T Don'T we're WE'RE y'all'd've 'quoted' ''double''",
    "\u00a0nbsp\u2003emspace\u3000ideographic\u200bzero-width",
]

PROBES = CORPUS + [
    "", " ", "  ", "\n", " \n", "a", " a", "a ", "a  b", "'s", "'S", "x's y'T", "1234567", " 12 345",
    "!!!", " !!!\n\n", "a\r\nb", "\r\n\r\n", "   \n   x", "end.  \n", "ß", "ſ's", "e\u0301", "\u0301abc",
    "🙂", "a🙂b", "日本語", "3日後", "#hashtag @user $var %d", "x=1;y=2", "  \t ", "\x00\x01ctl",
]


def _train(pre, decoder, normalizer=None, byte_fallback=False, specials=(), post=None, vocab=600,
           ignore_merges=False, alphabet=None):
    model = models.BPE(byte_fallback=byte_fallback, unk_token="<unk>" if byte_fallback else None,
                       ignore_merges=ignore_merges)
    tk = Tokenizer(model)
    if normalizer is not None:
        tk.normalizer = normalizer
    if pre is not None:
        tk.pre_tokenizer = pre
    tk.decoder = decoder
    sp = list(specials)
    if byte_fallback:
        sp = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + sp
    tr = trainers.BpeTrainer(vocab_size=vocab + len(sp), special_tokens=sp, show_progress=False,
                             initial_alphabet=alphabet or [])
    tk.train_from_iterator(CORPUS * 3, tr)
    if post is not None:
        tk.post_processor = post(tk)
    return tk


def _byte_level(patterns, **kw):
    if patterns is None:
        pre = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        seq = [pre_tokenizers.Split(Regex(p), behavior="isolated") for p in patterns]
        pre = pre_tokenizers.Sequence(seq + [pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    return _train(pre, decoders.ByteLevel(), alphabet=pre_tokenizers.ByteLevel.alphabet(),
                  specials=["<|endoftext|>", "<|im_start|>", "<|im_end|>"], **kw)


FAMILIES = {
    "gpt2": (None, E.PreFamily.GPT2),
    "llama3": ([LLAMA3], E.PreFamily.LLAMA3),
    "qwen2": ([QWEN2], E.PreFamily.QWEN2),
    "qwen35": ([QWEN35], E.PreFamily.QWEN35),
    "deepseek_v3": (DS3, E.PreFamily.DEEPSEEK_V3),
}


@pytest.fixture(scope="module", params=list(FAMILIES))
def pair(request):
    patterns, fam = FAMILIES[request.param]
    hf = _byte_level(patterns)
    mine = E.Tokenizer.from_hf_json(hf.to_str())
    assert mine.family == fam
    return hf, mine, patterns, fam


def test_pretokenizer_splits_match(pair):
    hf, mine, patterns, fam = pair
    if patterns is None:
        splitter = pre_tokenizers.Split(Regex(GPT2), behavior="isolated")
    else:
        splitter = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(p), behavior="isolated") for p in patterns])
    for text in PROBES:
        want = [p for p, _ in splitter.pre_tokenize_str(text)]
        got = [p.decode("utf-8") for p in E.pretokenize(fam, text)]
        assert got == want, (text, got, want)


def test_encode_decode_match(pair):
    hf, mine, _, _ = pair
    rng = random.Random(0)
    pool = "".join(CORPUS)
    probes = list(PROBES)
    for _ in range(200):
        a = rng.randrange(len(pool))
        probes.append(pool[a:a + rng.randrange(1, 60)])
    for text in probes:
        want = hf.encode(text).ids
        got = mine.encode(text)
        assert got == want, (text, got, want)
        assert mine.decode(got, False) == hf.decode(want, skip_special_tokens=False)
        assert mine.decode(got, True) == hf.decode(want, skip_special_tokens=True)


def test_special_tokens_and_ignore_merges():
    hf = _byte_level([LLAMA3], ignore_merges=True,
                     post=lambda tk: processors.TemplateProcessing(
                         single="<|im_start|> $A", special_tokens=[("<|im_start|>", tk.token_to_id("<|im_start|>"))]))
    mine = E.Tokenizer.from_hf_json(hf.to_str())
    assert mine.adds_bos
    for text in PROBES:
        assert mine.encode(text) == hf.encode(text).ids, text
        assert mine.encode(text, False) == hf.encode(text, add_special_tokens=False).ids, text
    ids = mine.encode("<|im_start|>user<|im_end|>")
    assert mine.is_special(ids[0]) and mine.token_to_id("<|im_end|>") in ids


def _sentencepiece_style():
    norm = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    dec = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(),
                             decoders.Strip(" ", 1, 0)])
    return _train(None, dec, normalizer=norm, byte_fallback=True, vocab=500,
                  post=lambda tk: processors.TemplateProcessing(single="<s> $A", special_tokens=[("<s>", 1)]))


def test_sentencepiece_style_byte_fallback():
    hf = _sentencepiece_style()
    cfg = json.dumps({"bos_token": "<s>", "eos_token": {"content": "</s>"}, "unk_token": "<unk>"})
    mine = E.Tokenizer.from_hf_json(hf.to_str(), cfg)
    assert (mine.bos_id, mine.eos_id, mine.family) == (1, 2, E.PreFamily.NONE)
    for text in PROBES + ["unseen: ξ ж 🦙 \u4e2d"]:
        want = hf.encode(text).ids
        assert mine.encode(text) == want, (text, mine.encode(text), want)
        assert mine.decode(want, True) == hf.decode(want, skip_special_tokens=True), text


def test_metaspace_style():
    pre = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="first")
    hf = _train(pre, decoders.Metaspace(replacement="▁", prepend_scheme="first"), byte_fallback=True, vocab=500)
    mine = E.Tokenizer.from_hf_json(hf.to_str())
    for text in [p for p in PROBES if p.strip()]:
        want = hf.encode(text).ids
        assert mine.encode(text) == want, (text, mine.encode(text), want)


def test_gguf_vocab_round_trip():
    hf = _byte_level([QWEN2])
    j = json.loads(hf.to_str())
    vocab = j["model"]["vocab"]
    n = max(max(vocab.values()), max(a["id"] for a in j["added_tokens"])) + 1
    tokens = [b""] * n
    types = [1] * n
    for t, i in vocab.items():
        tokens[i] = t.encode()
    for a in j["added_tokens"]:
        tokens[a["id"]] = a["content"].encode()
        types[a["id"]] = 3
    merges = [(m if isinstance(m, str) else " ".join(m)).encode() for m in j["model"]["merges"]]
    mine = E.Tokenizer.from_gguf("gpt2", "qwen2", tokens, merges, types, -1, 0, False, False)
    for text in PROBES:
        assert mine.encode(text) == hf.encode(text).ids, text


@pytest.mark.parametrize("style", ["byte_level", "sentencepiece"])
def test_incremental_detokenizer_streams_exact_text(style):
    hf = _byte_level([LLAMA3]) if style == "byte_level" else _sentencepiece_style()
    mine = E.Tokenizer.from_hf_json(hf.to_str())
    for text in CORPUS + ["🙂🙃🦙 ends with emoji 👩‍👩‍👧‍👦"]:
        ids = mine.encode(text, False)
        prompt = mine.encode("Prompt text before.", False)
        d = E.IncrementalDetokenizer(mine, prompt, True, [], False, 0)
        deltas = []
        for i in ids:
            assert d.update([i], False) is None
            piece = d.get_next_output_text(False, True)
            assert "\ufffd" not in piece
            deltas.append(piece)
        full = d.get_next_output_text(True, False)
        assert "".join(deltas) == full
        want = mine.decode(prompt + ids, True)[len(mine.decode(prompt, True)):]
        assert full == want, (text, full, want)


def test_detokenizer_stop_strings_hold_back_and_truncate():
    hf = _byte_level([LLAMA3])
    mine = E.Tokenizer.from_hf_json(hf.to_str())
    ids = mine.encode("The quick brown fox jumps over the lazy dog", False)
    d = E.IncrementalDetokenizer(mine, [], True, ["lazy", "never-there"], False, 0)
    seen, stop = "", None
    for i in ids:
        stop = d.update([i], False)
        if stop is not None:
            break
        seen += d.get_next_output_text(False, True)
        assert "lazy" not in seen and "laz" not in seen[-3:]
    assert stop == "lazy"
    seen += d.get_next_output_text(True, True)
    assert seen == "The quick brown fox jumps over the "
    assert d.output_text == seen
    # include_stop_str_in_output keeps the stop string and nothing after it
    d2 = E.IncrementalDetokenizer(mine, [], True, ["lazy"], True, 0)
    assert d2.update(ids, False) == "lazy"
    assert d2.get_next_output_text(True, False) == "The quick brown fox jumps over the lazy"
    # min_tokens: text produced before the threshold is not searched
    d3 = E.IncrementalDetokenizer(mine, [], True, ["quick"], False, len(ids) + 1)
    assert d3.update(ids, False) is None
    # stop-terminated: the final (EOS-like) token produces no text
    d4 = E.IncrementalDetokenizer(mine, [], True, [], False, 0)
    d4.update(ids + [mine.token_to_id("<|endoftext|>")], True)
    assert d4.get_next_output_text(True, False) == "The quick brown fox jumps over the lazy dog"
    assert d4.num_output_tokens == len(ids) + 1
