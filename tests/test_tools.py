"""The small verification tools (tokenize corpus reader, container manifest, NVFP4 dequant dump, op dump)."""
import hashlib
import os

import numpy as np
import torch

from vllm_cpp_b200.entrypoints import tools


def test_corpus_reader_escapes_and_comments(tmp_path):
    p = tmp_path / "corpus.txt"
    p.write_bytes(b"# a comment\nplain\n\ntab\\there\\nnewline\nback\\\\slash\n")
    assert tools.read_corpus(str(p)) == ["plain", "", "tab\there\nnewline", "back\\slash"]


def test_corpus_reader_rejects_unknown_escape(tmp_path):
    p = tmp_path / "c.txt"
    p.write_text("bad\\q\n")
    try:
        tools.read_corpus(str(p))
    except ValueError as e:
        assert "bad escape" in str(e)
    else:
        raise AssertionError("an unknown escape must fail loudly")


def test_tokenize_prints_ids_and_empty(tmp_path, capsys):
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    import json
    import ref_assets
    tj = tmp_path / "tokenizer.json"
    tj.write_text(ref_assets.tokenizer_json(512))
    c = tmp_path / "c.txt"
    c.write_text("123\n\n")
    assert tools.main(["tokenize", str(tj), str(c)]) == 0
    lines = capsys.readouterr().out.strip().split("\n")
    assert len(lines) == 2 and lines[1] == "EMPTY"
    assert len(lines[0].split()) == 3


def test_dump_container_manifest(tmp_path, capsys):
    from vllm_cpp_b200.loader.safetensors import save_file
    a = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    b = torch.ones(5, dtype=torch.bfloat16)
    path = str(tmp_path / "m.safetensors")
    save_file({"z.weight": a, "a.bias": b}, path)
    lines = tools.manifest_lines(path)
    assert lines[-1] == "TOTAL 2 tensors"
    assert lines[0].startswith("a.bias BF16 [5] 10 ") and lines[1].startswith("z.weight F32 [3,4] 48 ")
    assert lines[1].split()[-1] == hashlib.sha256(a.numpy().tobytes()).hexdigest()


def test_dequant_nvfp4_dump_matches_reference(tmp_path, capsys):
    from vllm_cpp_b200.loader.safetensors import save_file
    from vllm_cpp_b200.ops.quant import ref_dequant_nvfp4, ref_quant_nvfp4_weights
    w = torch.randn(32, 64, generator=torch.Generator().manual_seed(1))
    packed, sf, g = ref_quant_nvfp4_weights(w)
    path = str(tmp_path / "q.safetensors")
    save_file({"w": packed, "s": sf.view(torch.float8_e4m3fn), "g": g}, path)
    out = str(tmp_path / "w.raw")
    assert tools.main(["dequant-nvfp4", path, "w", "s", "g", out]) == 0
    assert capsys.readouterr().out.split() == ["32", "64"]
    got = torch.from_numpy(np.fromfile(out, dtype="<i2")).view(torch.bfloat16).reshape(32, 64)
    want = ref_dequant_nvfp4(packed, sf, g).to(torch.bfloat16)
    assert torch.equal(got, want)
    assert (got.float() - w).abs().max() < 0.6          # fp4 grid: coarse but bounded


def test_dump_ops_writes_inputs_and_oracle_outputs(tmp_path):
    out = str(tmp_path / "ops.npz")
    assert tools.main(["dump-ops", out]) == 0
    z = np.load(out)
    assert {"rmsnorm.x", "rmsnorm.out", "gemm.out", "argmax.out", "silu_and_mul.out"} <= set(z.files)
    np.testing.assert_allclose(z["gemm.out"], z["gemm.a"] @ z["gemm.w"].T, rtol=1e-4, atol=1e-4)
    assert (z["argmax.out"] == z["argmax.logits"].argmax(-1)).all()
