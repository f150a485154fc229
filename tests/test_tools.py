"""Bench harness and CLI on a tiny CPU model."""
import json

from vllm_cpp_b200.entrypoints import bench_serve, cli


def test_bench_serve_closed_loop(capsys, tmp_path):
    out = tmp_path / "ids.json"
    rc = bench_serve.main(["--shape", "tiny-dense", "--device", "cpu", "--num-prompts", "6", "--input-len", "20",
                           "--output-len", "5", "--concurrency", "3", "--num-blocks", "64",
                           "--output-token-ids", str(out)])
    assert rc == 0
    res = json.loads(capsys.readouterr().out)
    assert res["completed"] == 6 and res["failed"] == 0
    assert res["total_output_tokens"] == 30 and res["total_input_tokens"] == 120
    assert res["output_throughput"] > 0 and res["ttft"]["mean_ms"] > 0 and res["tpot"]["median_ms"] >= 0
    ids = json.load(open(out))
    assert len(ids) == 6 and all(len(v) == 5 for v in ids.values())


def test_cli_generate_and_tokenize(tmp_path, capsys):
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import synthetic_config
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ck"), synthetic_config("tiny-qwen3"), seed=1)
    assert cli.main(["--model", d, "--prompt", "hello world", "--tokenize-only"]) == 0
    toks = capsys.readouterr().out.split()
    assert toks and all(t.isdigit() for t in toks)
    assert cli.main(["--model", d, "--prompt", "hello", "--max-tokens", "4", "--device", "cpu",
                     "--max-model-len", "128"]) == 0
    plain = capsys.readouterr().out
    assert cli.main(["--model", d, "--prompt", "hello", "--max-tokens", "4", "--device", "cpu",
                     "--max-model-len", "128", "--stream"]) == 0
    assert capsys.readouterr().out.strip() == plain.strip()
