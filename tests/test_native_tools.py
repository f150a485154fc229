"""The native executables (no interpreter): b200-bench runs the closed-loop workload of the
reference's bench tool over the native engine, b200-cli completes or tokenises a prompt."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "vllm_cpp_b200", "bin")


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from vllm_cpp_b200 import loader
    from vllm_cpp_b200.config import synthetic_config
    return loader.write_synthetic_checkpoint(str(tmp_path_factory.mktemp("t") / "ck"), synthetic_config("tiny-qwen3"), seed=5)


def test_native_bench_tool(ckpt):
    exe = os.path.join(BIN, "b200-bench")
    assert os.path.exists(exe), "native tools not built"
    assert "libpython" not in subprocess.run(["ldd", exe], capture_output=True, text=True).stdout
    r = subprocess.run([exe, "--model", ckpt, "--device", "cpu", "--num-prompts", "6", "--input-len", "24",
                        "--output-len", "5", "--concurrency", "3", "--json"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    assert rep["completed"] == 6 and rep["total_input"] == 144 and rep["total_output"] == 30
    assert rep["output_tok_s"] > 0 and rep["p50_ttft_ms"] > 0
    # a bad model path is an error message, not a crash
    r = subprocess.run([exe, "--model", "/nonexistent"], capture_output=True, text=True)
    assert r.returncode == 1 and "b200-bench:" in r.stderr


def test_native_cli_matches_the_python_engine(ckpt):
    exe = os.path.join(BIN, "b200-cli")
    r = subprocess.run([exe, "--model", ckpt, "--device", "cpu", "--prompt", "The quick brown", "--max-tokens", "8"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    from vllm_cpp_b200.config import EngineArgs
    from vllm_cpp_b200.engine import LLM, SamplingParams
    llm = LLM(EngineArgs(model=ckpt, device="cpu", cpu_backend="native", block_size=32, num_blocks=64, max_model_len=256))
    want = llm.generate(["The quick brown"], SamplingParams(temperature=0.0, max_tokens=8))[0].outputs[0].text
    assert r.stdout.rstrip("\n") == want
    t = subprocess.run([exe, "--model", ckpt, "--device", "cpu", "--prompt", "The quick brown", "--tokenize"],
                       capture_output=True, text=True, timeout=120)
    assert [int(x) for x in t.stdout.split()] == llm.tokenizer.encode("The quick brown")
