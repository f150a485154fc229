"""Tensor-parallel paths on 2+ GPUs (fused kernels over peer memory vs NCCL vs TP=1).

Runs the self-test module as one process per GPU. NVLS is switched off for NCCL so that a
rank that fails cannot leave peers bound to a multicast object."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_tp_selftest(world):
    """Fused primitives against fp32, then a dense and an expert-parallel MoE engine: greedy
    tokens of TP = world (fused, native stack and per-op) against NCCL mode and TP = 1."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs at least {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29541 + world), "-m",
           "vllm_cpp_b200.parallel.selftest"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(lines[-1])
    assert res["ok"] and res["primitives_status"] == 0 and res["world"] == world
    for tag in ("qwen3", "moe"):
        assert res[f"engine_{tag}"]["ranks_identical"] and res[f"engine_{tag}"]["status"] == 0
