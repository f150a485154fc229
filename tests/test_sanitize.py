"""The host engine under AddressSanitizer + UndefinedBehaviorSanitizer: a C++ driver (no Python,
no CUDA) runs the scheduler, KV-cache manager, input batch, draft-token path, offload policies
and the LMCache codec against a fake runner (csrc/engine_sanitize/sanitize_main.cpp)."""
import subprocess

import pytest


def test_engine_under_asan_ubsan():
    from vllm_cpp_b200 import _build
    try:
        exe = _build.build_sanitize_driver("address,undefined")
    except RuntimeError:
        pytest.skip("no sanitizer runtime for the available compiler")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "sanitize driver ok" in r.stdout
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr
