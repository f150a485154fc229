"""The kernel library's C header (csrc/kernels/api.h) declares every exported launcher, so a
C or C++ host can call them without copying prototypes out of the sources."""
import glob
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_declares_every_exported_launcher():
    libs = glob.glob(os.path.join(ROOT, "vllm_cpp_b200", "_kernels*.so"))
    assert libs, "kernel library not built"
    out = subprocess.run(["nm", "-D", "--defined-only", libs[0]], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T b200_" in l}
    header = open(os.path.join(ROOT, "csrc", "kernels", "api.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\(", header))
    assert exported - declared == set(), f"not declared in api.h: {sorted(exported - declared)}"
    assert declared - exported == set(), f"declared but not exported: {sorted(declared - exported)}"
