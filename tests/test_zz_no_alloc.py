"""The allocation-free small-M GEMM, called the way a C host would: through its exported
symbol with raw pointers. Named to be collected last; it must pass alone as well as after
every other GPU test has used the shared library."""
import ctypes
import glob
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 << 20


def _load():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hits = glob.glob(os.path.join(here, "vllm_cpp_b200", "_kernels*.so"))
    assert hits, "kernel library not built"
    lib = ctypes.CDLL(hits[0])
    vp, i = ctypes.c_void_p, ctypes.c_int
    lib.b200_gemm_bf16_smallm_static.argtypes = [vp, i, vp, i, vp, i, i, i, i, vp]
    lib.b200_gemm_bf16_smallm_static.restype = i
    lib.b200_gemm_bf16_smallm_static_error.restype = ctypes.c_char_p
    lib.b200_gemm_bf16_smallm_static_status.argtypes = [ctypes.POINTER(i)]
    lib.b200_gemm_bf16_smallm_static_status.restype = i
    lib.b200_gemm_bf16.argtypes = [vp, i, vp, i, vp, i, i, vp, vp, i, i, i, i, vp, ctypes.c_size_t, i, vp]
    lib.b200_gemm_bf16.restype = i
    return lib


def _rel(a, b):
    from _numerics import rel_err
    return rel_err(a, b, row_tol=0.15, abs_tol=0.1)


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (7, 1024, 14336), (256, 2048, 512),
                                   # at least as many 128-column tiles as SMs: the unsplit branch,
                                   # which writes the output directly and never touches the array
                                   (16, 19200, 256)])
def test_static_scratch_gemm_matches_workspace_gemm(M, N, K):
    lib = _load()
    torch.cuda.set_device(0)
    torch.manual_seed(M)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ws = torch.empty(SCRATCH_BYTES, dtype=torch.uint8, device="cuda")
    want = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.b200_gemm_bf16(a.data_ptr(), K, w.data_ptr(), K, want.data_ptr(), N, 0, None, None, 0,
                            M, N, K, ws.data_ptr(), SCRATCH_BYTES, 0, stream)
    assert rc == 0
    exact = a.float() @ w.float().t()
    for call in range(2):                       # the second call reuses the array uncleaned
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.b200_gemm_bf16_smallm_static(a.data_ptr(), K, w.data_ptr(), K, got.data_ptr(), N,
                                              M, N, K, stream)
        assert rc == 0, lib.b200_gemm_bf16_smallm_static_error()
        torch.cuda.synchronize()
        assert _rel(got, want) < 1e-3, f"call {call}"
        assert _rel(got, exact) < 2e-2, f"call {call}"
    st = ctypes.c_int(-1)
    assert lib.b200_gemm_bf16_smallm_static_status(ctypes.byref(st)) == 0
    assert st.value == 0


def test_static_scratch_gemm_refuses_oversize():
    lib = _load()
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8192, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(256, 8192, dtype=torch.bfloat16, device="cuda")
    # 2 * 256 * 8192 * 4 bytes = 16 MiB > the 8 MiB array
    rc = lib.b200_gemm_bf16_smallm_static(a.data_ptr(), 64, w.data_ptr(), 64, out.data_ptr(), 8192,
                                          256, 8192, 64, None)
    assert rc == -4
    assert b"B200_GEMM_STATIC_SCRATCH_BYTES" in lib.b200_gemm_bf16_smallm_static_error()
    rc = lib.b200_gemm_bf16_smallm_static(a.data_ptr(), 64, w.data_ptr(), 64, out.data_ptr(), 8192,
                                          300, 64, 64, None)
    assert rc == -4
    torch.cuda.synchronize()
