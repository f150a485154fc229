"""In-tree native build: CUDA kernels (sm_100a) -> ``_kernels.so``; host engine -> ``_engine*.so``.

Everything is compiled with explicit ``nvcc`` / ``g++`` command lines (no JIT cache), so the
shared objects sit inside the package directory and travel with the source tree.
Objects are rebuilt only when a source or header is newer than the object.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_HOME = Path(NVCC).resolve().parent.parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "-I", str(CSRC / "kernels"), "-I", str(ROOT / "include"),
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread",
             "-I", str(ROOT / "include"), "-I", str(CSRC), "-I", str(CSRC / "engine")]


def _newer(src: Path, deps: list[Path], obj: Path) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(d.stat().st_mtime > t for d in [src, *deps] if d.exists())


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {cmd[0]} {cmd[-1]}")


def build_kernels(verbose: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link ``_kernels.so``."""
    out = PKG / "_kernels.so"
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.h")) + sorted((CSRC / "kernels").glob("*.cuh"))
    objdir = BUILD / "kernels"
    objdir.mkdir(parents=True, exist_ok=True)
    jobs = []
    for s in srcs:
        o = objdir / (s.stem + ".o")
        if _newer(s, hdrs, o):
            jobs.append([NVCC, *NVCC_FLAGS, "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    objs = [objdir / (s.stem + ".o") for s in srcs]
    if jobs or not out.exists():
        _run([NVCC, "-shared", "-o", str(out), *map(str, objs), "-cudart", "shared",
              "-Xlinker", f"-rpath={CUDA_HOME}/lib64", "-Xlinker", "-soname=_kernels.so"])
    if verbose:
        print(f"built {out} from {len(srcs)} CUDA sources ({len(jobs)} recompiled)")
    return out


def build_engine(verbose: bool = False) -> Path:
    """Compile the host engine (scheduler, KV manager, tokenizer, C ABI ...) and its Python
    binding into ``_engine.so`` (pybind11 module) plus ``libvllm_b200.so`` (C ABI only)."""
    import pybind11

    out = PKG / ("_engine" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    srcs = sorted((CSRC / "engine").rglob("*.cpp"))
    hdrs = sorted((CSRC / "engine").rglob("*.h")) + sorted((ROOT / "include").rglob("*.h"))
    objdir = BUILD / "engine"
    objdir.mkdir(parents=True, exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    jobs = []
    objs = []
    for s in srcs:
        o = objdir / (str(s.relative_to(CSRC / "engine")).replace("/", "__")[:-4] + ".o")
        objs.append(o)
        if _newer(s, hdrs, o):
            jobs.append([CXX, *CXX_FLAGS, *inc, "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    if jobs or not out.exists():
        _run([CXX, "-shared", "-o", str(out), *map(str, objs), "-pthread"])
    if verbose:
        print(f"built {out} from {len(srcs)} C++ sources ({len(jobs)} recompiled)")
    return out


BINDING_STEMS = ("bindings", "tokenizer_bindings", "structured_bindings", "offload_bindings", "extras_bindings",
                 "parallel_bindings")


def build_capi(verbose: bool = False) -> Path:
    """The C interface of ``include/vllm.h``, twice:

    ``libvllm_b200.so``     the native runtime (``csrc/runtime`` + the host engine objects), linked
                            against libtorch (memory, streams), ``_kernels.so`` and ``_cpu.so``; no
                            interpreter. Only the ``vllm_*`` symbols are exported.
    ``libvllm_b200_py.so``  the same interface over the Python engine (embeds the interpreter); the
                            native library loads it on demand for models it does not cover."""
    build_capi_py(verbose)
    capi = PKG / "libvllm_b200.so"
    rt_srcs = sorted((CSRC / "runtime").glob("*.cpp")) + [CSRC / "capi" / "vllm_c.cpp"]
    if not (CSRC / "runtime").exists():
        return capi
    eng_srcs = [s for s in sorted((CSRC / "engine").rglob("*.cpp")) if s.stem not in BINDING_STEMS]
    hdrs = (sorted((CSRC / "runtime").glob("*.h")) + sorted((CSRC / "engine").rglob("*.h")) +
            [ROOT / "include" / "vllm.h", CSRC / "kernels" / "api.h"])
    from torch.utils import cpp_extension as ce
    import torch
    torch_inc = [x for p in ce.include_paths() for x in ("-I", p)]
    torch_lib = ce.library_paths()[0]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    objdir = BUILD / "runtime"
    objdir.mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for s in rt_srcs:
        o = objdir / (s.stem + ".o")
        objs.append(o)
        if _newer(s, hdrs, o):
            extra = torch_inc if s.stem == "tensor" else []      # the one libtorch translation unit
            jobs.append([CXX, *CXX_FLAGS, abi, "-I", str(CUDA_HOME / "include"), *extra, "-c", str(s), "-o", str(o)])
    eng_objdir = BUILD / "engine"
    for s in eng_srcs:
        o = eng_objdir / (str(s.relative_to(CSRC / "engine")).replace("/", "__")[:-4] + ".o")
        objs.append(o)
        if _newer(s, hdrs, o):
            jobs.append([CXX, *CXX_FLAGS, "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    deps = [PKG / "_kernels.so", PKG / "_cpu.so"]
    if jobs or not capi.exists() or any(d.exists() and d.stat().st_mtime > capi.stat().st_mtime for d in deps):
        _run([CXX, "-shared", "-o", str(capi), *map(str, objs), "-pthread", "-ldl",
              f"-L{PKG}", "-l:_kernels.so", "-l:_cpu.so",
              f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
              f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
              f"-Wl,--version-script={CSRC / 'capi' / 'export.map'}",
              f"-Wl,-rpath,$ORIGIN:{torch_lib}:{CUDA_HOME / 'lib64'}", "-Wl,--no-as-needed"])
        if verbose:
            print(f"built {capi}")
    # native executables over the same objects (everything but the C interface)
    bindir = PKG / "bin"
    bindir.mkdir(exist_ok=True)
    lib_objs = [o for o in objs if o.stem != "vllm_c"]
    for tool, src in (("b200-bench", CSRC / "tools" / "bench_main.cpp"), ("b200-cli", CSRC / "tools" / "cli_main.cpp")):
        exe = bindir / tool
        if src.exists() and (jobs or _newer(src, hdrs, exe)):
            _run([CXX, *CXX_FLAGS, "-o", str(exe), str(src), *map(str, lib_objs), "-pthread", "-ldl",
                  f"-L{PKG}", "-l:_kernels.so", "-l:_cpu.so",
                  f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
                  f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
                  f"-Wl,-rpath,$ORIGIN/..:{torch_lib}:{CUDA_HOME / 'lib64'}", "-Wl,--no-as-needed"])
            if verbose:
                print(f"built {exe}")
    return capi


def build_capi_py(verbose: bool = False) -> Path:
    """``libvllm_b200_py.so``: the C interface over the Python engine. It embeds the interpreter,
    so it links against libpython; only the ``vllm_*`` symbols are exported."""
    capi = PKG / "libvllm_b200_py.so"
    srcs = [CSRC / "capi" / "vllm_c_py.cpp"]
    if not srcs[0].exists():
        return capi
    hdrs = [ROOT / "include" / "vllm.h"]
    if any(_newer(s, hdrs, capi) for s in srcs):
        libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
        ver = sysconfig.get_config_var("LDVERSION") or "3.12"
        _run([CXX, *CXX_FLAGS, "-I", sysconfig.get_paths()["include"], "-shared", "-o", str(capi),
              *map(str, srcs), "-pthread", "-ldl", f"-L{libdir}", f"-lpython{ver}",
              f"-Wl,--version-script={CSRC / 'capi' / 'export.map'}", f"-Wl,-rpath,{libdir}"])
        if verbose:
            print(f"built {capi}")
    return capi


def build_cpu(verbose: bool = False) -> Path:
    """``_cpu.so``: the native CPU backend (thread pool + bf16 ops). Host floating point is pinned
    with -ffp-contract=off; the vector tiers are selected at run time inside the library."""
    out = PKG / "_cpu.so"
    srcs = sorted((CSRC / "cpu").glob("*.cpp"))
    if not srcs:
        return out
    hdrs = sorted((CSRC / "cpu").glob("*.h"))
    if any(_newer(s, hdrs, out) for s in srcs):
        _run([CXX, "-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-ffp-contract=off",
              "-fno-math-errno", "-shared", "-Wl,-soname,_cpu.so", "-o", str(out), *map(str, srcs)])
        if verbose:
            print(f"built {out} from {len(srcs)} C++ sources")
    return out


def build_sanitize_driver(kind: str = "address,undefined", verbose: bool = False) -> Path:
    """Compiles the host engine (no Python, no CUDA) with ``csrc/engine_sanitize/sanitize_main.cpp``
    under ``-fsanitize=<kind>`` into ``build/sanitize_<kind>``; running it exercises the
    scheduler, KV-cache manager, input batch, offload policies and the LMCache codec."""
    tag = kind.replace(",", "_")
    out = BUILD / f"sanitize_{tag}"
    srcs = [s for s in sorted((CSRC / "engine").rglob("*.cpp")) if s.stem not in BINDING_STEMS]
    srcs.append(CSRC / "engine_sanitize" / "sanitize_main.cpp")
    hdrs = sorted((CSRC / "engine").rglob("*.h"))
    BUILD.mkdir(parents=True, exist_ok=True)
    # the sanitizer runtimes ship with the distribution compiler, not necessarily with $CXX
    cxx = os.environ.get("SANITIZE_CXX") or ("/usr/bin/g++" if Path("/usr/bin/g++").exists() else CXX)
    if any(_newer(s, hdrs, out) for s in srcs):
        _run([cxx, "-O1", "-g", "-std=c++20", "-fno-omit-frame-pointer", f"-fsanitize={kind}",
              "-fno-sanitize-recover=all", "-pthread", "-I", str(ROOT / "include"), "-I", str(CSRC),
              "-I", str(CSRC / "engine"), "-o", str(out), *map(str, srcs)])
        if verbose:
            print(f"built {out}")
    return out


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    if (CSRC / "engine").exists():
        build_engine(verbose)
    build_cpu(verbose)
    build_capi(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
