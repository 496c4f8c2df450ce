"""In-tree build of the two native artefacts (no setuptools, no JIT cache):

  libcustom_cuda_b200.so   the C-ABI kernel library (nvcc, sm_100a only)
  _native.<abi>.so         the CPython module that validates torch tensors and
                           calls the C ABI (g++ against the torch headers)

    python -m custom_cuda_kernals_b200._build [--force] [--verbose]

Replaces the reference's build.rs (nvcc per translation unit into a static
archive linked into a Rust cdylib, build.rs:41-117).  nvcc cross-compiles, so
this runs on a machine without a GPU; outputs land next to this file so they
travel with the source tree.
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import pathlib
import shutil
import subprocess
import sys
import sysconfig

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libcustom_cuda_b200.so"
# --debug-bounds: the bandwidth-bound kernels compiled with -DCC_DEBUG_BOUNDS (csrc/common.cuh): every
# global access through the shared load / store helpers is checked against host-registered ranges,
# skipped and counted when outside.  A separate library, loaded only by the test that uses it.
DEBUG_LIB = PKG / "libcustom_cuda_b200_dbg.so"
DEBUG_SOURCES = ["swiglu.cu", "rmsnorm_residual.cu", "rope.cu"]

CU_SOURCES = ["swiglu.cu", "rmsnorm_residual.cu", "rope.cu", "fp8_quant.cu", "linear_ce_chunk_update.cu",
              "matmul_add_bias.cu", "matmul_fused.cu", "linear_cross_entropy.cu", "backward_elementwise.cu", "moe.cu"]
HEADERS = ["common.cuh", "ptx.cuh", "gemm_simt.cuh", "gemm_tcgen05.cuh", "gemm_splitk.cuh", "gemm_decode.cuh"]

# No --use_fast_math anywhere: fp8_quant.cu relies on IEEE division.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def native_path() -> pathlib.Path:
    return PKG / ("_native" + sysconfig.get_config_var("EXT_SUFFIX"))


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the CUDA kernels")
    return cand


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    proc = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")
    return proc.stdout + proc.stderr


def _stale(target: pathlib.Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(pathlib.Path(d).stat().st_mtime > t for d in deps)


def sources():
    return [CSRC / s for s in CU_SOURCES if (CSRC / s).exists()]


def build_library(force=False, verbose=False) -> pathlib.Path:
    """nvcc every .cu for sm_100a and link libcustom_cuda_b200.so."""
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdrs = [CSRC / h for h in HEADERS] + [PKG.parent / "include" / "custom_cuda_b200.h"]
    jobs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *hdrs]):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", PKG.parent / "include", "-c", src, "-o", obj])
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    objs = [OBJ / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        _run([nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined"], verbose)
    return LIB


def build_debug_library(force=False, verbose=False) -> pathlib.Path:
    """The -DCC_DEBUG_BOUNDS variant of the bandwidth-bound kernels, as its own shared library."""
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdrs = [CSRC / h for h in HEADERS]
    objs = []
    for name in DEBUG_SOURCES:
        src, obj = CSRC / name, OBJ / (pathlib.Path(name).stem + "_dbg.o")
        if force or _stale(obj, [src, *hdrs]):
            _run([nvcc, *NVCC_FLAGS, "-DCC_DEBUG_BOUNDS", "-I", PKG.parent / "include", "-c", src, "-o", obj], verbose)
        objs.append(obj)
    if force or _stale(DEBUG_LIB, objs):
        _run([nvcc, "-shared", "-o", DEBUG_LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined",
              "-Xlinker", "-Bsymbolic"], verbose)
    return DEBUG_LIB


def build_native(force=False, verbose=False) -> pathlib.Path:
    """g++ the CPython module against the torch headers; links the kernel library by $ORIGIN."""
    import torch
    from torch.utils import cpp_extension as ce

    out = native_path()
    src = CSRC / "native_module.cpp"
    if not (force or _stale(out, [src, PKG.parent / "include" / "custom_cuda_b200.h", LIB])):
        return out
    torch_lib = pathlib.Path(torch.__file__).parent / "lib"
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cuda_inc = pathlib.Path(_nvcc()).resolve().parent.parent / "include"
    inc.append(f"-I{cuda_inc}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wno-attributes",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_native", "-DTORCH_API_INCLUDE_EXTENSION_H",
           *inc, src, "-o", out,
           f"-L{PKG}", "-lcustom_cuda_b200", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
           "-ltorch_python", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False, debug_bounds=True):
    lib = build_library(force, verbose)
    native = build_native(force, verbose)
    if debug_bounds:
        build_debug_library(force, verbose)
    return lib, native


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--debug-bounds", action="store_true", help="only (re)build the -DCC_DEBUG_BOUNDS library")
    a = ap.parse_args(argv)
    if a.debug_bounds:
        print(f"built {build_debug_library(a.force, a.verbose)}")
        return 0
    lib, native = build_all(a.force, a.verbose)
    print(f"built {lib}\nbuilt {native}\nbuilt {DEBUG_LIB}")


if __name__ == "__main__":
    sys.exit(main())
