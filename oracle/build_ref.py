"""Compile the reference project's own hot-path CUDA kernels, unchanged, for sm_100a.

Test / measurement infrastructure only (nothing in the product loads the result).  The six
``.cu`` files are compiled where they lie in a checkout of the reference
(BhargavKumarNath/custom_cuda_kernals, ``csrc/kernels``) with the flags of its ``build.rs``
(build.rs:63-72: ``-O3 --use_fast_math -std=c++17 -I csrc/includes``), only the architecture
changed from its default ``sm_89``; no source is copied.  The output,
``oracle/_ref/libcustom_cuda_ref.so``, exports the reference's ``launch_*`` functions and is
used (a) by ``tests/test_gpu_vs_reference_kernels.py`` to compare this library's kernels with
the reference's on a GPU and (b) by ``bench.py`` to time the reference's kernels on the same
B200 beside ours.  The reference's Rust/PyO3 layer is not needed for either and cannot be built
here (no Rust toolchain).

    python oracle/build_ref.py --reference /path/to/reference

Without ``--reference`` the checkout is looked for in ``$CUSTOM_CUDA_REFERENCE`` and then in a
directory named ``reference`` beside this repository; if neither exists nothing is built.
"""

from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libcustom_cuda_ref.so"
KERNELS = ["rmsnorm_residual", "swiglu", "rope", "fp8_quant", "matmul_add_bias", "linear_cross_entropy",
           "moe_router", "token_permute"]


def find_reference() -> pathlib.Path | None:
    """A checkout of the reference project: ``$CUSTOM_CUDA_REFERENCE``, else a ``reference``
    directory beside this repository.  None when neither holds ``csrc/kernels``."""
    for cand in (os.environ.get("CUSTOM_CUDA_REFERENCE"), HERE.parent.parent / "reference"):
        if cand and (pathlib.Path(cand) / "csrc" / "kernels").is_dir():
            return pathlib.Path(cand)
    return None


def build(reference: str | pathlib.Path, verbose: bool = False) -> pathlib.Path | None:
    ref = pathlib.Path(reference)
    src_dir, inc_dir = ref / "csrc" / "kernels", ref / "csrc" / "includes"
    if not src_dir.is_dir():
        return None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT.mkdir(exist_ok=True)
    objs = []
    for name in KERNELS:
        obj = OUT / f"{name}.o"
        cmd = [nvcc, "-c", str(src_dir / f"{name}.cu"), "-o", str(obj), "-O3", "--use_fast_math",
               "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(inc_dir), "-std=c++17", "-Xcompiler", "-fPIC"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    # -Bsymbolic: the library binds its own symbols, it shares names with libcustom_cuda_b200
    subprocess.run([nvcc, "-shared", "-o", str(LIB), *objs, "-cudart", "static", "-Xlinker", "-Bsymbolic",
                    "-Wno-deprecated-gpu-targets"], check=True)
    for o in objs:
        pathlib.Path(o).unlink()
    return LIB


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", default=None)
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    reference = a.reference or find_reference()
    lib = build(reference, a.verbose) if reference else None
    print(f"built {lib}" if lib else f"no reference checkout ({reference}); nothing built")
    return 0


if __name__ == "__main__":
    sys.exit(main())
