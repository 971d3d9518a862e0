"""TEST INFRASTRUCTURE ONLY - builds oracle/_ref/libpat_ref_tree.so.

Compiles ``oracle/ref_tree_shim.cpp`` against the reference's header-only C++
scheduler (``csrc/prefix_tree.h``) where it lies in the read-only reference
checkout, with plain g++ against the installed libtorch (the header stores its
plan in ``torch::Tensor`` objects).  The reference's own build system is not
run; its CUDA kernels are not built (they need CUTLASS and target sm80).
Output goes to ``oracle/_ref/`` only, which is git-ignored.

    python oracle/build_ref.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libpat_ref_tree.so")
# The reference checkout: PAT_REFERENCE_ROOT, else a directory named "reference" beside this repository.
REFERENCE_ROOT = os.environ.get("PAT_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def reference_header() -> str:
    return os.path.join(REFERENCE_ROOT, "csrc", "prefix_tree.h")


def build(force: bool = False) -> str | None:
    """Returns the path of the library, or ``None`` when the reference checkout
    is absent and nothing was built before."""
    if not os.path.isfile(reference_header()):
        return OUT if os.path.isfile(OUT) else None
    shim = os.path.join(HERE, "ref_tree_shim.cpp")
    if (not force and os.path.isfile(OUT)
            and os.path.getmtime(OUT) >= max(os.path.getmtime(shim), os.path.getmtime(reference_header()))):
        return OUT
    import torch
    from torch.utils import cpp_extension as ext
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in ext.include_paths()] + [f"-I{os.path.dirname(reference_header())}"]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-shared", "-fPIC", "-O1", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           *inc, shim, "-o", OUT, f"-L{libdir}", f"-Wl,-rpath,{libdir}",
           "-ltorch", "-ltorch_cpu", "-lc10"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the reference scheduler failed:\n{res.stderr[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
