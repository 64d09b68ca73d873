"""Build libagpt_b200.so in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libagpt_b200.so")
SOURCES = [os.path.join(HERE, "csrc", "kernels.cu"), os.path.join(HERE, "csrc", "dense.cu"),
           os.path.join(HERE, "csrc", "gemm3x.cu"), os.path.join(HERE, "csrc", "host_trie.cpp")]


def cutlass_include():
    """CUTLASS header tree vendored inside an installed Python package (header-only; templates are instantiated in
    gemm3x.cu).  None if no tree is found: the library is then built with AGPT_NO_CUTLASS."""
    import importlib.util
    for pkg, rel in (("flashinfer", ("data", "cutlass", "include")), ("tilelang", ("3rdparty", "cutlass", "include"))):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.submodule_search_locations:
            path = os.path.join(list(spec.submodule_search_locations)[0], *rel)
            if os.path.exists(os.path.join(path, "cutlass", "gemm", "device", "gemm_universal.h")):
                return path
    return None
HEADERS = [os.path.join(HERE, "csrc", "internal.h"), os.path.join(HERE, "..", "include", "agpt_b200.h")]


def nvcc_command(extra=()):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    inc = cutlass_include()
    extra = tuple(extra) + (("-I" + inc,) if inc else ("-DAGPT_NO_CUTLASS",))
    return [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "-shared", "-Xcompiler", "-fPIC", *extra, "-o", SO, *SOURCES]


def needs_build() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    return any(os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    if force or needs_build():
        cmd = nvcc_command(("-Xptxas", "-v") if verbose else ())
        subprocess.check_call(cmd)
    return SO


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(SO)
