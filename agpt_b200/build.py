"""Build libagpt_b200.so in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libagpt_b200.so")
SOURCES = [os.path.join(HERE, "csrc", "kernels.cu"), os.path.join(HERE, "csrc", "dense.cu"),
           os.path.join(HERE, "csrc", "rowops.cu"), os.path.join(HERE, "csrc", "optim.cu"),
           os.path.join(HERE, "csrc", "gemm3x.cu"), os.path.join(HERE, "csrc", "gemm_sm100.cu"),
           os.path.join(HERE, "csrc", "host_trie.cpp"), os.path.join(HERE, "csrc", "trie_suffix.cpp"),
           os.path.join(HERE, "csrc", "trie_gpu.cu")]


# The two GEMM translation units instantiate CUTLASS templates, and gemm_sm100.cu re-instantiates the SM100 fast-FP32
# mainloop through type aliases of that collective, so the header tree is pinned to the release it was written and
# measured against.  AGPT_CUTLASS_INCLUDE names a tree explicitly (a checkout of that release); otherwise the copies
# shipped inside installed Python packages are tried, and one of another release is passed over.
CUTLASS_PINNED = (4, 5)


def cutlass_version(include_dir):
    """(major, minor, patch) from cutlass/version.h of a header tree, or None."""
    import re
    try:
        text = open(os.path.join(include_dir, "cutlass", "version.h")).read()
    except OSError:
        return None
    got = [re.search(r"#define\s+CUTLASS_%s\s+(\d+)" % k, text) for k in ("MAJOR", "MINOR", "PATCH")]
    return tuple(int(m.group(1)) for m in got) if all(got) else None


def cutlass_include():
    """CUTLASS header tree of the pinned release (header-only).  None if there is none: the library is then built with
    AGPT_NO_CUTLASS (the GEMM entry points report that; everything else works)."""
    import importlib.util
    explicit = os.environ.get("AGPT_CUTLASS_INCLUDE")
    if explicit:
        v = cutlass_version(explicit)
        if v is None or v[:2] != CUTLASS_PINNED:
            raise RuntimeError(f"AGPT_CUTLASS_INCLUDE={explicit}: CUTLASS {v} found, {CUTLASS_PINNED[0]}.{CUTLASS_PINNED[1]}.x needed")
        return explicit
    for pkg, rel in (("flashinfer", ("data", "cutlass", "include")), ("tilelang", ("3rdparty", "cutlass", "include"))):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.submodule_search_locations:
            path = os.path.join(list(spec.submodule_search_locations)[0], *rel)
            v = cutlass_version(path)
            if v is not None and v[:2] == CUTLASS_PINNED and os.path.exists(os.path.join(path, "cutlass", "gemm", "device", "gemm_universal.h")):
                return path
    return None


HEADERS = [os.path.join(HERE, "csrc", "internal.h"), os.path.join(HERE, "..", "include", "agpt_b200.h")]


OBJ_DIR = os.path.join(HERE, "_build")


def nvcc_command(src, obj, extra=()):
    """Compile one source to an object for sm_100a."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    inc = cutlass_include()
    flags = ["-I" + inc, "--expt-relaxed-constexpr", "-diag-suppress", "20012,20013,20015"] if inc else ["-DAGPT_NO_CUTLASS"]
    return [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
            *flags, *extra, "-c", "-o", obj, src]


def link_command(objs):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    return [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", SO, *objs]


def _obj(src):
    return os.path.join(OBJ_DIR, os.path.basename(src) + ".o")


def _stale(src):
    o = _obj(src)
    return not os.path.exists(o) or any(os.path.getmtime(f) > os.path.getmtime(o) for f in [src] + HEADERS)


def needs_build() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    return any(os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the sources that changed (in parallel; the two CUTLASS translation units take minutes) and link."""
    if force or needs_build():
        from concurrent.futures import ThreadPoolExecutor
        os.makedirs(OBJ_DIR, exist_ok=True)
        todo = [f for f in SOURCES if force or _stale(f)]
        extra = ("-Xptxas", "-v") if verbose else ()
        with ThreadPoolExecutor(max_workers=max(1, len(todo))) as pool:
            list(pool.map(lambda f: subprocess.check_call(nvcc_command(f, _obj(f), extra)), todo))
        subprocess.check_call(link_command([_obj(f) for f in SOURCES]))
    return SO


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(SO)
