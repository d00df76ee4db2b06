"""Build the C-ABI CUDA library (libhilda_b200.so) in-tree with nvcc for sm_100a.

Usage: ``python -m hilda_kernel_b200._build [--force] [--debug]`` or ``build()``. ``--debug`` (or
HILDA_DEBUG=1 in the environment) builds ``libhilda_b200_debug.so`` with ``-DHILDA_DEBUG``: every launch
is followed by a device synchronisation and an error check, so an asynchronous fault is reported by
the entry point that caused it (not usable under stream capture); ``_lib`` loads that library when
HILDA_DEBUG=1 is set and it exists. Object files are cached under
``hilda_kernel_b200/build`` keyed on the modification times of each source and of the headers it includes, so a
rebuild after touching one file recompiles only what depends on it. nvcc cross-compiles; no GPU is needed.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libhilda_b200.so")
DEBUG_LIB_PATH = os.path.join(PKG_DIR, "libhilda_b200_debug.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime(src: str, seen: set | None = None) -> float:
    """Newest modification time of `src` and of the project headers it includes (recursively), so
    that touching one header recompiles only the sources that use it."""
    import re
    seen = seen if seen is not None else set()
    if src in seen or not os.path.exists(src):
        return 0.0
    seen.add(src)
    newest = os.path.getmtime(src)
    inc = os.path.join(os.path.dirname(PKG_DIR), "include")
    for name in re.findall(r'^\s*#\s*include\s*"([^"]+)"', open(src).read(), flags=re.M):
        for base in (os.path.dirname(src), CSRC, inc):
            cand = os.path.join(base, name)
            if os.path.exists(cand):
                newest = max(newest, _deps_mtime(cand, seen))
                break
    return newest


def compile_one(src: str, obj: str, debug: bool = False) -> list[str]:
    """The nvcc command line for one source (used by build() and by the test that the debug flag compiles)."""
    inc = os.path.join(os.path.dirname(PKG_DIR), "include")
    return [_nvcc(), *NVCC_FLAGS, *(["-DHILDA_DEBUG"] if debug else []), "-I", inc, "-I", CSRC, "-c", src, "-o", obj]


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> str:
    """Compile every csrc/*.cu and link libhilda_b200.so (libhilda_b200_debug.so with debug). Returns the library path."""
    nvcc = _nvcc()
    build_dir = BUILD_DIR + ("_debug" if debug else "")
    lib_path = DEBUG_LIB_PATH if debug else LIB_PATH
    os.makedirs(build_dir, exist_ok=True)
    inc = os.path.join(os.path.dirname(PKG_DIR), "include")
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(build_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < _deps_mtime(src)
        if stale:
            jobs.append(compile_one(src, obj, debug))

    def run(cmd):
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        return r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    need_link = bool(jobs) or not os.path.exists(lib_path) or any(
        os.path.getmtime(o) > os.path.getmtime(lib_path) for o in objs)
    if need_link:
        run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib_path, *objs,
             "-cudart", "static"])
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True,
                debug="--debug" in sys.argv or os.environ.get("HILDA_DEBUG", "0") not in ("", "0")))
