"""Builds the engine's native libraries in-tree with nvcc and g++, without any torch headers.

Two shared libraries are produced under ``carbon_engine_b200/_build``:

* ``libcarbon_kernels.so`` - every CUDA source of ``csrc/kernels`` compiled for sm_100a;
* ``libcarbon_runtime.so`` - the host runtime of ``csrc/runtime`` (cache manager, scheduler).

Each source compiles to an object named after a hash of its text, of the headers and of the flags,
so a rebuild happens exactly when something changed.  Compiles run in parallel and a line is
printed for each so that a first call on a fresh checkout shows progress.  If the package folder
cannot be written the build goes to a per-user folder under the system's temporary directory.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import List, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
KERNEL_DIR = os.path.join(_HERE, "kernels")
RUNTIME_DIR = os.path.join(_HERE, "runtime")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-DCE_BUILD_ARCH=100", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]

_lock = threading.Lock()
_print_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    with _print_lock:
        print(f"[carbon_engine_b200 build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    d = os.path.join(_PKG, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"carbon_engine_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _nvcc() -> str:
    for cand in (os.environ.get("CE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels cannot be built (set CE_NVCC)")


def _digest(paths: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as fh:
            h.update(fh.read())
        h.update(b"\0")
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _sources(folder: str, exts: Sequence[str]) -> List[str]:
    return sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(tuple(exts)))


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def _compile_all(compiler: str, flags: List[str], srcs: List[str], headers: List[str], out: str, tag: str) -> List[str]:
    jobs = []
    objs = []
    for src in srcs:
        key = _digest([src] + headers, [compiler] + flags)
        obj = os.path.join(out, f"{tag}_{os.path.splitext(os.path.basename(src))[0]}_{key}.o")
        objs.append(obj)
        if not os.path.exists(obj):
            jobs.append((src, obj))

    def one(job):
        src, obj = job
        _say(f"compiling {os.path.relpath(src, _PKG)}")
        tmp = obj + f".tmp{os.getpid()}"
        _run([compiler] + flags + ["-c", src, "-o", tmp], f"compiling {src}")
        os.replace(tmp, obj)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(one, jobs))
    return objs


def _link(linker: str, flags: List[str], objs: List[str], lib: str) -> str:
    stamp = lib + ".stamp"
    want = hashlib.sha256("\n".join(objs).encode()).hexdigest()
    if os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read() == want:
        return lib
    _say(f"linking {os.path.basename(lib)}")
    tmp = lib + f".tmp{os.getpid()}"
    _run([linker] + flags + objs + ["-o", tmp], f"linking {lib}")
    os.replace(tmp, lib)
    with open(stamp, "w") as fh:
        fh.write(want)
    # objects of older source versions are no longer needed
    keep = set(objs)
    folder = os.path.dirname(lib)
    prefix = os.path.basename(objs[0]).split("_")[0] + "_" if objs else None
    for f in os.listdir(folder):
        full = os.path.join(folder, f)
        if prefix and f.startswith(prefix) and f.endswith(".o") and full not in keep:
            try:
                os.remove(full)
            except OSError:
                pass
    return lib


def build_kernels(verbose: bool = True) -> str:
    """Compile csrc/kernels/*.cu for sm_100a and return the path of libcarbon_kernels.so."""
    with _lock:
        out = build_dir()
        nvcc = _nvcc()
        srcs = _sources(KERNEL_DIR, (".cu",))
        headers = _sources(KERNEL_DIR, (".cuh", ".h"))
        objs = _compile_all(nvcc, NVCC_FLAGS, srcs, headers, out, "k")
        return _link(nvcc, ["-shared", "-gencode", "arch=compute_100a,code=sm_100a"], objs,
                     os.path.join(out, "libcarbon_kernels.so"))


def build_runtime(verbose: bool = True) -> str:
    """Compile csrc/runtime/*.cpp and return the path of libcarbon_runtime.so."""
    with _lock:
        out = build_dir()
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found: the host runtime cannot be built")
        srcs = _sources(RUNTIME_DIR, (".cpp",))
        headers = _sources(RUNTIME_DIR, (".h", ".hpp"))
        objs = _compile_all(cxx, CXX_FLAGS, srcs, headers, out, "r")
        return _link(cxx, ["-shared"], objs, os.path.join(out, "libcarbon_runtime.so"))


def build_all() -> None:
    build_runtime()
    build_kernels()


if __name__ == "__main__":
    build_all()
    print("built", build_dir())
