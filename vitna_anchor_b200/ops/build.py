"""Compiling the CUDA sources into one shared library for sm_100a.

Every .cu file under csrc/ is compiled by nvcc to an object file and the
objects are linked into libvitna_kernels.so.  Objects are reused while the
hash of their source (and of the headers) is unchanged, so only what changed
is compiled again.  The library is kept in the source tree (csrc/_build/) so
that it is found without any per-user cache; when the tree cannot be written
to, a folder under the system's temporary directory stands in.
Progress is printed to stderr, one line per file, so that a first call that
has to compile everything does not look hung.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libvitna_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[vitna_anchor_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked in CUDA_HOME, /usr/local/cuda and PATH); "
                     "the engine's kernels cannot be compiled and there is no fallback")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"vitna_anchor_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """The path of the built library, compiling what is out of date first."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    hh = _headers_hash()
    todo, objs, stamps = [], [], {}
    for src in _sources():
        with open(os.path.join(CSRC, src), "rb") as fh:
            digest = hashlib.sha256(fh.read() + hh.encode()).hexdigest()
        obj = os.path.join(bdir, src[:-3] + ".o")
        stamp = obj + ".sha"
        objs.append(obj)
        stamps[src] = (stamp, digest)
        try:
            with open(stamp) as fh:
                fresh = fh.read().strip() == digest and os.path.exists(obj)
        except OSError:
            fresh = False
        if not fresh:
            todo.append((src, obj))
    if not todo and os.path.exists(lib):
        return lib
    if not build:
        raise BuildError(f"{lib} is missing or out of date")
    nvcc = find_nvcc()
    t0 = time.time()
    if verbose and todo:
        _say(f"compiling {len(todo)} CUDA source file(s) for sm_100a into {bdir} (first call only)")

    def compile_one(item):
        src, obj = item
        t1 = time.time()
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{p.stdout}\n{p.stderr}")
        with open(stamps[src][0], "w") as fh:
            fh.write(stamps[src][1])
        if verbose:
            _say(f"  compiled {src} in {time.time() - t1:.0f} s")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as pool:
        list(pool.map(compile_one, todo))
    tmp = lib + f".tmp{os.getpid()}"
    p = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{p.stdout}\n{p.stderr}")
    os.replace(tmp, lib)
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib
