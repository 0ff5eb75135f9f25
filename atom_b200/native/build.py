"""Builds the sm_100a kernel library from the sources under ``csrc/`` with nvcc.

The kernels expose a plain C interface (raw pointers, sizes, a stream) and include no
framework headers, so a cold build takes well under a minute.  Objects are cached by a
hash of their source, the shared headers and the compiler flags; a second call does
nothing.  The library is placed inside the package (``native/_build``) when that folder
can be written, else in a per-user folder under the system's temporary directory.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LIB_NAME = "libatom_b200.so"


class NativeBuildError(RuntimeError):
    """The kernel library could not be built; the product path does not run without it."""


def _log(msg: str) -> None:
    print(f"[atom_b200.native] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    if os.environ.get("CUDA_HOME"):
        cands.append(os.path.join(os.environ["CUDA_HOME"], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise NativeBuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin, PATH)")


def build_dir() -> str:
    """Where objects and the library go: inside the package if writable."""
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        tag = hashlib.sha1(_HERE.encode()).hexdigest()[:10]
        d = os.path.join(tempfile.gettempdir(), f"atom_b200_build_{os.getuid()}_{tag}")
        os.makedirs(d, exist_ok=True)
        return d


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_hash() -> str:
    h = hashlib.sha1()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    return h.hexdigest()


def _source_key(src: str, hdr: str, flags: Sequence[str]) -> str:
    h = hashlib.sha1()
    with open(os.path.join(CSRC, src), "rb") as fh:
        h.update(fh.read())
    h.update(hdr.encode())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise NativeBuildError(f"{what} failed:\n{' '.join(cmd)}\n{p.stdout}")


def build(verbose: bool = True, extra_defines: Optional[Dict[str, str]] = None) -> str:
    """Compiles what is out of date and returns the path of the shared library."""
    nvcc = find_nvcc()
    bdir = build_dir()
    lock_path = os.path.join(bdir, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(nvcc, bdir, verbose, extra_defines or {})
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(nvcc: str, bdir: str, verbose: bool, defines: Dict[str, str]) -> str:
    flags = ARCH_FLAGS + NVCC_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    hdr = _headers_hash()
    srcs = sources()
    if not srcs:
        raise NativeBuildError(f"no .cu sources under {CSRC}")
    objs, todo = [], []
    for s in srcs:
        key = _source_key(s, hdr, flags)
        obj = os.path.join(bdir, f"{os.path.splitext(s)[0]}.{key}.o")
        objs.append(obj)
        if not os.path.isfile(obj):
            todo.append((s, obj))
    link_key = hashlib.sha1("".join(os.path.basename(o) for o in objs).encode()).hexdigest()[:16]
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "link.stamp")
    linked = ""
    if os.path.isfile(stamp) and os.path.isfile(lib):
        with open(stamp) as f:
            linked = f.read().strip()
    if not todo and linked == link_key:
        return lib

    if todo and verbose:
        _log(f"compiling {len(todo)} CUDA source(s) for sm_100a into {bdir} (first call only)")
    t0 = time.time()
    done = [0]
    stop = threading.Event()

    def ticker() -> None:
        while not stop.wait(10.0):
            _log(f"  ... still compiling ({done[0]}/{len(todo)} done, {time.time() - t0:.0f} s)")

    def compile_one(item) -> None:
        s, obj = item
        tmp = obj + f".tmp{os.getpid()}"
        _run([nvcc] + flags + ["-I", CSRC, "-c", os.path.join(CSRC, s), "-o", tmp], f"nvcc {s}")
        os.replace(tmp, obj)
        done[0] += 1
        if verbose:
            _log(f"  compiled {s} ({done[0]}/{len(todo)})")

    th = threading.Thread(target=ticker, daemon=True)
    if todo and verbose:
        th.start()
    try:
        workers = max(1, min(len(todo), os.cpu_count() or 1))
        if todo:
            with concurrent.futures.ThreadPoolExecutor(workers) as ex:
                list(ex.map(compile_one, todo))
        # Remove objects of older source versions.
        keep = {os.path.basename(o) for o in objs}
        for f in os.listdir(bdir):
            if f.endswith(".o") and f not in keep:
                try:
                    os.remove(os.path.join(bdir, f))
                except OSError:
                    pass
        tmp = lib + f".tmp{os.getpid()}"
        cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
        _run(
            [nvcc, "-shared", "-o", tmp] + objs + ["-L", cuda_lib, "-lcublas"],
            "link",
        )
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(link_key)
    finally:
        stop.set()
    if verbose:
        _log(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return lib


def build_all(verbose: bool = True) -> str:
    """Compiles everything the package can need (the build check); returns the library path."""
    return build(verbose=verbose)


if __name__ == "__main__":
    print(build_all())
