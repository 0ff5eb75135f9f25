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


_build_dir: Optional[str] = None
_build_dir_lock = threading.Lock()


def build_dir() -> str:
    """Where objects and the libraries go: inside the package if writable, else a per-user
    folder under the system's temporary directory."""
    global _build_dir
    with _build_dir_lock:
        if _build_dir is None:
            d = os.path.join(_HERE, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                probe = os.path.join(d, f".w{os.getpid()}")
                with open(probe, "w"):
                    pass
                os.remove(probe)
            except OSError:
                tag = hashlib.sha1(_HERE.encode()).hexdigest()[:10]
                d = os.path.join(tempfile.gettempdir(), f"atom_b200_build_{os.getuid()}_{tag}")
                os.makedirs(d, exist_ok=True)
            _build_dir = d
        return _build_dir


# Sources that are compiled per variant (one library per value of their -D parameters), on
# first use by a model that needs that variant; everything else goes into the core library.
VARIANT_SOURCES = {"attention_flash.cu"}


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu") and f not in VARIANT_SOURCES)


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


def build(verbose: bool = True) -> str:
    """Compiles what is out of date of the core library and returns its path."""
    return _build(LIB_NAME, sources(), {}, verbose, ["-lcublas"])


def build_variant(source: str, defines: Dict[str, object], verbose: bool = True) -> str:
    """Compiles one variant source with its -D parameters into a library of its own, e.g.
    attention_flash.cu with ATOM_HD=128 -> libatom_attention_flash_ATOM_HD128.so."""
    if source not in VARIANT_SOURCES:
        raise NativeBuildError(f"{source} is not a variant source")
    tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items()))
    name = f"libatom_{os.path.splitext(source)[0]}_{tag}.so"
    return _build(name, [source], {k: str(v) for k, v in defines.items()}, verbose, [])


def _build(lib_name: str, srcs: List[str], defines: Dict[str, str], verbose: bool, link_libs: List[str]) -> str:
    nvcc = find_nvcc()
    bdir = build_dir()
    lock_path = os.path.join(bdir, f".lock.{lib_name}")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(nvcc, bdir, verbose, defines, lib_name, srcs, link_libs)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(nvcc: str, bdir: str, verbose: bool, defines: Dict[str, str], lib_name: str,
                  srcs: List[str], link_libs: List[str]) -> str:
    flags = ARCH_FLAGS + NVCC_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    hdr = _headers_hash()
    if not srcs:
        raise NativeBuildError(f"no .cu sources under {CSRC}")
    # An object is named <source>.<defines>.<hash>.o, so that the objects of older versions of
    # the same source and variant can be told from those of other variants and removed.
    tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items())) or "core"
    objs, todo = [], []
    for s in srcs:
        key = _source_key(s, hdr, flags)
        obj = os.path.join(bdir, f"{os.path.splitext(s)[0]}.{tag}.{key}.o")
        objs.append(obj)
        if not os.path.isfile(obj):
            todo.append((s, obj))
    link_key = hashlib.sha1("".join(os.path.basename(o) for o in objs).encode()).hexdigest()[:16]
    lib = os.path.join(bdir, lib_name)
    stamp = os.path.join(bdir, lib_name + ".stamp")
    linked = ""
    if os.path.isfile(stamp) and os.path.isfile(lib):
        with open(stamp) as f:
            linked = f.read().strip()
    if not todo and linked == link_key:
        return lib

    if todo and verbose:
        _log(f"compiling {len(todo)} CUDA source(s) of {lib_name} for sm_100a into {bdir} (first call only)")
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
        _prune(bdir, srcs, tag, {os.path.basename(o) for o in objs})
        tmp = lib + f".tmp{os.getpid()}"
        cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
        _run([nvcc, "-shared", "-o", tmp] + objs + ["-L", cuda_lib] + link_libs, "link")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(link_key)
    finally:
        stop.set()
    if verbose:
        _log(f"built {lib_name} in {time.time() - t0:.1f} s")
    return lib


def _prune(bdir: str, srcs: Sequence[str], tag: str, keep: set) -> None:
    """Removes the objects of this variant that the library just linked does not hold (older versions of
    its sources, and sources that are gone), and objects named in an older scheme (<source>.<hash>.o)
    whatever they belonged to."""
    for f in os.listdir(bdir):
        if not f.endswith(".o") or f in keep:
            continue
        parts = f.split(".")
        stale = (len(parts) == 4 and parts[1] == tag) or len(parts) == 3
        if stale:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass


# Head sizes whose attention variant the build check compiles ahead of use.
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 128, 256)


def build_all(verbose: bool = True) -> str:
    """Compiles the core library and the usual variants (the build check); returns the core's path."""
    core = build(verbose=verbose)
    with concurrent.futures.ThreadPoolExecutor(max(1, min(len(PREBUILT_HEAD_DIMS), os.cpu_count() or 1))) as ex:
        list(ex.map(lambda hd: build_variant("attention_flash.cu", {"ATOM_HD": hd}, verbose), PREBUILT_HEAD_DIMS))
    return core


if __name__ == "__main__":
    print(build_all())
