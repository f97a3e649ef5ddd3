"""Compiles the CUDA sources of this folder for sm_100a into one shared library, in the tree.

The library is plain C ABI (no torch headers), so a file compiles in seconds.  It is built at the
first call that needs it and rebuilt when a source, a header or a flag changed (a hash of them is
kept beside the library).  While nvcc runs, a line is printed now and then.  If the package's
folder cannot be written, the library goes to a per-user folder under the system's temporary
directory instead.
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libcima_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[cima_b200 build] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (CUDA_HOME, /usr/local/cuda/bin, PATH): the CUDA kernels cannot be built")


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    in_tree = os.path.join(os.path.dirname(HERE), "_lib")
    if _writable(in_tree):
        return in_tree
    alt = os.path.join(tempfile.gettempdir(), f"cima_b200_{os.getuid()}", "_lib")
    if _writable(alt):
        return alt
    raise BuildError(f"neither {in_tree} nor {alt} can be written; the CUDA kernels cannot be built")


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, building it if needed."""
    out = build_dir()
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, "build.json")
    want = source_hash()

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return json.load(f).get("hash") == want and os.path.isfile(lib)
        except (OSError, ValueError):
            return False

    if fresh():
        return lib
    if not build:
        raise BuildError(f"{lib} is missing or out of date")
    with open(os.path.join(out, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():                      # another process built it meanwhile
                return lib
            _compile(out, lib, verbose)
            with open(stamp, "w") as f:
                json.dump({"hash": want, "flags": NVCC_FLAGS, "sources": sources()}, f)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed ({' '.join(cmd)}):\n{p.stdout}\n{p.stderr}")


def _compile(out: str, lib: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _log(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {out}")
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _log(f"still compiling ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    objs = [os.path.join(out, s[:-3] + ".o") for s in srcs]
    try:
        def one(pair):
            s, o = pair
            _run([nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, s), "-o", o], f"compiling {s}")
            if verbose:
                _log(f"compiled {s} ({time.time() - t0:.0f} s)")
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            list(ex.map(one, zip(srcs, objs)))
        tmp = lib + f".tmp{os.getpid()}"
        _run([nvcc, "-shared", "-o", tmp, *objs], "linking")
        os.replace(tmp, lib)
    finally:
        done.set()
    if verbose:
        _log(f"built {lib} in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    print(library_path())
