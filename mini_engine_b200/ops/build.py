"""Builds the CUDA kernels of ``csrc/`` into one shared library, in the tree.

``nvcc -gencode arch=compute_100a,code=sm_100a`` per source file (in parallel), then one
link.  The kernels have a plain C interface (no torch headers), so a full build takes well
under a minute.  The library is rebuilt when a source, a header or a flag changes; a build
prints what it does and a line every few seconds while the compiler runs.  If the package
folder cannot be written, the build goes to a per-user folder under the temporary directory.
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

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libmini_engine_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"] + os.environ.get("MINI_ENGINE_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[mini_engine_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be built and the engine has no other path")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
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
        d = os.path.join(tempfile.gettempdir(), f"mini_engine_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, building it first if needed."""
    d = _build_dir()
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "stamp.json")
    want = _fingerprint()

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return json.load(f).get("fingerprint") == want and os.path.isfile(lib)
        except (OSError, ValueError):
            return False

    if fresh():
        return lib
    if not build:
        raise BuildError(f"{lib} is missing or stale and building was not allowed")
    with open(os.path.join(d, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():                       # another process built it while we waited
                return lib
            _compile_all(d, lib, verbose)
            with open(stamp, "w") as f:
                json.dump({"fingerprint": want, "built": time.time()}, f)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def _compile_all(d: str, lib: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"building {len(srcs)} CUDA files for sm_100a into {d} (first call only)")
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling... {time.time() - t0:.0f} s")
    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()

    def one(name: str) -> str:
        obj = os.path.join(d, name[:-3] + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"compiled {name} ({time.time() - t0:.0f} s)")
        return obj
    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
    finally:
        done.set()
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
