"""Compiles the CUDA sources under csrc/ into one shared library for sm_100a.

The reference compiles its kernel string at run time with NVRTC for whatever GPU is installed and
keeps the binary in an on-disk cache keyed by source and options (src/cuda.rs:5485-5563).  Here the
sources are separate .cu files compiled ahead of time by nvcc for one target, sm_100a; the first
call in a fresh checkout does the compiling, later calls find the library and a stamp that names
the sources' hash.  Nothing is fetched and nothing outside the checkout (or, if that is read-only,
a per-user temporary folder) is written.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libghost_infer_kernels.so"
# fast math is never asked for: norms, softmax and rotation angles use the accurate 32-bit functions
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[ghost-infer_b200 build] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _hash_sources() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the kernels cannot be compiled")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    """In the checkout if it can be written, else a per-user temporary folder."""
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    alt = os.path.join(tempfile.gettempdir(), f"ghost_infer_b200_build_{os.getuid()}")
    if _writable_dir(alt):
        return alt
    raise BuildError(f"neither {in_tree} nor {alt} can be written: nowhere to put the compiled kernels")


def library_path(create: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, compiling it first if need be."""
    want = _hash_sources()
    candidates = [os.path.join(CSRC, "_build"), os.path.join(tempfile.gettempdir(), f"ghost_infer_b200_build_{os.getuid()}")]
    for d in candidates:
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
        try:
            if os.path.isfile(lib) and open(stamp).read().strip() == want:
                return lib
        except OSError:
            pass
    if not create:
        raise BuildError("the kernel library has not been built")
    return compile_all(verbose=verbose)


def compile_all(verbose: bool = True, jobs: Optional[int] = None) -> str:
    nvcc = _find_nvcc()
    out = build_dir()
    srcs = sources()
    want = _hash_sources()
    jobs = jobs or max(1, min(len(srcs), os.cpu_count() or 4))
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a with {jobs} jobs into {out}")
    t0 = time.time()
    done = []
    lock = threading.Lock()

    def one(src: str) -> str:
        obj = os.path.join(out, src[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{p.stdout}")
        with lock:
            done.append(src)
            if verbose:
                _say(f"  {src} done ({len(done)}/{len(srcs)}, {time.time() - t0:.0f}s)")
        return obj

    stop = threading.Event()

    def heartbeat():
        while not stop.wait(10.0):
            if verbose:
                _say(f"  still compiling ({len(done)}/{len(srcs)} files done, {time.time() - t0:.0f}s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        with ThreadPoolExecutor(max_workers=jobs) as ex:
            objs = list(ex.map(one, srcs))
        lib_tmp = os.path.join(out, f".{LIB_NAME}.{os.getpid()}")
        p = subprocess.run([nvcc, "-shared", "-o", lib_tmp] + objs, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise BuildError(f"linking the kernel library failed:\n{p.stdout}")
        lib = os.path.join(out, LIB_NAME)
        os.replace(lib_tmp, lib)
        with open(os.path.join(out, "stamp.txt"), "w") as f:
            f.write(want + "\n")
    finally:
        stop.set()
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f}s")
    return lib


if __name__ == "__main__":
    print(library_path())
