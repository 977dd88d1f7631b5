"""Builds the kernel library from the ``.cu`` files beside this file.

``nvcc -gencode arch=compute_100a,code=sm_100a`` compiles each source to an object
(in parallel) and links them into ``_build/libzinfer_b200.so``.  The library is
rebuilt when a source, a header or the flags change.  The build folder lies beside
the sources when that is writable, else under the system's temporary folder, so a
read-only checkout and a user without a home directory still work.  Nothing here
needs a GPU: nvcc cross-compiles.
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

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libzinfer_b200.so"
# ZINFER_B200_TRACE=1 builds a second library (in a folder of its own) whose kernels leave time stamps
# for a timeline of the chain (common.cuh, zinfer_b200.profiling.chain_timeline)
TRACE = os.environ.get("ZINFER_B200_TRACE", "0") not in ("", "0")
BUILD_FOLDER = "_build_trace" if TRACE else "_build"
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
] + (["-DZI_TRACE"] if TRACE else [])


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the kernel library cannot be built (set NVCC or put nvcc on PATH)")


def sources() -> list[str]:
    """The kernels (.cu) and the native host runtime (.cpp); nvcc compiles both."""
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cpp")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cuh", ".h", ".cpp")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    local = os.path.join(HERE, BUILD_FOLDER)
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"zinfer_b200{BUILD_FOLDER}_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, building it first if necessary."""
    fp = _fingerprint()
    candidates = [os.path.join(HERE, BUILD_FOLDER)]
    tmp = os.path.join(tempfile.gettempdir(), f"zinfer_b200{BUILD_FOLDER}_{os.getuid()}")
    candidates.append(tmp)
    for d in candidates:
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "fingerprint")
        if os.path.exists(lib) and os.path.exists(stamp):
            with open(stamp) as f:
                if f.read().strip() == fp:
                    return lib
    if not build_if_needed:
        raise FileNotFoundError("the kernel library is not built")
    return build(verbose=verbose)


def build(verbose: bool = True) -> str:
    nvcc = _nvcc()
    out_dir = _build_dir()
    srcs = sources()
    fp = _fingerprint()
    t0 = time.time()

    def say(msg: str) -> None:
        if verbose:
            print(f"[zinfer_b200] {msg}", file=sys.stderr, flush=True)

    say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} (first use only)")
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(15.0):
            say(f"still compiling... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        def compile_one(src: str) -> str:
            obj = os.path.join(out_dir, os.path.splitext(src)[0] + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            say(f"compiled {src} ({time.time() - t0:.0f} s)")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp_lib = os.path.join(out_dir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", tmp_lib, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking the kernel library failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_lib, os.path.join(out_dir, LIB_NAME))  # atomic: concurrent builders do not clash
        with open(os.path.join(out_dir, "fingerprint"), "w") as f:
            f.write(fp)
    finally:
        done.set()
    say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return os.path.join(out_dir, LIB_NAME)


if __name__ == "__main__":
    print(build())
