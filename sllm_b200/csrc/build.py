"""Build the kernels into one shared library with nvcc, for sm_100a only.

The reference builds its kernels with one nvcc line into ``sllm_gpu.so``
(kernels/cuda/build.sh:15-18) and loads it with ctypes (kernels/_sllm_cuda.py).
Here every ``.cu`` file of this folder is compiled on its own (in parallel) and
linked into ``libsllm_b200.so`` beside the sources; a stamp of the sources' and
flags' hash decides whether anything has to be compiled.  The first caller
compiles; while it does, a line is printed now and then.  If the folder cannot be
written (a read-only install), the build goes to ``$SLLM_B200_BUILD_DIR`` or a
per-user temporary folder.
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
LIB_NAME = "libsllm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]
NVCC_FLAGS += os.environ.get("SLLM_NVCC_EXTRA", "").split()     # e.g. -DSLLM_PDL_EARLY=1 for an experiment


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("SLLM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found (looked at $SLLM_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                       "the kernels cannot be built")


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _out_dir() -> str:
    env = os.environ.get("SLLM_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    if _writable(HERE):
        return HERE
    d = os.path.join(tempfile.gettempdir(), f"sllm_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, compiling first if need be."""
    out = _out_dir()
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, LIB_NAME + ".stamp")
    want = _digest()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build:
        raise RuntimeError(f"{lib} is missing or stale and building was not allowed")
    _build(out, lib, stamp, want, verbose)
    return lib


def _say(msg: str) -> None:
    print(f"[sllm_b200 build] {msg}", file=sys.stderr, flush=True)


def _build(out: str, lib: str, stamp: str, want: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    objdir = os.path.join(out, "_build")
    os.makedirs(objdir, exist_ok=True)
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} (first call only) ...")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)                       # atomic: a concurrent reader sees old or new
        with open(stamp, "w") as f:
            f.write(want)
    finally:
        done.set()
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    print(library_path())
