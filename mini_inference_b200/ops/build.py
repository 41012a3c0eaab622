"""Builds the CUDA sources under csrc/ into one shared library next to the package, for
sm_100a only, with nvcc directly (no JIT cache outside the tree, nothing needed from the
network or from HOME).  The library is rebuilt when a source changed; otherwise it is loaded
as it lies.  The first call of a fresh checkout compiles, printing a line per source file."""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")


def _out_dir() -> str:
    """The package folder; a per-user folder under the temporary directory when the checkout
    is read-only for this user."""
    if os.access(PKG, os.W_OK):
        return PKG
    import tempfile
    d = os.path.join(tempfile.gettempdir(), f"mini_inference_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


BUILD = os.path.join(_out_dir(), "_build")
LIB = os.path.join(_out_dir(), "_kernels.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
NVCC_FLAGS += os.environ.get("MI_NVCC_EXTRA", "").split()        # e.g. -DMI_ATT_TIMING for the kernels' phase counters


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels of mini_inference_b200 cannot be built")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    return h.hexdigest()


def _log(msg):
    print(f"[mini_inference_b200 build] {msg}", file=sys.stderr, flush=True)


def is_current() -> bool:
    stamp = os.path.join(BUILD, "stamp.json")
    if not (os.path.isfile(LIB) and os.path.isfile(stamp)):
        return False
    try:
        with open(stamp) as f:
            return json.load(f).get("digest") == _digest()
    except (OSError, ValueError):
        return False


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every .cu under csrc/ (in parallel) and link _kernels.so.  Returns its path."""
    if not force and is_current():
        return LIB
    nvcc = _nvcc()
    os.makedirs(BUILD, exist_ok=True)
    sources = _sources()
    t0 = time.time()
    if verbose:
        _log(f"compiling {len(sources)} CUDA sources for sm_100a with {nvcc} (first call only)")

    def compile_one(src):
        obj = os.path.join(BUILD, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _log(f"  compiled {src} ({time.time() - t0:.0f}s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, sources))
    tmp = LIB + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking _kernels.so failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    with open(os.path.join(BUILD, "stamp.json"), "w") as f:
        json.dump({"digest": _digest(), "sources": sources}, f)
    if verbose:
        _log(f"built {LIB} in {time.time() - t0:.0f}s")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv)
