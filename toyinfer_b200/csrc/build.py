"""Builds the CUDA kernels of this package into one shared library with nvcc.

``ensure_built()`` returns the path of ``libtoyinfer_kernels.so``, compiling first when
the library is missing or older than its sources (a hash of sources and flags is kept
beside it).  Every ``.cu`` file is compiled for sm_100a only, files in parallel, and a
line is printed when each file starts and every few seconds while the compiler runs, so
that a first call on a fresh checkout does not look hung.  The library is built in-tree
under ``csrc/_build``; when that folder cannot be written (a read-only checkout) it goes
to a per-user folder under the system's temporary directory.
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
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libtoyinfer_kernels.so"
MEASURE_LIB_NAME = "libtoyinfer_measure.so"      # measurement kernels (csrc/measure), built only when asked for
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "--expt-extended-lambda",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[toyinfer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("TOYINFER_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at TOYINFER_NVCC, CUDA_HOME, PATH, /usr/local/cuda/bin)")


def sources() -> List[str]:
    return sorted(os.path.join(HERE, n) for n in os.listdir(HERE) if n.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(HERE, n) for n in os.listdir(HERE) if n.endswith((".cuh", ".h")))


def measure_sources() -> List[str]:
    d = os.path.join(HERE, "measure")
    return sorted(os.path.join(d, n) for n in os.listdir(d) if n.endswith(".cu"))


def source_hash(srcs=None) -> str:
    h = hashlib.sha256()
    for p in (sources() if srcs is None else srcs) + _headers():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"toyinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> None:
    cmd = [nvcc, "-c", src, "-o", obj, "-I", HERE] + ARCH_FLAGS + NVCC_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    _say(f"compiling {os.path.basename(src)} for sm_100a")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)


def build(force: bool = False, verbose: bool = False, measure: bool = False) -> str:
    """Compiles the kernels (or, with ``measure``, the measurement kernels of csrc/measure) and
    returns the library's path."""
    out_dir = _build_dir()
    name = MEASURE_LIB_NAME if measure else LIB_NAME
    lib = os.path.join(out_dir, name)
    stamp = os.path.join(out_dir, "measure.hash" if measure else "source.hash")
    want = source_hash(measure_sources() if measure else None)
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    nvcc = find_nvcc()
    srcs = measure_sources() if measure else sources()
    objs = [os.path.join(out_dir, ("measure_" if measure else "") + os.path.basename(s)[:-3] + ".o") for s in srcs]
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        # the longest compiles start first; the text a file pulls in from this folder stands for its time
        order = sorted(range(len(srcs)), key=lambda i: -_text_size(srcs[i]))
        with ThreadPoolExecutor(max_workers=min(max(4, os.cpu_count() or 4), len(srcs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, srcs[i], objs[i], verbose) for i in order]
            for f in futs:
                f.result()
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-o", tmp] + objs + ARCH_FLAGS + ["-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {name} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(want)
    finally:
        done.set()
    _say(f"built {name} in {time.time() - t0:.0f} s")
    return lib


def _text_size(path: str, seen=None) -> int:
    """Bytes of a source file and of the headers of this folder that it includes."""
    seen = set() if seen is None else seen
    if path in seen or not os.path.isfile(path):
        return 0
    seen.add(path)
    with open(path, errors="replace") as f:
        text = f.read()
    total = len(text)
    for line in text.splitlines():
        line = line.strip()
        if line.startswith('#include "'):
            total += _text_size(os.path.join(HERE, line.split('"')[1]), seen)
    return total


def ensure_built() -> str:
    return build(force=False)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
