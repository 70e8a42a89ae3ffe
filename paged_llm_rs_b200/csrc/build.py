"""Compile the CUDA sources of this folder for sm_100a into one shared library.

The library is built in-tree (``csrc/_build/``) at the first call that needs it
and rebuilt when a source, a header or a flag changes.  Each ``.cu`` file is
compiled by its own ``nvcc`` process, several at a time, and a line is printed
to stderr as each one starts and ends, so a first call is never silent.  No
Python headers and no torch headers are involved: the library exports plain C
entry points (see the ``PLLM_EXPORT`` functions) that are called through ctypes
with device pointers.

If the package folder cannot be written to, ``PAGED_LLM_BUILD_DIR`` or a folder
under the system's temporary directory is used instead.
"""

from __future__ import annotations

import ctypes
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

from ..errors import KernelError

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]

# PAGED_LLM_NVCC_DEFINES="A=1 B" adds -DA=1 -DB to every compile (a build of its own, named by
# its own hash): PLLM_TRACE=1 makes the kernels stamp the time around their wait for the kernel
# before them, for a timeline of a step (read with pllm_trace_read_<file>).
NVCC_FLAGS += [f"-D{d}" for d in os.environ.get("PAGED_LLM_NVCC_DEFINES", "").split()]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _say(msg: str) -> None:
    print(f"[paged_llm_rs_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelError("nvcc was not found (CUDA_HOME, PATH, /usr/local/cuda): the CUDA kernels cannot be built, "
                      "and there is no fallback without them")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(os.path.join(HERE, p), "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def build_dir() -> str:
    env = os.environ.get("PAGED_LLM_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"paged_llm_rs_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelError(f"no writable build folder among {cands}")


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> None:
    t0 = time.time()
    _say(f"compiling {src} ...")
    tmp = f"{obj}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", tmp]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        sys.stderr.write(r.stderr)
    os.replace(tmp, obj)
    _say(f"compiled {src} in {time.time() - t0:.1f} s")


def library_path(verbose: bool = False) -> str:
    """Build what is missing and return the path of the shared library."""
    srcs = sources()
    hdr_digest = _digest(_headers(), " ".join(NVCC_FLAGS))
    out = build_dir()
    objs, todo = [], []
    for s in srcs:
        d = _digest([s], hdr_digest)
        obj = os.path.join(out, f"{s[:-3]}.{d}.o")
        objs.append(obj)
        if not os.path.exists(obj):
            todo.append((s, obj))
    lib = os.path.join(out, f"libpllm_kernels.{_digest(srcs, hdr_digest)}.so")
    if os.path.exists(lib) and not todo:
        return lib
    nvcc = find_nvcc()
    if todo:
        _say(f"{len(todo)} CUDA source file(s) to compile for sm_100a into {out}")
        workers = max(1, min(len(todo), (os.cpu_count() or 2)))
        with ThreadPoolExecutor(workers) as pool:
            for f in [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in todo]:
                f.result()
    tmp = f"{lib}.{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp] + objs + ["-lcuda"], capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelError(f"linking the kernel library failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    _say(f"linked {os.path.basename(lib)}")
    # drop objects and libraries of older sources
    keep = {os.path.basename(p) for p in objs + [lib]}
    for f in os.listdir(out):
        if f.endswith((".o", ".so")) and f not in keep:
            try:
                os.remove(os.path.join(out, f))
            except OSError:
                pass
    return lib


def load_library() -> ctypes.CDLL:
    """The kernel library, built if need be.  Raises KernelError when it cannot be
    had; nothing in the engine runs without it."""
    global _lib
    with _lock:
        if _lib is None:
            path = library_path()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"loading {path} failed: {e}") from e
        return _lib


if __name__ == "__main__":
    print(library_path(verbose="-v" in sys.argv))
