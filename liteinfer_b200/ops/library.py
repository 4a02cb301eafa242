"""Builds and loads the CUDA libraries of `liteinfer_b200/csrc`.

Each `.cu` file becomes one shared library `liteinfer_b200/_build/<name>.so`,
compiled with nvcc for sm_100a the first time something in it is called (or all
at once by `build_all`).  A library is rebuilt when its source, `common.cuh` or
the compile flags change.  The libraries export plain C functions taking device
pointers and a stream; they are loaded with ctypes, so nothing here needs
torch's extension machinery, a home directory or the network.

There is no fallback: when nvcc is missing, the compile fails or the library does
not load, the call raises `KernelLibraryError`.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
BUILD_DIR = Path(__file__).resolve().parent.parent / "_build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
    "-diag-suppress", "177",
]

# Source file (without .cu) of every library.
SOURCES = ("elementwise", "rope_cache", "attention_generic", "attention_mma", "attention_stream", "attention_tcgen05",
           "gemm_simt", "gemm_skinny", "gemm_skinny_static", "gemm_stream", "gemm_tcgen05", "sampling")


class KernelLibraryError(RuntimeError):
    """A CUDA library could not be built or loaded; there is no other path."""


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def find_nvcc() -> str:
    candidates = [os.environ.get("LITEINFER_NVCC")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(str(Path(root) / "bin" / "nvcc"))
    candidates.append(shutil.which("nvcc"))
    for c in candidates:
        if c and Path(c).is_file() and os.access(c, os.X_OK):
            return c
    raise KernelLibraryError("nvcc was not found (looked at LITEINFER_NVCC, CUDA_HOME, /usr/local/cuda, PATH); "
                             "liteinfer_b200 has no path that runs without its CUDA kernels")


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _stamp(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in [CSRC / f"{name}.cu", *_headers()]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return BUILD_DIR / f"{name}.so"


def is_current(name: str) -> bool:
    stamp_file = BUILD_DIR / f"{name}.stamp"
    return library_path(name).is_file() and stamp_file.is_file() and stamp_file.read_text() == _stamp(name)


def _compile(name: str, verbose: bool = True) -> None:
    src = CSRC / f"{name}.cu"
    if not src.is_file():
        raise KernelLibraryError(f"no such kernel source: {src}")
    nvcc = find_nvcc()
    try:
        BUILD_DIR.mkdir(parents=True, exist_ok=True)
    except OSError as error:
        raise KernelLibraryError(f"cannot create {BUILD_DIR}: {error}") from error
    tmp = BUILD_DIR / f".{name}.{os.getpid()}.so"
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), str(src), "-o", str(tmp)]
    if verbose:
        print(f"[liteinfer_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env={**os.environ, "TMPDIR": str(BUILD_DIR)})
    # Say that the compile is alive every few seconds: a first call may take a while.
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[liteinfer_b200] ... still compiling {src.name} ({time.time() - start:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelLibraryError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp, library_path(name))
    (BUILD_DIR / f"{name}.stamp").write_text(_stamp(name))
    if verbose:
        print(f"[liteinfer_b200] built {name}.so in {time.time() - start:.1f} s", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> Path:
    """Compile `name` if its library is missing or stale; return the library's path."""
    with _lock:
        if not is_current(name):
            _compile(name, verbose)
    return library_path(name)


def build_all(verbose: bool = True) -> list[Path]:
    """Compile every library (in parallel); used by `__graft_entry__.build` and the CLI."""
    from concurrent.futures import ThreadPoolExecutor

    stale = [n for n in SOURCES if not is_current(n)]
    if stale:
        with ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as pool:
            list(pool.map(lambda n: _compile(n, verbose), stale))
    return [library_path(n) for n in SOURCES]


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, building it first when needed."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    path = build(name)
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as error:
                raise KernelLibraryError(f"cannot load {path}: {error}") from error
            _loaded[name] = lib
    return lib
