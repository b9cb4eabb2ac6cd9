"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each ``name.cu`` becomes ``_build/libsb_name.so`` next to the sources (or, if that
folder cannot be written, under the system temp folder), built by ``nvcc`` the
first time a kernel of that file is needed and again whenever the source, the
shared header or the flags change.  The libraries export plain C entry points
and are loaded with ``ctypes``; nothing links against torch, so a build takes
seconds.  There is no other implementation behind these entry points: if a
library can be neither found nor built, the call fails.
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

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]

#: every kernel source of the library; ``build_all`` compiles all of them
SOURCES = (
    "elementwise",
    "rope_cache",
    "attention_rowwise",
    "attention_decode",
    "attention_decode_mma",
    "attention_decode_noalloc",
    "attention_prefill",
    "attention_prefill_tc",
    "linear_small",
    "sgemm",
    "gemm_tcgen05",
    "gemm_prompt_tcgen05",
    "dense_chain",
    "sampling",
)

_lock = threading.Lock()
_loaded: dict = {}


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the CUDA kernels of "
        "starter_b200 cannot be built and there is no other implementation to fall back to"
    )


_dir_lock = threading.Lock()
_dir = None


def _build_dir() -> str:
    global _dir
    with _dir_lock:
        if _dir is not None:
            return _dir
        local = os.path.join(HERE, "_build")
        try:
            os.makedirs(local, exist_ok=True)
            probe = os.path.join(local, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            _dir = local
        except OSError:
            _dir = os.path.join(tempfile.gettempdir(), f"starter_b200_build_{os.getuid()}")
            os.makedirs(_dir, exist_ok=True)
        return _dir


def _headers() -> list:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _included_sources(name: str) -> list:
    """Other ``.cu`` files of this folder that ``name.cu`` includes."""
    found = []
    with open(os.path.join(HERE, name + ".cu"), "r", encoding="utf-8") as handle:
        for line in handle:
            line = line.strip()
            if line.startswith("#include \"") and line.endswith(".cu\""):
                found.append(line[len("#include \""):-1])
    return found


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fname in [name + ".cu"] + _included_sources(name) + _headers():
        with open(os.path.join(HERE, fname), "rb") as handle:
            h.update(fname.encode())
            h.update(handle.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    """Path of the built library for ``name.cu``, compiling it first if it is missing or stale."""
    src = os.path.join(HERE, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    out_dir = _build_dir()
    lib = os.path.join(out_dir, f"libsb_{name}.so")
    stamp = lib + ".stamp"
    digest = _digest(name)
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as handle:
            if handle.read().strip() == digest:
                return lib
    tmp = f"{lib}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", HERE, "-o", tmp, src]
    print(f"[starter_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    started = time.monotonic()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            print(f"[starter_b200] ... still compiling {name}.cu "
                  f"({time.monotonic() - started:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {name}.cu:\n{out}")
    os.replace(tmp, lib)
    with open(stamp, "w") as handle:
        handle.write(digest)
    print(f"[starter_b200] built {os.path.basename(lib)} in {time.monotonic() - started:.1f} s",
          file=sys.stderr, flush=True)
    return lib


def load(name: str) -> ctypes.CDLL:
    """The loaded library of ``name.cu`` (built on first use)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(library_path(name))
            _loaded[name] = lib
        return lib


def build_all(names=SOURCES) -> list:
    """Compile every kernel source (in parallel) and return the library paths."""
    results = {}
    errors = []

    def work(n):
        try:
            results[n] = library_path(n)
        except Exception as exc:  # noqa: BLE001 - collected and re-raised below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return [results[n] for n in names]
