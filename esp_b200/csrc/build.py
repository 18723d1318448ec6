"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each library is a handful of ``.cu`` files with ``extern "C"`` entry points
that take raw device pointers and a stream; Python reaches them through
ctypes.  A library is compiled the first time something asks for it, so a
process pays only for the kernels that its model and dtype need.  Objects and
``.so`` files go to ``_build/`` beside the sources when that folder can be
written, else to a per-user folder under the system's temporary directory.  A
stamp of the sources and flags decides whether a rebuild is needed.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ..errors import Backend

CSRC = Path(__file__).resolve().parent

# library name -> its sources.  Headers (*.cuh) are shared by all of them.
LIBRARIES = {
    "core": ["elementwise.cu", "gemm_simt.cu", "rope_kv.cu", "attn_simt.cu", "moe_route.cu", "sampling.cu"],
    # bfloat16 only: loaded when a model runs in bfloat16
    "bf16": ["gemm_skinny.cu", "attn_decode.cu", "attn_prefill.cu"],
    # TMA + tcgen05/TMEM products for steps with many rows (bfloat16 prefill)
    "tc05": ["gemm_tc05.cu", "attn_prefill_tc05.cu"],
}

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# further flags for a one-off build (e.g. -D switches of a kernel's tuning constants); part of the stamp, so a
# changed value rebuilds; use ESP_B200_BUILD_DIR to keep such a build apart from the ordinary one
NVCC_FLAGS += os.environ.get("ESP_B200_NVCC_FLAGS", "").split()

_loaded: dict = {}
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[esp_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("ESP_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise Backend("nvcc was not found (set ESP_B200_NVCC or put nvcc on PATH); the kernels cannot be compiled")


def build_dir() -> Path:
    override = os.environ.get("ESP_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"esp_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _stamp(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for src in sorted(LIBRARIES[name]) + sorted(p.name for p in CSRC.glob("*.cuh")):
        h.update(src.encode())
        h.update((CSRC / src).read_bytes())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return build_dir() / f"libesp_b200_{name}.so"


def build_library(name: str, verbose: bool = True) -> Path:
    """Compile ``name`` if its stamp is stale; returns the path of the .so."""
    if name not in LIBRARIES:
        raise Backend(f"unknown kernel library {name!r}")
    out_dir = build_dir()
    so = out_dir / f"libesp_b200_{name}.so"
    stamp_file = out_dir / f"{name}.stamp"
    want = _stamp(name)
    with open(out_dir / f"{name}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if so.is_file() and stamp_file.is_file() and stamp_file.read_text() == want:
            return so
        nvcc = find_nvcc()
        sources = LIBRARIES[name]
        if verbose:
            _say(f"compiling library '{name}' ({len(sources)} files) for sm_100a into {out_dir}")
        t0 = time.time()
        done = [0]

        def compile_one(src: str) -> Path:
            obj = out_dir / f"{name}__{Path(src).stem}.o"
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise Backend(f"nvcc failed on {src}:\n{proc.stderr[-4000:]}")
            done[0] += 1
            if verbose:
                _say(f"  {src} done ({done[0]}/{len(sources)}, {time.time() - t0:.0f} s)")
            return obj

        stop = threading.Event()

        def heartbeat():
            while not stop.wait(10.0):
                if verbose:
                    _say(f"  still compiling '{name}' ({done[0]}/{len(sources)} files done, {time.time() - t0:.0f} s)")

        beat = threading.Thread(target=heartbeat, daemon=True)
        beat.start()
        try:
            with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
                objs = list(pool.map(compile_one, sources))
        finally:
            stop.set()
        tmp = out_dir / f"libesp_b200_{name}.{os.getpid()}.tmp.so"
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-lcudart", "-lcuda"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise Backend(f"linking library '{name}' failed:\n{proc.stderr[-4000:]}")
        os.replace(tmp, so)
        stamp_file.write_text(want)
        if verbose:
            _say(f"library '{name}' ready in {time.time() - t0:.0f} s")
        return so


def load_library(name: str) -> ctypes.CDLL:
    """The compiled library, built first if needed.  Raises Backend, never
    falls back to anything else."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise Backend(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> list:
    return [build_library(name, verbose) for name in LIBRARIES]
