"""Compiling the CUDA sources into shared libraries, and loading them.

Each library is built from the ``.cu`` files under ``wick_b200/csrc`` by one
``nvcc`` call for sm_100a and is loaded with ``ctypes``; its exported functions
follow a plain C convention (raw pointers, sizes, a stream; a non-zero return
code plus ``wick_last_error()``).  A library's file name carries a hash of its
sources, headers and flags, so an up-to-date build is found and an outdated one
is never used.  Libraries are built on first use; while ``nvcc`` runs, a line is
printed to stderr every few seconds.

Built files go to ``wick_b200/csrc/_build`` when that folder can be written
(so that they travel with the source tree) and to a per-user temporary folder
otherwise; ``WICK_B200_BUILD_DIR`` overrides both.
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
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("WICK_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (set CUDA_HOME or WICK_B200_NVCC); the CUDA kernels cannot be built")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        env = os.environ.get("WICK_B200_BUILD_DIR")
        cands = [env] if env else []
        cands.append(os.path.join(CSRC, "_build"))
        cands.append(os.path.join(tempfile.gettempdir(), f"wick_b200-build-{os.getuid()}"))
        for c in cands:
            if c and _writable_dir(c):
                _build_dir = c
                break
        else:
            raise BuildError(f"no writable build folder among {cands}")
    return _build_dir


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in list(sources) + _headers():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update("\0".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> Tuple[str, List[str], List[str]]:
    srcs = [os.path.join(CSRC, s) for s in sources]
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines]
    tag = _digest(srcs, flags)
    return os.path.join(build_dir(), f"{name}-{tag}.so"), srcs, flags


def _note(msg: str) -> None:
    print(f"wick_b200: {msg}", file=sys.stderr, flush=True)


def compile_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Build the library if its file is absent; return the file's path."""
    out, srcs, flags = library_path(name, sources, defines)
    if os.path.exists(out):
        return out
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(out):
                return out
            nvcc = find_nvcc()
            tmp = f"{out}.{os.getpid()}.tmp"
            cmd = [nvcc] + flags + ["-I", CSRC, "-o", tmp] + srcs
            if verbose:
                _note(f"compiling {name} for sm_100a ({', '.join(os.path.basename(s) for s in srcs)}) ...")
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def heartbeat():
                while not done.wait(10.0):
                    _note(f"still compiling {name} ({time.time() - t0:.0f} s)")

            hb = threading.Thread(target=heartbeat, daemon=True)
            if verbose:
                hb.start()
            log, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                try:
                    os.remove(tmp)
                except OSError:
                    pass
                raise BuildError(f"nvcc failed for {name} (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
            os.replace(tmp, out)
            # earlier builds of the same library (other source or flag hashes) are of no use any more
            prefix = f"{name}-"
            for f in os.listdir(os.path.dirname(out)):
                if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out) \
                        and len(f) == len(os.path.basename(out)):
                    try:
                        os.remove(os.path.join(os.path.dirname(out), f))
                    except OSError:
                        pass
            if verbose:
                _note(f"compiled {name} in {time.time() - t0:.0f} s -> {out}")
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            try:
                os.remove(lock_path)
            except OSError:
                pass


_loaded: Dict[str, ctypes.CDLL] = {}


def load_library(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = name + "|" + ",".join(defines)
    lib = _loaded.get(key)
    if lib is None:
        path = compile_library(name, sources, defines)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
        lib.wick_last_error.restype = ctypes.c_char_p
        _loaded[key] = lib
    return lib


def loaded_libraries() -> List[str]:
    return sorted(getattr(l, "_name", "?") for l in _loaded.values())
