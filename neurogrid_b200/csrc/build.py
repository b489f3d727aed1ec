"""Builds the CUDA sources of this folder for sm_100a, one shared library per source file.

A library is compiled the first time something needs it (``load("shortconv")``) and is kept
in ``csrc/_build`` (or, if the package folder is read-only, in a per-user folder under the
system's temporary directory; ``NEUROGRID_B200_BUILD_DIR`` overrides both).  The file name
carries a hash of the source, of the shared header, of the compile flags and of the
``-D`` specialisation, so an edited source or another head size never loads a stale binary.
While nvcc runs, a line is printed now and then so that a first call does not look hung.

The launchers have a C ABI and are reached through ``ctypes``: no binding layer has to be
compiled, which keeps a cold build to seconds per file.
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
from typing import Dict, Mapping, Optional, Sequence, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]

# name -> extra link flags
SOURCES: Dict[str, Sequence[str]] = {
    "elementwise": (), "gemm_f32": (), "shortconv": (), "rope_cache": (),
    "attention_generic": (), "sampling": (), "attention_bf16": (),
    "gemm_sm100": (),
    "attention_sm100": (),
}

_lock = threading.RLock()
_loaded: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("NEUROGRID_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or NEUROGRID_B200_NVCC); the kernels of this "
                     "package are compiled from source and there is no other code path")


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        with _lock:
            if _build_dir is None:
                _build_dir = _find_build_dir()
    return _build_dir


def _find_build_dir() -> str:
    env = os.environ.get("NEUROGRID_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"neurogrid_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}.{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(name: str, defines: Mapping[str, object]) -> str:
    h = hashlib.sha256()
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith((".cuh", ".h")) or fn == name + ".cu":
            with open(os.path.join(HERE, fn), "rb") as f:
                h.update(fn.encode() + b"\0" + f.read())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS + list(SOURCES.get(name, ()))).encode())
    h.update(repr(sorted((k, str(v)) for k, v in defines.items())).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: Optional[Mapping[str, object]] = None) -> str:
    defines = defines or {}
    tag = "".join(f"-{k}{v}" for k, v in sorted(defines.items()))
    return os.path.join(build_dir(), f"ng_{name}{tag}-{_digest(name, defines)}.so")


def compile_library(name: str, defines: Optional[Mapping[str, object]] = None, *, verbose: bool = True) -> str:
    """Compile ``<name>.cu`` if its library is not there yet; returns the library's path."""
    defines = defines or {}
    src = os.path.join(HERE, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no such kernel source: {src}")
    out = library_path(name, defines)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc_path(), *ARCH_FLAGS, *BASE_FLAGS, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           "-I", HERE, *SOURCES.get(name, ()), "-o", tmp, src]
    spec = (" " + " ".join(f"{k}={v}" for k, v in sorted(defines.items()))) if defines else ""
    if verbose:
        print(f"[neurogrid_b200] compiling {name}.cu{spec} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=HERE)
    log: list = []
    reader = threading.Thread(target=lambda: log.append(proc.stdout.read()), daemon=True)
    reader.start()
    beat = t0
    while proc.poll() is None:
        time.sleep(0.2)
        if verbose and time.time() - beat > 10:
            beat = time.time()
            print(f"[neurogrid_b200]   ... still compiling {name}.cu ({beat - t0:.0f} s)", file=sys.stderr, flush=True)
    reader.join()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed for {name}.cu:\n{' '.join(cmd)}\n{''.join(log)}")
    os.replace(tmp, out)
    stem = os.path.basename(out).rsplit("-", 1)[0] + "-"
    for fn in os.listdir(os.path.dirname(out)):               # older builds of the same source and specialisation
        if fn.startswith(stem) and fn.endswith(".so") and fn != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[neurogrid_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load(name: str, defines: Optional[Mapping[str, object]] = None) -> ctypes.CDLL:
    """The library for ``name`` (+ specialisation), compiled on first use."""
    key = (name, tuple(sorted((k, str(v)) for k, v in (defines or {}).items())))
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name, defines))
            _loaded[key] = lib
    return lib


def compile_many(jobs: Sequence[Tuple[str, Optional[Mapping[str, object]]]], *, verbose: bool = True) -> None:
    """Compile several libraries side by side (nvcc is single-threaded per file)."""
    jobs = [(n, d) for n, d in jobs if not os.path.isfile(library_path(n, d))]
    if not jobs:
        return
    with ThreadPoolExecutor(max_workers=min(len(jobs), max(1, (os.cpu_count() or 2)))) as pool:
        list(pool.map(lambda j: compile_library(j[0], j[1], verbose=verbose), jobs))


def build_all(extra: Sequence[Tuple[str, Mapping[str, object]]] = (), *, verbose: bool = True) -> None:
    """Every unspecialised library plus the given specialisations."""
    compile_many([(n, None) for n in SOURCES if n not in SPECIALISED] + list(extra), verbose=verbose)


# sources that only exist as ``-D`` specialisations (never built bare)
SPECIALISED: Dict[str, Sequence[str]] = {"attention_bf16": ("NG_HEAD_DIM",), "shortconv": ("NG_CONV_L",),
                                         "rope_cache": ("NG_ROPE_PAIRS",)}
