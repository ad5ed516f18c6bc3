"""Build and load ``libfluxb.so`` — the native half of the package.

All device code and the C++ runtime live under ``csrc/``; they are compiled with plain
``nvcc`` for ``sm_100a`` into one shared library that sits inside the package directory, and
Python talks to it through ``ctypes`` (no torch C++ headers are involved, so a full rebuild
takes seconds). The reference instead builds ``libflux_cuda.so`` through CMake plus seven code
generators and binds it with pybind11 (reference: ``build.sh``, ``src/pybind/ths_op.cc``).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
_CSRC = _ROOT / "csrc"
_LIBDIR = _PKG / "_lib"
_LIB = _LIBDIR / "libfluxb.so"
_OBJDIR = _ROOT / "build" / "obj"
# the self-checking build (FLUXB_DEBUG=1): same sources with -DFLUXB_DEBUG_CHECKS, see
# csrc/sm100/ptx.cuh::dcheck
_LIB_DEBUG = _LIBDIR / "libfluxb_debug.so"
_OBJDIR_DEBUG = _ROOT / "build" / "obj_debug"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]

_lock = threading.Lock()
_handle = None


class NativeError(RuntimeError):
    """Raised when a libfluxb entry point reports a failure."""


def _nvcc() -> str:
    for cand in (os.environ.get("FLUXB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise NativeError("nvcc not found; set FLUXB_NVCC")


def sources() -> list[Path]:
    out = []
    for pat in ("**/*.cu", "**/*.cc"):
        out.extend(sorted(_CSRC.glob(pat)))
    return out


def debug_enabled() -> bool:
    return os.environ.get("FLUXB_DEBUG", "0") not in ("", "0")


def _headers_digest(flags) -> str:
    h = hashlib.sha1()
    for pat in ("**/*.cuh", "**/*.h"):
        for f in sorted(_CSRC.glob(pat)):
            h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> Path:
    """Compile every source under ``csrc/`` for sm_100a and link ``_lib/libfluxb.so``
    (``debug``: ``_lib/libfluxb_debug.so`` with the device-side self-checks compiled in).

    Incremental: an object is rebuilt when its source, any header or the flags changed.
    """
    nvcc = _nvcc()
    objdir = _OBJDIR_DEBUG if debug else _OBJDIR
    target = _LIB_DEBUG if debug else _LIB
    flags = NVCC_FLAGS + (["-DFLUXB_DEBUG_CHECKS=1"] if debug else [])
    objdir.mkdir(parents=True, exist_ok=True)
    _LIBDIR.mkdir(parents=True, exist_ok=True)
    hdig = _headers_digest(flags)
    jobs = []
    objs = []
    for src in sources():
        rel = src.relative_to(_CSRC)
        obj = objdir / (str(rel).replace("/", "__") + ".o")
        stamp = obj.with_suffix(".stamp")
        dig = hashlib.sha1(src.read_bytes() + hdig.encode()).hexdigest()
        objs.append(obj)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
            continue
        jobs.append((src, obj, stamp, dig))

    def compile_one(job):
        src, obj, stamp, dig = job
        cmd = [nvcc, *flags, "-I", str(_CSRC / "include"), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise NativeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and (r.stdout or r.stderr):
            print(r.stdout, r.stderr)
        stamp.write_text(dig)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not target.exists() or force:
        tmp = target.with_suffix(".so.tmp%d" % os.getpid())
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static",
               "-Xcompiler", "-fPIC", "-lrt", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise NativeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, target)
    return target


def lib() -> ctypes.CDLL:
    """The loaded library (built first if the shared object is missing)."""
    global _handle
    if _handle is not None:
        return _handle
    with _lock:
        if _handle is None:
            dbg = debug_enabled()
            path = _LIB_DEBUG if dbg else _LIB
            if not path.exists():
                build(debug=dbg)
            h = ctypes.CDLL(str(path))
            h.fluxb_last_error.restype = ctypes.c_char_p
            h.fluxb_launch_count.restype = ctypes.c_uint64
            _handle = h
    return _handle


def check(rc: int, what: str = "libfluxb call") -> None:
    if rc != 0:
        msg = lib().fluxb_last_error().decode(errors="replace")
        raise NativeError(f"{what} failed (code {rc}): {msg}")


def launch_count() -> int:
    return int(lib().fluxb_launch_count())
