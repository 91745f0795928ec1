"""Native code: build and load.

Two shared objects are built in-tree under ``noeira_b200/_lib``:

* ``libnoeira_b200.so``      — every ``csrc/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); exported symbols are plain ``extern "C"``
  launchers that take raw device pointers and a ``cudaStream_t``.
* ``libnoeira_b200_host.so`` — every ``csrc/host/*.cpp`` compiled by g++ (checkpoint/safetensors
  I/O, SPSC rings and worker threads, serial/HTTP shims, the CPU physics oracle...).

Both are loaded with ``ctypes``; there is no pybind layer, so a kernel file rebuilds in seconds and
the same symbols are callable from C, C++ or Python.  On a machine with a GPU a missing CUDA library
is an error (ops never silently fall back to eager PyTorch).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
LIBDIR = _PKG / "_lib"
CUDA_LIB = LIBDIR / "libnoeira_b200.so"
# the same sources compiled with -DNB_BOUNDS=1 (index-driven kernels test their indices; see csrc/common.cuh);
# selected with NOEIRA_B200_BOUNDS=1
CUDA_LIB_BOUNDS = LIBDIR / "libnoeira_b200_bounds.so"
HOST_LIB = LIBDIR / "libnoeira_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
GXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-Wall"]

_lock = threading.Lock()
_cuda = None
_host = None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, log: Path):
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"native build failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r


def _build_one(srcs, headers, objdir: Path, compiler_cmd, suffix: str):
    """Compile each source whose digest (source + all headers + flags) changed; return object list."""
    objdir.mkdir(parents=True, exist_ok=True)
    hdr_digest = _digest(headers, " ".join(compiler_cmd))
    jobs = []
    objs = []
    for s in srcs:
        o = objdir / (s.stem + ".o")
        stamp = objdir / (s.stem + ".sha")
        d = hashlib.sha256((hdr_digest + s.read_text()).encode()).hexdigest()
        objs.append(o)
        if o.exists() and stamp.exists() and stamp.read_text() == d:
            continue
        jobs.append((s, o, stamp, d))

    def go(job):
        s, o, stamp, d = job
        _run(compiler_cmd + ["-c", str(s), "-o", str(o)], objdir / (s.stem + ".log"))
        stamp.write_text(d)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(go, jobs))
    return objs, bool(jobs)


def build(force: bool = False, verbose: bool = False) -> None:
    """Compile every CUDA and C++ source in-tree (cross-compiles without a GPU)."""
    with _lock:
        LIBDIR.mkdir(exist_ok=True)
        if force:
            shutil.rmtree(LIBDIR / "obj", ignore_errors=True)
        cu = sorted(CSRC.glob("*.cu"))
        hdr = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted((CSRC / "host").glob("*.h"))
        if cu:
            for lib, objdir, extra in ((CUDA_LIB, "cuda", []), (CUDA_LIB_BOUNDS, "cuda_bounds", ["-DNB_BOUNDS=1"])):
                nv = [_nvcc()] + NVCC_FLAGS + extra + ["-I", str(CSRC)]
                objs, changed = _build_one(cu, hdr, LIBDIR / "obj" / objdir, nv, ".cu")
                if changed or not lib.exists():
                    _run([_nvcc(), "-shared", "-o", str(lib)] + [str(o) for o in objs]
                         + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-lpthread", "-ldl"],
                         LIBDIR / "obj" / f"link_{objdir}.log")
        cpp = sorted((CSRC / "host").glob("*.cpp"))
        if cpp:
            gx = [shutil.which("g++") or "g++"] + GXX_FLAGS + ["-I", str(CSRC), "-I", str(CSRC / "host")]
            objs, changed = _build_one(cpp, hdr, LIBDIR / "obj" / "host", gx, ".cpp")
            if changed or not HOST_LIB.exists():
                _run([gx[0], "-shared", "-o", str(HOST_LIB)] + [str(o) for o in objs] + ["-pthread", "-ldl", "-lz", "-lssl", "-lcrypto"],
                     LIBDIR / "obj" / "link_host.log")
        if verbose:
            for log in sorted((LIBDIR / "obj" / "cuda").glob("*.log")):
                sys.stdout.write(log.read_text())


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel as printed by ``-Xptxas -v`` at build time."""
    out = []
    for log in sorted((LIBDIR / "obj" / "cuda").glob("*.log")):
        out.append(f"== {log.stem}\n{log.read_text()}")
    return "\n".join(out)


def _autobuild_allowed() -> bool:
    return os.environ.get("NOEIRA_B200_NO_AUTOBUILD", "0") != "1"


def host_lib() -> ctypes.CDLL:
    """The C++ host runtime (always available; built on demand)."""
    global _host
    if _host is None:
        if not HOST_LIB.exists() and _autobuild_allowed():
            build()
        _host = ctypes.CDLL(str(HOST_LIB))
    return _host


def cuda_lib() -> ctypes.CDLL:
    """The sm_100a kernel library.  Raises if it cannot be loaded — there is no eager fallback."""
    global _cuda
    if _cuda is None:
        bounds = os.environ.get("NOEIRA_B200_BOUNDS", "0") == "1"
        lib = CUDA_LIB_BOUNDS if bounds else CUDA_LIB
        if not lib.exists() and _autobuild_allowed():
            build()
        if not lib.exists():
            raise RuntimeError(f"{lib} is missing: run `python -m noeira_b200.build`")
        _cuda = ctypes.CDLL(str(lib))
        _cuda._bounds_registered = set()
    return _cuda


def register_bounds_status(status_tensor) -> int:
    """Bounds-checked build only: point every translation unit's bounds reporter at the device status word of the
    CURRENT device.  Returns how many units were registered (0 in the normal build)."""
    lib = cuda_lib()
    if os.environ.get("NOEIRA_B200_BOUNDS", "0") != "1":
        return 0
    key = status_tensor.data_ptr()
    if key in lib._bounds_registered:
        return 0
    n = 0
    for tu in ("misc_ops", "replay", "ppo_kernels"):
        fn = getattr(lib, f"nb_bounds_register_{tu}", None)
        if fn is not None:
            check(fn(ctypes.c_void_p(key)), f"bounds_register_{tu}")
            n += 1
    lib._bounds_registered.add(key)
    return n


def have_cuda_lib() -> bool:
    return CUDA_LIB.exists()


class NativeError(RuntimeError):
    pass


_ERRS = {10001: "bad argument", 10002: "unaligned pointer/extent", 10003: "size beyond supported maximum",
         10004: "driver symbol not found", 10005: "cuTensorMapEncodeTiled failed"}


_LAUNCHES = 0


def launch_count() -> int:
    """Number of launcher calls made through `check` (graph replays add their captured count)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def check(rc: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if rc != 0:
        msg = _ERRS.get(rc)
        if msg is None:
            msg = f"cudaError {rc}"
        raise NativeError(f"{what}: {msg}")


def ptr(t) -> ctypes.c_void_p:
    """Raw device/host pointer of a torch tensor (None → NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr(stream=None) -> ctypes.c_void_p:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)
