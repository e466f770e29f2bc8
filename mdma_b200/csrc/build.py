"""Builds the CUDA libraries with nvcc for sm_100a and loads them with ctypes.

Each library is a group of `.cu` files compiled into one shared object with a
plain C interface.  A library is built the first time something needs it, so a
float32 engine never compiles the tensor-core kernels.  Objects are compiled in
parallel, a progress line is printed every few seconds, and the result is kept
under `csrc/_build/` (or a per-user folder in the temporary directory when the
package folder is read-only), keyed by a hash of sources and flags.
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

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

LIBRARIES = {
    # name: (sources, headers, link flags)
    "core": (["elementwise.cu", "gemm_simt.cu", "attention_simple.cu", "sampling.cu"], ["common.cuh"], []),
    "tensor": (["gemm_tcgen05.cu", "attention_mma.cu", "attention_tc.cu"], ["common.cuh", "ptx.cuh", "attention_mma.cuh"], []),
    "noalloc": (["attention_noalloc.cu"], ["common.cuh", "ptx.cuh", "attention_mma.cuh", "attention_noalloc.h"], []),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("MDMA_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $MDMA_NVCC, PATH and /usr/local/cuda/bin); "
                     "the engine has no fallback without its CUDA libraries")


def _build_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"mdma_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _hash(name: str) -> str:
    sources, headers, link = LIBRARIES[name]
    h = hashlib.sha256(" ".join(NVCC_FLAGS + link).encode())
    for f in sources + headers:
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libmdma_{name}-{_hash(name)}.so")


def build(name: str, verbose: bool = True) -> str:
    """Compile library `name` if its shared object is not there yet; return its path."""
    sources, _, link = LIBRARIES[name]
    if not sources:
        raise BuildError(f"library {name!r} has no sources")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    tag = os.path.basename(out)[:-3]
    say = (lambda m: print(f"[mdma_b200] {m}", file=sys.stderr, flush=True)) if verbose else (lambda m: None)
    say(f"compiling CUDA library '{name}' for sm_100a ({len(sources)} files) ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    procs = []
    for src in sources:
        obj = os.path.join(bdir, f"{tag}-{src[:-3]}.{os.getpid()}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
    last = time.time()
    pending = list(procs)
    while pending:
        pending = [p for p in pending if p[2].poll() is None]
        if pending and time.time() - last > 10:
            say(f"  still compiling {', '.join(p[0] for p in pending)} ({time.time() - t0:.0f} s)")
            last = time.time()
        time.sleep(0.2)
    objs = []
    for src, obj, proc in procs:
        log = proc.stdout.read().decode(errors="replace")
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{log}")
        objs.append(obj)
    tmp_out = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc, "-shared", "-o", tmp_out, *objs, *link]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    for obj in objs:
        try:
            os.remove(obj)
        except OSError:
            pass
    if res.returncode != 0:
        raise BuildError(f"linking {name} failed:\n{res.stdout.decode(errors='replace')}")
    os.replace(tmp_out, out)      # atomic: concurrent builders end with one good file
    for stale in os.listdir(bdir):      # older builds of this library
        if stale.startswith(f"libmdma_{name}-") and stale.endswith(".so") and stale != os.path.basename(out):
            try:
                os.remove(os.path.join(bdir, stale))
            except OSError:
                pass
    say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s")
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library; builds it on first use.  Raises if it cannot be had."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            lib.mdma_last_error.restype = ctypes.c_char_p
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> list[str]:
    return [build(n, verbose) for n, (srcs, _, _) in LIBRARIES.items() if srcs]
