"""Builds and loads the engine's native code.

Two libraries are built in-tree, at the first call that needs them, from ``csrc/``:

* ``libcbis_kernels.so``: the hand-written sm_100a CUDA kernels, ``extern "C"`` launchers
  called through ctypes with raw pointers and a stream (nvcc, ``compute_100a/sm_100a``);
* ``_cbis_host``: the host runtime (cache manager and scheduler), a C++17 module bound
  with pybind11 (g++; it needs no GPU, so CPU-only tests use it too).

A build is keyed by a hash of its sources and flags; a stale or missing library is rebuilt.
There is no fallback: a missing compiler or a failed build raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_CSRC = os.path.join(_PKG, "csrc")
_LOCK = threading.Lock()
_KERNELS = None
_OPTIONAL = None
_HOST = None

# Kernels that are options (off by default) live in a library of their own, built when first asked for: a first call
# compiles what the model in front of it needs, not what it might be told to try.
OPTIONAL_SOURCES = ("decode_layers.cu",)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[cbis_b200 build] {msg}", file=sys.stderr, flush=True)


def _build_dir() -> str:
    """In-tree ``kernels/_build``; a per-user temporary folder if the tree cannot be written."""
    d = os.path.join(_PKG, "kernels", "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"cbis_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _sources(sub: str, exts):
    root = os.path.join(_CSRC, sub)
    return sorted(os.path.join(root, f) for f in os.listdir(root) if f.endswith(exts))


def _digest(files, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _find(tool: str, extra_dirs=()) -> str:
    p = shutil.which(tool)
    if p:
        return p
    for d in extra_dirs:
        c = os.path.join(d, tool)
        if os.path.isfile(c):
            return c
    raise BuildError(f"'{tool}' was not found; it is needed to build the engine's native code")


def _run(cmd, what):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {what} failed:\n{' '.join(cmd)}\n{r.stdout}")


def build_kernels(verbose: bool = True, optional: bool = False) -> str:
    """Compiles the .cu files under csrc/kernels for sm_100a (``optional``: those of OPTIONAL_SOURCES, into a library
    of their own; else all the others); returns the library's path."""
    cus = [f for f in _sources("kernels", (".cu",)) if (os.path.basename(f) in OPTIONAL_SOURCES) == optional]
    deps = _sources("kernels", (".cuh", ".h")) + cus
    tag = _digest(deps, " ".join(NVCC_FLAGS))
    out_dir = _build_dir()
    lib = os.path.join(out_dir, "libcbis_kernels_optional.so" if optional else "libcbis_kernels.so")
    stamp = lib + ".hash"
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == tag:
        return lib
    nvcc = _find("nvcc", ("/usr/local/cuda/bin",))
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(cus)} CUDA files for sm_100a into {out_dir} (first call only)")
    objs = []

    def one(cu):
        obj = os.path.join(out_dir, os.path.basename(cu)[:-3] + f".{tag}.o")
        _run([nvcc, *NVCC_FLAGS, "-c", cu, "-o", obj], os.path.basename(cu))
        if verbose:
            _say(f"  {os.path.basename(cu)} done ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(one, cus))
    tmp = lib + f".tmp{os.getpid()}"
    _run([nvcc, "-shared", "-o", tmp, *objs], os.path.basename(lib))
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(tag)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    if verbose:
        _say(f"kernels built in {time.time() - t0:.0f} s")
    return lib


def build_host(verbose: bool = True) -> str:
    """Compiles the host runtime (cache manager, scheduler) into a pybind11 module."""
    import pybind11
    srcs = _sources("host", (".cpp",))
    deps = _sources("host", (".cpp", ".hpp", ".h"))
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
    tag = _digest(deps, " ".join(flags) + sys.version)
    out_dir = _build_dir()
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    lib = os.path.join(out_dir, "_cbis_host" + suffix)
    stamp = lib + ".hash"
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == tag:
        return lib
    gxx = _find("g++")
    t0 = time.time()
    if verbose:
        _say("compiling the host runtime (cache manager, scheduler)")
    tmp = lib + f".tmp{os.getpid()}"
    _run([gxx, *flags, f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
          *srcs, "-o", tmp], "_cbis_host")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(tag)
    if verbose:
        _say(f"host runtime built in {time.time() - t0:.0f} s")
    return lib


def host():
    """The pybind11 module of the host runtime (built on first use)."""
    global _HOST
    with _LOCK:
        if _HOST is None:
            path = build_host()
            spec = importlib.util.spec_from_file_location("_cbis_host", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _HOST = mod
        return _HOST


def optional_kernels() -> ctypes.CDLL:
    """The library of the kernels that are options (built on first use)."""
    global _OPTIONAL
    with _LOCK:
        if _OPTIONAL is None:
            _OPTIONAL = ctypes.CDLL(build_kernels(optional=True))
        return _OPTIONAL


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library (built on first use).  Raises if it cannot be built or loaded."""
    global _KERNELS
    with _LOCK:
        if _KERNELS is None:
            _KERNELS = ctypes.CDLL(build_kernels())
        return _KERNELS
