"""Compiles the CUDA sources under ``csrc/`` for sm_100a and loads them with ctypes.

Each ``csrc/<name>.cu`` becomes one shared library
``_build/<name>[-<macros>]-<hash>.so`` next to the package (in-tree, so a built
library travels with the source folder).  A library is compiled at the first call
that needs it; the hash covers the source, the headers it includes from ``csrc/``,
the flags and the macros, so an edit rebuilds it.  While nvcc runs, a line is
printed now and then.

If the package folder cannot be written, ``$BLACKWELLLLM_B200_BUILD_DIR`` or a
per-user temporary folder is used.  There is no fallback to another
implementation: a missing compiler or a failed build raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Mapping, Optional

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels of blackwellllm_b200 cannot be built")


def build_dir() -> str:
    env = os.environ.get("BLACKWELLLLM_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(_PKG, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"blackwellllm_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".w"):
                pass
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _source_hash(path: str, flags, macros: Mapping[str, object]) -> str:
    h = hashlib.sha256()
    seen = set()

    def add(p):
        if p in seen or not os.path.isfile(p):
            return
        seen.add(p)
        with open(p, "rb") as f:
            data = f.read()
        h.update(os.path.basename(p).encode())
        h.update(data)
        for inc in re.findall(rb'#include\s+"([^"]+)"', data):
            add(os.path.join(os.path.dirname(p), inc.decode()))

    add(path)
    h.update(repr(list(flags)).encode())
    h.update(repr(sorted(macros.items())).encode())
    return h.hexdigest()[:16]


def _tag(macros: Mapping[str, object]) -> str:
    if not macros:
        return ""
    return "-" + "_".join(f"{k.lower()}{v}" for k, v in sorted(macros.items()))


def library_path(name: str, macros: Optional[Mapping[str, object]] = None,
                 extra_flags=()) -> str:
    macros = dict(macros or {})
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no such kernel source: {src}")
    flags = ARCH_FLAGS + BASE_FLAGS + list(extra_flags)
    return os.path.join(build_dir(), f"{name}{_tag(macros)}-{_source_hash(src, flags, macros)}.so")


def compile_library(name: str, macros: Optional[Mapping[str, object]] = None,
                    extra_flags=(), verbose: bool = True) -> str:
    """Builds (if needed) and returns the path of the shared library of ``csrc/<name>.cu``."""
    macros = dict(macros or {})
    out = library_path(name, macros, extra_flags)
    if os.path.isfile(out):
        return out
    src = os.path.join(CSRC, name + ".cu")
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + BASE_FLAGS + list(extra_flags)
    cmd += [f"-D{k}={v}" for k, v in sorted(macros.items())]
    cmd += ["-I", CSRC, "-o", tmp, src]
    label = name + _tag(macros)
    if verbose:
        print(f"[blackwellllm_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                print(f"[blackwellllm_b200] ... still compiling {label} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed for {label} (exit {proc.returncode}):\n"
                         f"{' '.join(cmd)}\n{log.decode(errors='replace')}")
    os.replace(tmp, out)
    if verbose:
        print(f"[blackwellllm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def load_library(name: str, macros: Optional[Mapping[str, object]] = None,
                 extra_flags=()) -> ctypes.CDLL:
    key = name + _tag(dict(macros or {})) + "|" + " ".join(extra_flags)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, macros, extra_flags)
            lib = ctypes.CDLL(path)
            _loaded[key] = lib
        return lib


# ------------------------------------------------------------------ host libraries (no GPU code)
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def find_cxx() -> str:
    for c in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        if c and shutil.which(c):
            return shutil.which(c)
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++); the host runtime of "
                     "blackwellllm_b200 cannot be built")


def compile_host_library(name: str, verbose: bool = True) -> str:
    """Builds (if needed) ``csrc/<name>.cpp`` with the host compiler; returns the library's path."""
    src = os.path.join(CSRC, name + ".cpp")
    if not os.path.isfile(src):
        raise BuildError(f"no such source: {src}")
    out = os.path.join(build_dir(), f"{name}-{_source_hash(src, HOST_FLAGS, {})}.so")
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [find_cxx()] + HOST_FLAGS + ["-I", CSRC, "-o", tmp, src]
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"the host compiler failed for {name} (exit {proc.returncode}):\n"
                         f"{' '.join(cmd)}\n{proc.stdout.decode(errors='replace')}")
    os.replace(tmp, out)
    if verbose:
        print(f"[blackwellllm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def load_host_library(name: str) -> ctypes.CDLL:
    key = "host|" + name
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_host_library(name))
            _loaded[key] = lib
        return lib
