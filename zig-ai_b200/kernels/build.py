"""Compiling and loading the CUDA kernels under csrc/.

Every `csrc/<name>.cu` becomes one shared library `lib<name>.so` with a plain C interface, built
with `nvcc -gencode arch=compute_100a,code=sm_100a` and loaded with ctypes.  (The reference compiles
its `.cu` files to cubins for the detected architecture at build time and loads them with
`cuModuleLoad`, build.zig:52-86, src/cuda/layer_kernels.zig:19-27.)  A library is built the first
time it is needed, or when its source, a header or the flags changed; the build prints a line
when it starts and every few seconds while the compiler runs.  Libraries live beside the sources
in `csrc/_build/` when that folder can be written, else in a per-user temporary folder.
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
from typing import Dict, List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]
# ZAI_TIMELINE=1: kernels note the global timer around their dependency wait (csrc/common.cuh); these
# libraries are kept in a folder of their own
TIMELINE = os.environ.get("ZAI_TIMELINE", "0") == "1"
if TIMELINE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DZAI_TIMELINE"]
EXTRA_FLAGS: Dict[str, List[str]] = {}
EXTRA_LIBS: Dict[str, List[str]] = {}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def find_nvcc() -> str:
    cands = [os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be compiled")


_lib_dir = None


def lib_dir() -> str:
    global _lib_dir
    with _dir_lock:
        if _lib_dir is None:
            _lib_dir = _find_lib_dir()
        return _lib_dir


def _find_lib_dir() -> str:
    d = os.path.join(CSRC, "_build_timeline" if TIMELINE else "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"zig_ai_b200_{os.getuid()}", "_build_timeline" if TIMELINE else "_build")
        os.makedirs(d, exist_ok=True)
        return d


def source_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS.get(name, []) + EXTRA_LIBS.get(name, [])).encode())
    for f in [name + ".cu"] + sorted(x for x in os.listdir(CSRC) if x.endswith((".cuh", ".h"))):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()


def lib_path(name: str) -> str:
    return os.path.join(lib_dir(), f"lib{name}.so")


def is_current(name: str) -> bool:
    p = lib_path(name)
    try:
        with open(p + ".hash") as f:
            return os.path.isfile(p) and f.read().strip() == source_hash(name)
    except OSError:
        return False


def compile_one(name: str, verbose: bool = True) -> str:
    """Compile csrc/<name>.cu; returns the library's path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    out = lib_path(name)
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [find_nvcc()] + NVCC_FLAGS + EXTRA_FLAGS.get(name, []) + ["-I", CSRC, "-o", tmp, src] + EXTRA_LIBS.get(name, [])
    t0 = time.time()
    if verbose:
        print(f"[zig-ai_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            if verbose:
                print(f"[zig-ai_b200] ... still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {name}.cu:\n{log}")
    os.replace(tmp, out)
    with open(out + ".hash", "w") as f:
        f.write(source_hash(name))
    if verbose:
        print(f"[zig-ai_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def build_all(verbose: bool = True, force: bool = False) -> List[str]:
    """Compile every kernel source that is missing or out of date, a few at a time."""
    names = [n for n in sources() if force or not is_current(n)]
    if names:
        with ThreadPoolExecutor(max_workers=min(len(names), os.cpu_count() or 2)) as ex:
            list(ex.map(lambda n: compile_one(n, verbose), names))
    return [lib_path(n) for n in sources()]


def build_some(names: List[str], verbose: bool = True) -> None:
    """Compile those of the named sources that are missing or out of date, a few at a time."""
    todo = [n for n in names if not is_current(n)]
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2)) as ex:
            list(ex.map(lambda n: compile_one(n, verbose), todo))


def load(name: str) -> ctypes.CDLL:
    """The library of csrc/<name>.cu, compiled first if needed."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        if not is_current(name):
            compile_one(name)
        try:
            lib = ctypes.CDLL(lib_path(name))
        except OSError as e:
            raise KernelBuildError(f"cannot load {lib_path(name)}: {e}") from e
        _loaded[name] = lib
        return lib
