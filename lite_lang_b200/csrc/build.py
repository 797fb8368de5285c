"""Compiles the CUDA sources of this folder with nvcc and loads them with ctypes.

Each *library* is a set of ``.cu`` files (plus optional ``-D`` definitions)
that becomes one shared object under ``_build/`` beside the sources.  A library
is compiled at its first use, when its shared object is missing or was built
from other sources (a digest of sources, headers and flags is part of the file
name), and only the libraries that a model's parts ask for are ever built.
There is no fallback: without nvcc, or on a compile error, loading raises.

The launchers are plain C functions (raw pointers, sizes, a ``cudaStream_t``)
that return a ``cudaError_t`` as an int; ``Library.call`` raises on non-zero.
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
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# --use_fast_math is NOT used: expf, division and sqrtf keep their IEEE forms.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# name -> (sources, definitions)
LIBRARIES: Dict[str, Tuple[Tuple[str, ...], Tuple[str, ...]]] = {
    "core": (("embedding.cu", "norm.cu", "rope.cu", "activation.cu", "sampling.cu", "attention_generic.cu"), ()),
    "attn_mma": (("attention_mma.cu", "attention_prefill.cu", "attention_decode.cu"), ()),
    "gemm_smallm": (("gemm_smallm.cu",), ()),
    "gemm_stream": (("gemm_stream.cu",), ()),
    "gemm_tc": (("gemm_tc.cu",), ()),
    "gemm_pair": (("gemm_pair.cu",), ()),
    "attn_tc": (("attention_prefill_tc.cu",), ()),
    "attn_mma_static": (("attention_mma_static.cu",), ()),
}

_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)
LAUNCHES = 0   # launcher calls so far (each launches one kernel unless its docstring says otherwise)
_lock = threading.Lock()
_loaded: Dict[str, "Library"] = {}


class BuildError(RuntimeError):
    pass


def register_library(name: str, sources: Sequence[str], definitions: Sequence[str] = ()) -> None:
    """Declare a library made of ``sources`` (paths relative to this folder, or absolute)."""
    LIBRARIES[name] = (tuple(sources), tuple(definitions))


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand is None:
        for c in ("/usr/local/cuda/bin/nvcc",):
            if os.path.isfile(c):
                cand = c
                break
    if cand is None:
        raise BuildError("nvcc was not found (set NVCC or put it on PATH); the CUDA kernels cannot be built "
                         "and there is no fallback")
    return cand


def _build_dir() -> str:
    d = os.environ.get("LITE_LANG_B200_BUILD_DIR")
    if d:
        os.makedirs(d, exist_ok=True)
        return d
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"lite_lang_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _src_path(s: str) -> str:
    return s if os.path.isabs(s) else os.path.join(_HERE, s)


def _with_includes(sources: Iterable[str]) -> List[str]:
    """The sources and every file of this folder they include with #include "..." (recursively)."""
    seen: List[str] = []
    todo = [_src_path(s) for s in sources]
    while todo:
        path = todo.pop(0)
        if path in seen or not os.path.isfile(path):
            continue
        seen.append(path)
        with open(path, "r", encoding="utf-8") as fh:
            for inc in _INCLUDE.findall(fh.read()):
                todo.append(os.path.join(os.path.dirname(path), inc))
    return seen


def _digest(sources: Iterable[str], definitions: Iterable[str]) -> str:
    h = hashlib.sha256()
    for s in _with_includes(sources):
        with open(s, "rb") as fh:
            h.update(fh.read())
        h.update(b"\0")
    h.update(" ".join(list(definitions) + ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _say(msg: str) -> None:
    print(f"[lite_lang_b200 build] {msg}", file=sys.stderr, flush=True)


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    t0 = time.time()
    last = t0
    while True:
        try:
            out, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if time.time() - last >= 10:
                _say(f"... still compiling {what} ({time.time() - t0:.0f} s)")
                last = time.time()
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{out}")
    if os.environ.get("LITE_LANG_B200_VERBOSE_BUILD") and out.strip():
        _say(out)


def timeline_build() -> bool:
    """LITE_LANG_B200_TIMELINE=1: the libraries are built with the kernels' time stamps compiled in (a build of
    its own beside the ordinary one; see ``LL_TIMELINE_STAMP`` in common.cuh)."""
    return os.environ.get("LITE_LANG_B200_TIMELINE", "0") == "1"


def _library(name: str):
    sources, definitions = LIBRARIES[name]
    if timeline_build():
        definitions = tuple(definitions) + ("-DLL_TIMELINE",)
    return sources, definitions


def _file_prefix(name: str) -> str:
    return f"liblitelang_{name}-timeline_" if timeline_build() else f"liblitelang_{name}_"


def library_path(name: str) -> str:
    sources, definitions = _library(name)
    return os.path.join(_build_dir(), f"{_file_prefix(name)}{_digest(sources, definitions)}.so")


def build_library(name: str, verbose: bool = True) -> str:
    """Compile ``name`` if needed and return the path of its shared object."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    sources, definitions = _library(name)
    target = library_path(name)
    if os.path.isfile(target):
        return target
    nvcc = _nvcc()
    bdir = os.path.dirname(target)
    tag = os.path.basename(target)[:-3]
    if verbose:
        _say(f"compiling kernel library '{name}' ({len(sources)} files) for sm_100a; this happens once")
    t0 = time.time()
    objs: List[str] = []

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, f"{tag}_{os.path.basename(src)}.{os.getpid()}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *definitions, "-I", _HERE, "-c", _src_path(src), "-o", obj]
        _run(cmd, os.path.basename(src))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    tmp = target + f".{os.getpid()}.tmp"
    _run([nvcc, *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", tmp, *objs], f"link {name}")
    os.replace(tmp, target)
    prefix = _file_prefix(name)
    for old in os.listdir(bdir):  # shared objects of this library built from older sources
        if (old.startswith(prefix) and old.endswith(".so") and len(old) == len(prefix) + 16 + 3
                and os.path.join(bdir, old) != target):
            try:
                os.remove(os.path.join(bdir, old))
            except OSError:
                pass
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    if verbose:
        _say(f"built {os.path.basename(target)} in {time.time() - t0:.1f} s")
    return target


class Library:
    """A loaded kernel library; ``call(symbol, *args)`` checks the returned cudaError_t."""

    def __init__(self, name: str, path: str):
        self.name = name
        self.path = path
        self._dll = ctypes.CDLL(path)
        self._fns: Dict[str, ctypes._CFuncPtr] = {}

    def fn(self, symbol: str):
        f = self._fns.get(symbol)
        if f is None:
            try:
                f = getattr(self._dll, symbol)
            except AttributeError:
                raise BuildError(f"kernel library {self.name!r} ({self.path}) has no symbol {symbol!r}") from None
            f.restype = ctypes.c_int
            self._fns[symbol] = f
        return f

    def call(self, symbol: str, *args) -> None:
        global LAUNCHES
        LAUNCHES += 1
        err = self.fn(symbol)(*args)
        if err != 0:
            raise RuntimeError(f"{symbol} failed with CUDA error {err} "
                               f"(1 = invalid value: a size this kernel does not take)")


def load_library(name: str) -> Library:
    """Build (if needed) and load a kernel library.  Raises if that is not possible."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = Library(name, build_library(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    """Compile every declared library (used by the repository's build check)."""
    return [build_library(n, verbose) for n in sorted(LIBRARIES)]
