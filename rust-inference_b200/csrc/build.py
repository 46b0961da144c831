"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each ``.cu`` file becomes one shared library of plain C entry points.  A
library is compiled the first time something asks for it (``library(name)``),
so a process compiles what its model needs and nothing else; the result is kept
in ``_build/`` beside the sources under a name that carries a hash of the
sources and flags, so a changed source is compiled again and an unchanged one
never is.  While nvcc runs, a line is printed to stderr now and then.

There is no fallback: if nvcc is missing or a compile fails, the caller gets a
``KernelBuildError``.
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
from typing import Dict, Iterable, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--threads", "2"]

# every kernel source of the package, with the headers it includes
SOURCES: Dict[str, Tuple[str, ...]] = {
    "elementwise": ("elementwise.cu", "common.cuh", "linear_skinny_geometry.cuh"),
    "rope_kv": ("rope_kv.cu", "common.cuh"),
    "attention_rows": ("attention_rows.cu", "common.cuh"),
    "linear_f32": ("linear_f32.cu", "common.cuh"),
    "sampling": ("sampling.cu", "common.cuh"),
    "attention_decode": ("attention_decode.cu", "common.cuh", "mma_helpers.cuh"),
    "attention_prefill": ("attention_prefill.cu", "common.cuh", "mma_helpers.cuh"),
    "linear_skinny": ("linear_skinny.cu", "common.cuh", "mma_helpers.cuh", "linear_skinny_geometry.cuh"),
    "linear_stream_tc": ("linear_stream_tc.cu", "common.cuh", "mma_helpers.cuh"),
    "attention_prefill_tc": ("attention_prefill_tc.cu", "common.cuh", "mma_helpers.cuh"),
    "attention_decode_noalloc": ("attention_decode_noalloc.cu", "attention_decode_noalloc.h", "attention_decode.cu",
                                 "common.cuh", "mma_helpers.cuh"),
    "random_fill": ("random_fill.cu", "common.cuh", "random_fill.cuh"),
    # host code only: the same random values as random_fill.cu gives on the device
    "host_random": ("host_random.cpp", "random_fill.cuh"),
    # host code only (the cache's bookkeeping): built with the host compiler
    "host_cache": ("host_cache.cpp",),
    # host code only: the check of a step's entries and its int32 tables
    "host_step": ("host_step.cpp",),
}
# no fused multiply-adds: host_random.cpp must give the bits that the device gives
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-ffp-contract=off", "-pthread"]

# sources that are compiled once per value of a macro (the model's head size);
# the build check compiles these values, a model with another one compiles its own
HEAD_DIMS = (16, 32, 48, 64, 80, 96, 128, 256)
VARIANTS: Dict[str, Tuple[Dict[str, object], ...]] = {
    "attention_decode": tuple({"RI_HEAD_DIM": d} for d in HEAD_DIMS),
    "attention_prefill": tuple({"RI_HEAD_DIM": d} for d in HEAD_DIMS),
    "attention_decode_noalloc": ({"RI_HEAD_DIM": 64}, {"RI_HEAD_DIM": 128}),
    "attention_prefill_tc": ({"RI_HEAD_DIM": 64}, {"RI_HEAD_DIM": 128}),
}


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _log(msg: str) -> None:
    print(f"[rust_inference_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the CUDA kernels cannot be built")


def _host_compiler() -> Optional[str]:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and (os.path.exists(cand) or shutil.which(cand)):
            return cand
    return None


def build_dir() -> str:
    """``_build/`` beside the sources if it can be written, else a per-user folder
    under the temporary directory (a read-only installation)."""
    override = os.environ.get("RUST_INFERENCE_B200_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"rust_inference_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            if os.access(d, os.W_OK | os.X_OK):
                return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {cands}")


def _with_env_defines(defines: Optional[Dict[str, object]]) -> Optional[Dict[str, object]]:
    """Extra -D flags for every compile from RUST_INFERENCE_B200_DEFINES="A=1,B=2" (for experiments)."""
    extra = os.environ.get("RUST_INFERENCE_B200_DEFINES", "")
    if not extra:
        return defines
    out = dict(defines or {})
    for item in extra.split(","):
        if item.strip():
            k, _, v = item.partition("=")
            out[k.strip()] = v.strip() or "1"
    return out


def _variant_name(name: str, defines: Optional[Dict[str, object]]) -> str:
    if not defines:
        return name
    return name + "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))


def _fingerprint(name: str, defines: Optional[Dict[str, object]]) -> str:
    h = hashlib.sha256()
    for fn in SOURCES[name]:
        with open(os.path.join(HERE, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    h.update(repr(HOST_FLAGS if SOURCES[name][0].endswith(".cpp") else ARCH_FLAGS + BASE_FLAGS).encode())
    h.update(repr(sorted((defines or {}).items())).encode())
    return h.hexdigest()[:12]


def library_path(name: str, defines: Optional[Dict[str, object]] = None, where: Optional[str] = None) -> str:
    return os.path.join(where or build_dir(), f"{_variant_name(name, defines)}-{_fingerprint(name, defines)}.so")


def find_built(name: str, defines: Optional[Dict[str, object]] = None) -> Optional[str]:
    """An up-to-date library built earlier: in the in-tree folder even when that is
    read-only now, else in the writable build folder."""
    for d in (os.path.join(HERE, "_build"), None):
        try:
            p = library_path(name, defines, d)
        except KernelBuildError:
            continue
        if os.path.exists(p):
            return p
    return None


def compile_library(name: str, defines: Optional[Dict[str, object]] = None, verbose: bool = False) -> str:
    """Compile one source (if its library is not there yet) and return the path."""
    defines = _with_env_defines(defines)
    if name not in SOURCES:
        raise KernelBuildError(f"unknown kernel library {name!r}")
    have = find_built(name, defines)
    if have:
        return have
    out = library_path(name, defines)
    src = os.path.join(HERE, SOURCES[name][0])
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    macros = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    if src.endswith(".cpp"):
        # host code: the host compiler, or nvcc (which hands the file to it) where none is on the path
        cxx = _host_compiler()
        cmd = ([cxx] + HOST_FLAGS if cxx else [_nvcc(), "-O2", "-std=c++17", "-shared", "-Xcompiler",
                                               "-fPIC,-ffp-contract=off,-pthread"]) + macros
        _log(f"compiling {_variant_name(name, defines)} (host code) ...")
    else:
        cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + macros
        if verbose:
            cmd += ["-Xptxas", "-v"]
        _log(f"compiling {_variant_name(name, defines)} for sm_100a ...")
    cmd += ["-I", HERE, "-o", tmp, src]
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=build_dir())
    while True:
        try:
            log, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _log(f"still compiling {_variant_name(name, defines)} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {SOURCES[name][0]}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    _log(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    if verbose and log:
        print(log, file=sys.stderr)
    return out


def library(name: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    """The loaded library of ``name`` (compiled first if need be)."""
    defines = _with_env_defines(defines)
    key = _variant_name(name, defines)
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            lib.ri_last_error.restype = ctypes.c_char_p
            _loaded[key] = lib
    return lib


def prepare(requests: Iterable[Tuple[str, Optional[Dict[str, object]]]]) -> None:
    """Compile several libraries side by side (each at most once)."""
    todo = []
    for name, defines in requests:
        if _variant_name(name, defines) not in _loaded and not find_built(name, defines):
            todo.append((name, defines))
    if not todo:
        return
    errors = []

    def work(item):
        try:
            compile_library(*item)
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    gate = threading.Semaphore(max(2, (os.cpu_count() or 4) // 2))

    def gated(item):
        with gate:
            work(item)

    threads = [threading.Thread(target=gated, args=(item,)) for item in todo]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def build_all(extra: Iterable[Tuple[str, Optional[Dict[str, object]]]] = ()) -> None:
    """Compile every library (used by the repository's build check)."""
    reqs = []
    for n in SOURCES:
        if n in VARIANTS:
            reqs.extend((n, d) for d in VARIANTS[n])
        else:
            reqs.append((n, None))
    prepare(reqs + list(extra))
    # libraries of sources that have changed since are of no use to anyone: remove them
    keep = {os.path.basename(library_path(n, _with_env_defines(d), os.path.join(HERE, "_build"))) for n, d in reqs}
    built = os.path.join(HERE, "_build")
    if os.path.isdir(built) and not os.environ.get("RUST_INFERENCE_B200_DEFINES"):
        for fn in os.listdir(built):
            if fn.endswith(".so") and fn not in keep:
                try:
                    os.unlink(os.path.join(built, fn))
                except OSError:
                    pass
