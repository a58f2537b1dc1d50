"""Compiles the CUDA sources of this folder for sm_100a with nvcc (and the host runtime with
the C++ compiler) and loads the result with ctypes.

A library is named by a hash of its sources, headers, compile-time definitions and
flags, so a stale build is never loaded.  Libraries live in ``<package>/_lib`` when that
folder can be written (the built ``.so`` then sits inside the tree) and otherwise in a
per-user folder under the system's temporary directory.  Compilation happens at the
first call that needs a library and prints a progress line every few seconds.
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
from typing import Dict, Iterable, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(HERE)

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr", "-DCO_TARGET_ARCH=100"]

# The core library: everything that is not specialised by a compile-time size.
CORE_SOURCES = ["runtime.cu", "elementwise.cu", "gemm_simt.cu", "attention_simple.cu",
                "sampling.cu", "gemm_bf16_small.cu", "gemm_tc.cu", "gemm_tc_few.cu", "seeded_fill.cu", "selftest.cu",
                "block_runner.cu"]
HEADERS = ["common.cuh"]


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of this engine cannot be built")


def _lib_dir() -> str:
    override = os.environ.get("COHERYN_B200_LIB_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(PACKAGE, "_lib"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"coheryn_b200_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for the compiled kernels: tried " + ", ".join(candidates))


def _existing_lib(name: str) -> Optional[str]:
    """A previously built library of this exact name in any known folder."""
    dirs = [os.environ.get("COHERYN_B200_LIB_DIR"), os.path.join(PACKAGE, "_lib"),
            os.path.join(tempfile.gettempdir(), f"coheryn_b200_{os.getuid()}")]
    for d in dirs:
        if d and os.path.isfile(os.path.join(d, name)):
            return os.path.join(d, name)
    return None


def _digest(sources: Sequence[str], defines: Dict[str, object], extra: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in list(sources) + HEADERS + sorted(x for x in os.listdir(HERE) if x.endswith((".cuh", ".h"))):
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS + list(extra)).encode())
    return h.hexdigest()[:16]


def _progress(label: str, stop: threading.Event) -> None:
    t0 = time.time()
    while not stop.wait(5.0):
        print(f"[coheryn-b200] compiling {label} ... {time.time() - t0:.0f} s",
              file=sys.stderr, flush=True)


def _drop_stale(out_dir: str, prefix: str, keep: str) -> None:
    """Earlier builds of the same library (other source hashes) are of no use to anyone."""
    try:
        for f in os.listdir(out_dir):
            if f.startswith(prefix) and f.endswith(".so") and f != keep:
                os.unlink(os.path.join(out_dir, f))
    except OSError:
        pass


def build_library(label: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None,
                  extra_flags: Iterable[str] = (), verbose: bool = False) -> str:
    """Compile ``sources`` into one shared library and return its path (cached)."""
    defines = dict(defines or {})
    extra = list(extra_flags)
    name = f"libcoheryn_b200_{label}_{_digest(sources, defines, extra)}.so"
    found = _existing_lib(name)
    if found:
        return found
    out_dir = _lib_dir()
    target = os.path.join(out_dir, name)
    nvcc = nvcc_path()
    work = tempfile.mkdtemp(prefix="build_", dir=out_dir)
    flags = ARCH_FLAGS + BASE_FLAGS + extra + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    if verbose:
        flags += ["-Xptxas", "-v"]
    print(f"[coheryn-b200] compiling {label} ({len(sources)} CUDA files) for sm_100a; "
          "this happens once", file=sys.stderr, flush=True)
    stop = threading.Event()
    ticker = threading.Thread(target=_progress, args=(label, stop), daemon=True)
    ticker.start()
    try:
        procs = []
        for src in sources:
            obj = os.path.join(work, src.replace(".cu", ".o"))
            cmd = [nvcc, "-c", os.path.join(HERE, src), "-o", obj, "-I", HERE] + flags
            procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                     stderr=subprocess.STDOUT, text=True)))
        objs: List[str] = []
        failures = []
        for src, obj, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                failures.append(f"--- {src}\n{out}")
            elif verbose and out:
                print(out, file=sys.stderr)
            objs.append(obj)
        if failures:
            raise BuildError("nvcc failed:\n" + "\n".join(failures))
        tmp_target = os.path.join(work, name)
        link = [nvcc, "-shared", "-o", tmp_target] + objs + ARCH_FLAGS
        r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError("linking failed:\n" + r.stdout)
        os.replace(tmp_target, target)
        _drop_stale(out_dir, f"libcoheryn_b200_{label}_", name)
    finally:
        stop.set()
        shutil.rmtree(work, ignore_errors=True)
    print(f"[coheryn-b200] built {target}", file=sys.stderr, flush=True)
    return target


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def load_library(label: str, sources: Sequence[str], defines: Optional[Dict[str, object]] = None,
                 extra_flags: Iterable[str] = ()) -> ctypes.CDLL:
    key = label + repr(sorted((defines or {}).items()))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build_library(label, sources, defines, extra_flags)
            lib = ctypes.CDLL(path)
            lib.coheryn_library_path = path  # type: ignore[attr-defined]
            _loaded[key] = lib
        return lib


def host_compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); the host runtime "
                     "of this engine cannot be built")


HOST_SOURCES = ["host_pages.cpp", "host_engine.cpp", "host_seeded.cpp"]
# -ffp-contract=off: the seeded weights must round after every operation, as the CUDA kernel does.
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-ffp-contract=off", "-pthread"]


def build_host_library() -> str:
    """The host runtime (page and slot bookkeeping): plain C++, no CUDA, compiled in a second."""
    h = hashlib.sha256()
    for f in HOST_SOURCES + ["seeded_values.h", "host_pools.h", "host_sha256.h"]:
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(repr(HOST_FLAGS).encode())
    name = f"libcoheryn_b200_host_{h.hexdigest()[:16]}.so"
    found = _existing_lib(name)
    if found:
        return found
    out_dir = _lib_dir()
    target = os.path.join(out_dir, name)
    tmp_target = os.path.join(out_dir, f".{os.getpid()}_{name}")
    cmd = [host_compiler()] + HOST_FLAGS + [os.path.join(HERE, f) for f in HOST_SOURCES] + ["-o", tmp_target]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError("the host runtime did not compile:\n" + r.stdout)
    os.replace(tmp_target, target)
    _drop_stale(out_dir, "libcoheryn_b200_host_", name)
    print(f"[coheryn-b200] built {target}", file=sys.stderr, flush=True)
    return target


def host_library() -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get("host")
        if lib is None:
            path = build_host_library()
            lib = ctypes.CDLL(path)
            lib.coheryn_library_path = path  # type: ignore[attr-defined]
            _loaded["host"] = lib
        return lib


def core_library() -> ctypes.CDLL:
    return load_library("core", CORE_SOURCES)


def attention_library(head_dim: int) -> ctypes.CDLL:
    """The bfloat16 tensor-core attention kernels, compiled for one head size."""
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise BuildError(f"the bfloat16 attention kernels take head sizes 16..256 in steps "
                         f"of 16, not {head_dim}")
    return load_library(f"attn_hd{head_dim}", ["attention_bf16.cu", "attention_tc.cu", "runtime.cu"],
                        {"CO_HEAD_DIM": head_dim})


def build_all(head_dims: Sequence[int] = (16, 32, 64, 128)) -> List[str]:
    """Compile everything ahead of time (no GPU needed)."""
    paths = [build_host_library(), build_library("core", CORE_SOURCES)]
    for hd in head_dims:
        paths.append(build_library(f"attn_hd{hd}", ["attention_bf16.cu", "attention_tc.cu", "runtime.cu"],
                                   {"CO_HEAD_DIM": hd}))
    return paths
