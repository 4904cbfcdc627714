"""Compiles the CUDA sources under ``csrc/`` for sm_100a into shared libraries, in-tree.

A library is named after a hash of its sources, its defines and the compiler flags, so a stale
build is never loaded.  Libraries are kept in ``mrun_b200/_build`` when that folder can be
written, else in a per-user folder under the system's temporary directory.  Compilation happens
at the first call that needs a library and prints a line per file meanwhile.

Only what a model needs is built: the core library (norms, rotary, cache write, generic
attention, 32-bit GEMM, sampling) and, per head size, the tensor-core attention specialisation.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, Optional, Sequence

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "csrc")
CSRC = os.path.normpath(CSRC)
PACKAGE = os.path.dirname(CSRC)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]

_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("MRUN_NVCC"), shutil.which("nvcc"),
                      "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $MRUN_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other code path")


def _say(message: str) -> None:
    print(f"[mrun_b200 build] {message}", file=sys.stderr, flush=True)


def build_dir() -> str:
    override = os.environ.get("MRUN_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(PACKAGE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"mrun_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith((".cuh", ".h")))


def _digest(sources: Sequence[str], defines: Dict[str, object]) -> str:
    h = hashlib.sha256()
    for path in list(sources) + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(repr(sorted(defines.items())).encode())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Dict[str, object]) -> str:
    return os.path.join(build_dir(), f"lib{name}_{_digest(sources, defines)}.so")


def _compile_one(nvcc: str, source: str, obj: str, defines: Dict[str, object]) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           "-c", source, "-o", obj]
    start = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(source)}:\n{proc.stdout}")
    _say(f"compiled {os.path.basename(source)} in {time.time() - start:.1f} s")


def build_library(name: str, source_names: Iterable[str],
                  defines: Optional[Dict[str, object]] = None, extra_link: Sequence[str] = ()) -> str:
    """Builds (if needed) and returns the path of ``lib<name>_<hash>.so``."""
    defines = dict(defines or {})
    sources = [os.path.join(CSRC, n) for n in source_names]
    for path in sources:
        if not os.path.exists(path):
            raise BuildError(f"kernel source {path} is missing")
    with _lock:
        target = library_path(name, sources, defines)
        if os.path.exists(target):
            return target
        nvcc = find_nvcc()
        _say(f"building {os.path.basename(target)} from {len(sources)} file(s) for sm_100a ...")
        work = tempfile.mkdtemp(prefix="obj_", dir=os.path.dirname(target))
        try:
            objects = [os.path.join(work, os.path.basename(s) + ".o") for s in sources]
            with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
                futures = [pool.submit(_compile_one, nvcc, s, o, defines)
                           for s, o in zip(sources, objects)]
                for future in futures:
                    future.result()
            tmp = target + f".{os.getpid()}.tmp"
            link = [nvcc, "-shared", "-o", tmp, *objects, "-lcudart", *extra_link]
            proc = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise BuildError(f"linking {os.path.basename(target)} failed:\n{proc.stdout}")
            os.replace(tmp, target)
            _say(f"built {os.path.basename(target)}")
            prefix = f"lib{name}_"
            for other in os.listdir(os.path.dirname(target)):      # builds of older sources
                if other.startswith(prefix) and other.endswith(".so") and other != os.path.basename(target):
                    try:
                        os.remove(os.path.join(os.path.dirname(target), other))
                    except OSError:
                        pass
        finally:
            shutil.rmtree(work, ignore_errors=True)
        return target


HOST_SOURCES = ("host/cache_core.cpp", "host/sched_core.cpp")
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def find_cxx() -> str:
    for candidate in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if candidate and (os.path.exists(candidate) or shutil.which(candidate)):
            return candidate
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); the host runtime library "
                     "cannot be built")


def build_host() -> str:
    """The host-side runtime library (the cache manager's bookkeeping, the scheduler's decisions):
    plain C++, no CUDA."""
    sources = [os.path.join(CSRC, n) for n in HOST_SOURCES]
    h = hashlib.sha256()
    for path in sources:
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(CXX_FLAGS).encode())
    with _lock:
        target = os.path.join(build_dir(), f"libmrun_host_{h.hexdigest()[:16]}.so")
        if os.path.exists(target):
            return target
        cxx = find_cxx()
        _say(f"building {os.path.basename(target)} from {len(sources)} file(s) ...")
        tmp = target + f".{os.getpid()}.tmp"
        proc = subprocess.run([cxx, *CXX_FLAGS, "-o", tmp, *sources], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError(f"{cxx} failed on the host runtime library:\n{proc.stdout}")
        os.replace(tmp, target)
        _say(f"built {os.path.basename(target)}")
        for other in os.listdir(os.path.dirname(target)):
            if other.startswith("libmrun_host_") and other.endswith(".so") and other != os.path.basename(target):
                try:
                    os.remove(os.path.join(os.path.dirname(target), other))
                except OSError:
                    pass
        return target


CORE_SOURCES = ("common.cu", "elementwise.cu", "gemm_f32.cu", "gemm_skinny.cu", "gemm_tc5.cu",
                "attention_generic.cu", "sampling.cu")


def build_core() -> str:
    return build_library("mrun_core", CORE_SOURCES, {})


ATTENTION_SOURCES = ("common.cu", "attention_mma.cu", "attention_decode_tma.cu", "attention_tc5.cu")


def build_attention(head_dim: int) -> str:
    """The tensor-core attention kernels specialised for one head size."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise BuildError(f"the tensor-core attention takes head sizes 16, 32, ... 256, not {head_dim}")
    return build_library(f"mrun_attn_d{head_dim}", ATTENTION_SOURCES, {"MRUN_HEAD_DIM": head_dim})


# head sizes of the configurations this repository measures and tests
COMMON_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 128, 256)      # the head sizes the tests and the measured shapes use


def build_all() -> list[str]:
    """Every library the package loads for the configurations it measures and tests; other head
    sizes are built when a model with them is first run."""
    return [build_host(), build_core()] + [build_attention(d) for d in COMMON_HEAD_DIMS]
