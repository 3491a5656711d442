"""Builds the CUDA sources of this folder into one shared library for sm_100a.

The library is plain ``nvcc`` output with ``extern "C"`` entry points (no
Python or torch headers), so a first build takes seconds per file.  It is built
at the first call that needs it, into ``_build/`` beside the sources (or, when
that folder cannot be written, into a per-user folder under the system's
temporary directory), and rebuilt when a source or a flag changes.  While
``nvcc`` runs a line is printed now and then so that a first call does not look
hung.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))

SOURCES = [
    "elementwise.cu",
    "gemm_simt.cu",
    "attention_plain.cu",
    "sampling.cu",
    "gemm_tcgen05.cu",
    "gemm_chain.cu",
    "attention_mma.cu",
    "attention_tcgen05.cu",
    "wait_selftest.cu",
]
HEADERS = ["common.cuh", "sm100.cuh", "tensor_map.cuh", "no_alloc.h"]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-lineinfo",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]
LIBRARY_NAME = "libkirai_b200.so"


class BuildError(RuntimeError):
    pass


def _log(message: str) -> None:
    print(f"[kirai_b200 build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("KIRAI_NVCC"), shutil.which("nvcc")]
    cuda_home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    if cuda_home:
        candidates.append(os.path.join(cuda_home, "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc not found: set KIRAI_NVCC or CUDA_HOME, or put nvcc on PATH")


def _source_hash() -> str:
    digest = hashlib.sha256()
    for name in SOURCES + HEADERS:
        with open(os.path.join(HERE, name), "rb") as handle:
            digest.update(name.encode())
            digest.update(handle.read())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def _build_dir() -> str:
    preferred = os.path.join(HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"kirai_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _compile_one(nvcc: str, source: str, obj: str, verbose_ptxas: bool) -> str:
    command = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, source), "-o", obj]
    if verbose_ptxas:
        command[1:1] = ["-Xptxas", "-v"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise BuildError(f"nvcc failed on {source}:\n{result.stdout}\n{result.stderr}")
    return result.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Compiles what is out of date and returns the path of the shared library."""
    out_dir = _build_dir()
    library = os.path.join(out_dir, LIBRARY_NAME)
    stamp = os.path.join(out_dir, "build.stamp")
    wanted = _source_hash()
    if not force and os.path.exists(library) and os.path.exists(stamp):
        with open(stamp) as handle:
            if handle.read().strip() == wanted:
                return library

    import fcntl

    with open(os.path.join(out_dir, "build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)  # one builder at a time; the others find the stamp afterwards
        if not force and os.path.exists(library) and os.path.exists(stamp):
            with open(stamp) as handle:
                if handle.read().strip() == wanted:
                    return library
        nvcc = find_nvcc()
        _log(f"compiling {len(SOURCES)} CUDA sources for sm_100a with {nvcc} into {out_dir}")
        started = time.time()
        objects = [os.path.join(out_dir, os.path.splitext(name)[0] + ".o") for name in SOURCES]
        workers = max(1, min(len(SOURCES), os.cpu_count() or 1))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            futures = {
                pool.submit(_compile_one, nvcc, source, obj, verbose_ptxas): source
                for source, obj in zip(SOURCES, objects)
            }
            pending = set(futures)
            while pending:
                done, pending = concurrent.futures.wait(pending, timeout=10.0)
                for future in done:
                    log = future.result()
                    _log(f"compiled {futures[future]} ({time.time() - started:.0f} s)")
                    if verbose_ptxas and log:
                        print(log, file=sys.stderr)
                if pending:
                    names = ", ".join(sorted(futures[f] for f in pending))
                    _log(f"still compiling: {names} ({time.time() - started:.0f} s)")
        temporary = library + f".tmp{os.getpid()}"
        link = subprocess.run(
            [nvcc, "-shared", "-o", temporary, *objects, "-gencode", "arch=compute_100a,code=sm_100a"],
            capture_output=True,
            text=True,
        )
        if link.returncode != 0:
            raise BuildError(f"linking {LIBRARY_NAME} failed:\n{link.stdout}\n{link.stderr}")
        os.replace(temporary, library)
        with open(stamp, "w") as handle:
            handle.write(wanted)
        _log(f"built {library} in {time.time() - started:.0f} s")
    return library


HOST_SOURCES = ["page_tables.cpp", "scheduler.cpp", "safetensors_reader.cpp"]
HOST_LIBRARY_NAME = "libkirai_host.so"


def build_host(force: bool = False) -> str:
    """Builds the host-only C++ runtime pieces (no CUDA needed) and returns the library's path."""
    out_dir = _build_dir()
    library = os.path.join(out_dir, HOST_LIBRARY_NAME)
    stamp = os.path.join(out_dir, "host.stamp")
    digest = hashlib.sha256()
    for name in HOST_SOURCES:
        with open(os.path.join(HERE, name), "rb") as handle:
            digest.update(handle.read())
    wanted = digest.hexdigest()[:16]
    if not force and os.path.exists(library) and os.path.exists(stamp):
        with open(stamp) as handle:
            if handle.read().strip() == wanted:
                return library
    import fcntl

    with open(os.path.join(out_dir, "host.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and os.path.exists(library) and os.path.exists(stamp):
            with open(stamp) as handle:
                if handle.read().strip() == wanted:
                    return library
        compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if compiler is None:
            raise BuildError("no C++ compiler found (g++ or c++) for the host runtime")
        temporary = library + f".tmp{os.getpid()}"
        command = [compiler, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
                   *[os.path.join(HERE, name) for name in HOST_SOURCES], "-o", temporary]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise BuildError(f"building {HOST_LIBRARY_NAME} failed:\n{result.stdout}\n{result.stderr}")
        os.replace(temporary, library)
        with open(stamp, "w") as handle:
            handle.write(wanted)
    return library


if __name__ == "__main__":
    print(build_host(force="--force" in sys.argv))
    print(build(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv))
