"""Builds the CUDA kernels of this package into one shared library, for sm_100a only.

Each `.cu` file is compiled by nvcc on its own (in parallel) and the objects are linked into
`_build/libbt_b200.so` beside the sources.  A stamp of the sources and flags decides whether a
rebuild is needed, so a second call costs nothing.  If the package folder cannot be written to,
the build goes to a per-user folder under the system's temporary directory.
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
from pathlib import Path

from ..errors import KernelError

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libbt_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _say(message: str) -> None:
    print(f"[burn_transformers_b200 build] {message}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp(files: list[Path]) -> str:
    h = hashlib.sha256()
    for path in sorted(list(files) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                      "the CUDA kernels of this package cannot be built")


def _build_dir() -> Path:
    preferred = CSRC / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"burn_transformers_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def library_path() -> Path:
    """Where the built library lies (or would lie)."""
    return _build_dir() / LIB_NAME


def build(verbose: bool = True) -> Path:
    """Compiles what is out of date and returns the path of the shared library."""
    files = sources()
    out_dir = _build_dir()
    lib = out_dir / LIB_NAME
    stamp_file = out_dir / "stamp.txt"
    stamp = _stamp(files)
    if lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
        return lib
    nvcc = _nvcc()
    if verbose:
        _say(f"compiling {len(files)} CUDA files for sm_100a into {out_dir} (first use only)")
    started = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _say(f"still compiling, {time.time() - started:.0f} s so far")

    ticker = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        ticker.start()

    def compile_one(src: Path):
        # per-file stamps keep unchanged objects
        obj = out_dir / (src.stem + ".o")
        own = hashlib.sha256(src.read_bytes() + b"".join(p.read_bytes() for p in sorted(CSRC.glob("*.cuh")))
                             + " ".join(NVCC_FLAGS).encode()).hexdigest()
        own_file = out_dir / (src.stem + ".stamp")
        if obj.is_file() and own_file.is_file() and own_file.read_text() == own:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelError(f"nvcc failed on {src.name}:\n{result.stdout}\n{result.stderr}")
        own_file.write_text(own)
        if verbose:
            _say(f"compiled {src.name} ({time.time() - started:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objects = list(pool.map(compile_one, files))
        tmp = out_dir / f".{LIB_NAME}.{os.getpid()}"
        link = [nvcc, "-shared", "-o", str(tmp), *map(str, objects)]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelError(f"linking {LIB_NAME} failed:\n{result.stdout}\n{result.stderr}")
        os.replace(tmp, lib)
        stamp_file.write_text(stamp)
    finally:
        done.set()
    if verbose:
        _say(f"built {lib.name} in {time.time() - started:.0f} s")
    return lib


HOST_LIB_NAME = "libbt_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared"]


def host_sources() -> list[Path]:
    return sorted((CSRC / "host").glob("*.cpp"))


def build_host(verbose: bool = True) -> Path:
    """Compiles the host-side library (the cache's books and the packing of a step's integers: plain C++, no CUDA)
    with the system's C++ compiler and returns its path.  It needs no GPU and no nvcc, so everything that does not
    launch kernels (configuration, weights, the cache's bookkeeping, the generation loop's decisions) runs anywhere."""
    files = host_sources()
    out_dir = _build_dir()
    lib = out_dir / HOST_LIB_NAME
    stamp_file = out_dir / "host_stamp.txt"
    h = hashlib.sha256()
    for path in files:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    stamp = h.hexdigest()
    if lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
        return lib
    compiler = next((c for c in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++"))
                     if c and Path(c).is_file()), None)
    if compiler is None:
        raise KernelError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); the host library of this "
                          "package cannot be built")
    started = time.time()
    tmp = out_dir / f".{HOST_LIB_NAME}.{os.getpid()}"
    result = subprocess.run([compiler, *HOST_FLAGS, "-o", str(tmp), *map(str, files)], capture_output=True, text=True)
    if result.returncode != 0:
        raise KernelError(f"compiling {HOST_LIB_NAME} failed:\n{result.stdout}\n{result.stderr}")
    os.replace(tmp, lib)
    stamp_file.write_text(stamp)
    if verbose:
        _say(f"built {lib.name} in {time.time() - started:.0f} s")
    return lib


if __name__ == "__main__":
    print(build_host())
    print(build())
