"""Builds the CUDA library of this package with nvcc for sm_100a.

Each ``.cu`` file becomes an object; the objects are linked into one shared
library with a plain C interface (``ops.py`` loads it with ctypes).  Objects are
rebuilt only when their source, a header or the flags changed.  The library is
kept in ``csrc/_build`` inside the package; when that folder cannot be written
(a read-only install) a per-user folder under the system's temporary directory
is used.  Nothing here needs a GPU: nvcc cross-compiles.

While compiling, a line is printed to stderr for every file that starts and
finishes, so that a first call that has to build shows progress.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libayaka_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


if os.environ.get("AYAKA_B200_TRACE"):      # cycle marks inside the tensor-core kernels (debugging aid)
    NVCC_FLAGS.append("-DAYK_TRACE")


def _log(message: str) -> None:
    print(f"[ayaka_b200 build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (os.environ.get("AYAKA_NVCC"),
                      os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                      shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise RuntimeError("nvcc not found: set CUDA_HOME or AYAKA_NVCC; the kernels of this package "
                       "have no fallback")


def _build_dir() -> Path:
    preferred = HERE / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"ayaka_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def library_path() -> Path:
    return _build_dir() / LIB_NAME


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compiles what is out of date and returns the library's path."""
    out = _build_dir()
    headers = sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h"))
    flags = " ".join(NVCC_FLAGS)
    jobs = []
    objects = []
    for src in sources():
        obj = out / (src.stem + ".o")
        stamp = out / (src.stem + ".stamp")
        want = _digest([src] + headers, flags)
        objects.append(obj)
        if force or not obj.is_file() or not stamp.is_file() or stamp.read_text() != want:
            jobs.append((src, obj, stamp, want))
    lib = out / LIB_NAME
    lib_stamp = out / (LIB_NAME + ".stamp")
    link_want = _digest(sources() + headers, flags + "link")
    if not jobs and lib.is_file() and lib_stamp.is_file() and lib_stamp.read_text() == link_want:
        return lib

    nvcc = find_nvcc()

    def compile_one(job):
        src, obj, stamp, want = job
        t0 = time.time()
        if verbose:
            _log(f"compiling {src.name} ...")
        tmp = obj.with_suffix(f".o.tmp{os.getpid()}")
        proc = subprocess.run([nvcc, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(tmp)],
                              capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, obj)
        (out / (src.stem + ".ptxas.txt")).write_text(proc.stderr)
        stamp.write_text(want)
        if verbose:
            _log(f"compiled {src.name} in {time.time() - t0:.1f} s")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(compile_one, jobs))
    if verbose:
        _log(f"linking {LIB_NAME}")
    tmp = out / f"{LIB_NAME}.tmp{os.getpid()}"
    proc = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                           "-o", str(tmp), *map(str, objects)], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    lib_stamp.write_text(link_want)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
