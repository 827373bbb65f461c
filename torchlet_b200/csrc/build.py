"""Compiles the hand-written CUDA sources for sm_100a and loads them.

Each ``<name>.cu`` beside this file becomes one shared library ``lib<name>.so``,
compiled with ``nvcc`` alone (no Python or torch headers, so a file takes seconds)
and loaded with ``ctypes``.  A library is built the first time it is asked for and
kept beside a hash of its sources and flags; a matching hash means no rebuild.
Libraries live in ``csrc/_build`` inside the package when that folder can be written,
else in a per-user folder under the system's temporary directory.

There is no fallback: if ``nvcc`` or a source is missing, or compilation fails, the
caller gets an error that says so.
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
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--shared",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=default",
]

# TORCHLET_B200_DEBUG=1: the debug build, whose kernels check the indices they are given (token
# ids, positions, page ids, slots), record the first bad one and skip the access (common.cuh).
# Its libraries are built beside the ordinary ones under other names.
DEBUG_BUILD = os.environ.get("TORCHLET_B200_DEBUG", "") not in ("", "0")
if DEBUG_BUILD:
    NVCC_FLAGS = NVCC_FLAGS + ["-DTL_DEBUG"]
_SUFFIX = ".debug" if DEBUG_BUILD else ""

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def source_names() -> list[str]:
    return sorted(p.stem for p in SOURCE_DIR.glob("*.cu"))


def find_nvcc() -> str:
    candidates = [os.environ.get("TORCHLET_B200_NVCC"), shutil.which("nvcc")]
    cuda_home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    if cuda_home:
        candidates.append(str(Path(cuda_home) / "bin" / "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    for cand in candidates:
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be built")


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe.{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


_build_dir: Path | None = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        override = os.environ.get("TORCHLET_B200_BUILD_DIR")
        in_tree = SOURCE_DIR / "_build"
        if override and _writable(Path(override)):
            _build_dir = Path(override)
        elif _writable(in_tree):
            _build_dir = in_tree
        else:
            fallback = Path(tempfile.gettempdir()) / f"torchlet_b200_build_{os.getuid()}"
            if not _writable(fallback):
                raise BuildError(f"neither {in_tree} nor {fallback} can be written")
            _build_dir = fallback
    return _build_dir


def _source_hash(name: str) -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(NVCC_FLAGS).encode())
    # every header beside the sources counts: a changed constant must rebuild its users
    for path in [SOURCE_DIR / f"{name}.cu", *sorted(SOURCE_DIR.glob("*.cuh")), *sorted(SOURCE_DIR.glob("*.h"))]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _say(message: str) -> None:
    print(f"[torchlet_b200] {message}", file=sys.stderr, flush=True)


def ensure_built(name: str) -> Path:
    """Compile ``<name>.cu`` if its library is absent or stale; return the library's path."""
    source = SOURCE_DIR / f"{name}.cu"
    if not source.is_file():
        raise BuildError(f"no CUDA source {source}")
    wanted = _source_hash(name)
    candidates = [SOURCE_DIR / "_build", build_dir()]
    for folder in candidates:
        lib, stamp = folder / f"lib{name}{_SUFFIX}.so", folder / f"lib{name}{_SUFFIX}.hash"
        try:
            if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == wanted:
                return lib
        except OSError:
            continue
    folder = build_dir()
    lib, stamp = folder / f"lib{name}{_SUFFIX}.so", folder / f"lib{name}{_SUFFIX}.hash"
    tmp = folder / f"lib{name}{_SUFFIX}.{os.getpid()}.tmp.so"
    cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(SOURCE_DIR), "-o", str(tmp), str(source)]
    _say(f"compiling {name}.cu for sm_100a ...")
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(folder))
    while True:
        try:
            output, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {name}.cu ({time.time() - start:.0f} s)")
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed for {name}.cu:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, lib)
    stamp.write_text(wanted)
    _say(f"compiled {name}.cu in {time.time() - start:.1f} s")
    return lib


def load_library(name: str) -> ctypes.CDLL:
    """The library of ``<name>.cu``, built first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(ensure_built(name)))
            _loaded[name] = lib
        return lib


def build_all(parallel: int = 4) -> list[Path]:
    """Compile every source (used by the build check); returns the libraries."""
    from concurrent.futures import ThreadPoolExecutor

    build_dir()
    with ThreadPoolExecutor(max_workers=parallel) as pool:
        return list(pool.map(ensure_built, source_names()))
