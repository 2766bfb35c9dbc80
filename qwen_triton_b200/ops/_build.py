"""Compiles the CUDA sources for sm_100a at first use and loads them with ctypes.

Each ``csrc/<name>.cu`` becomes one shared library, built when an op from it is
first called, so a run compiles what it needs and nothing else.  Libraries are
kept under ``csrc/_build`` inside the package (or, where that is not writable,
in a per-user temporary folder) under a name that carries a hash of the
sources and flags, so a changed source is rebuilt.  There is no fallback: if
``nvcc`` is missing or the build fails, the op raises.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]

_LIBS: dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked in CUDA_HOME, /usr/local/cuda and PATH); "
                     "the CUDA kernels of qwen_triton_b200 cannot be built and there is no other path")


_BUILD_DIR: Path | None = None


def _build_dir() -> Path:
    global _BUILD_DIR
    if _BUILD_DIR is None:
        _BUILD_DIR = _find_build_dir()
    return _BUILD_DIR


def _find_build_dir() -> Path:
    override = os.environ.get("QWEN_TRITON_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"qwen_triton_b200_build_{os.getuid()}")
    for path in candidates:
        try:
            path.mkdir(parents=True, exist_ok=True)
            probe = path / f".probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_bytes(b"")
            probe.unlink()
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _source_hash(name: str) -> str:
    """Hash of the source, every header of the folder and the flags: any change rebuilds the library."""
    digest = hashlib.sha256()
    digest.update(" ".join(NVCC_FLAGS).encode())
    for path in [CSRC / f"{name}.cu", *sorted(CSRC.glob("*.cuh")), *sorted(CSRC.glob("*.h"))]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()[:16]


def library_path(name: str) -> Path:
    return _build_dir() / f"libqt_{name}-{_source_hash(name)}.so"


def sources() -> list[str]:
    return sorted(p.stem for p in CSRC.glob("*.cu"))


def compile_library(name: str, verbose: bool = True) -> Path:
    """Build ``csrc/<name>.cu`` if its library is not there yet; returns the library path."""
    source = CSRC / f"{name}.cu"
    if not source.exists():
        raise BuildError(f"no CUDA source {source}")
    target = library_path(name)
    if target.exists():
        return target
    tmp = target.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp), str(source)]
    if verbose:
        print(f"[qwen_triton_b200] compiling {source.name} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[qwen_triton_b200] still compiling {source.name} ({time.time() - started:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed on {source.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp, target)
    for stale in target.parent.glob(f"libqt_{name}-*.so"):      # libraries of earlier versions of this source
        if stale != target and ".tmp" not in stale.name:
            stale.unlink(missing_ok=True)
    if verbose:
        print(f"[qwen_triton_b200] built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return target


def load_library(name: str) -> ctypes.CDLL:
    with _LOCK:
        lib = _LIBS.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(compile_library(name)))
            getattr(lib, f"qt_last_error_{name}").restype = ctypes.c_char_p
            _LIBS[name] = lib
        return lib


def last_error(name: str) -> str:
    return getattr(load_library(name), f"qt_last_error_{name}")().decode("utf-8", "replace")


def build_all(verbose: bool = True) -> list[Path]:
    """Compile every CUDA source (in parallel); used by the build check."""
    names = sources()
    _build_dir()
    results: dict[str, Path | Exception] = {}

    def work(n: str) -> None:
        try:
            results[n] = compile_library(n, verbose)
        except Exception as exc:  # noqa: BLE001 - reported below
            results[n] = exc

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    failed = {n: r for n, r in results.items() if isinstance(r, Exception)}
    if failed:
        raise BuildError("\n".join(f"{n}: {e}" for n, e in failed.items()))
    return [results[n] for n in names]
