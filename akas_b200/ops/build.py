"""Compiles the CUDA sources of ``akas_b200/csrc`` for sm_100a and loads them with ctypes.

Each ``.cu`` file becomes one shared library with plain C entry points; nothing
links against Python or torch, so a file compiles in seconds. A library is built
on the first call that needs it and kept beside the package (``akas_b200/_build``)
or, where that folder cannot be written, in a per-user folder under the system's
temporary directory. The file name carries a hash of the source, the shared
header, the flags and the compiler version, so a stale build is never loaded.
While nvcc runs, a line goes to stderr now and then.
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
from pathlib import Path
from typing import Dict, Iterable, List

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LINK_FLAGS: Dict[str, List[str]] = {"gemm_bf16": ["-lcublasLt"]}
SOURCES = ("elementwise", "conv", "rope", "attention", "attention_prefill", "attention_prefill_tc", "attention_decode", "sgemm", "gemm_bf16", "gemm_tcgen05", "gemm_pair", "gemm_rows", "gemm_stream", "skinny_gemm", "decode_chain", "sampling")

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[akas_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("AKAS_B200_NVCC")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(str(Path(home) / "bin" / "nvcc"))
    candidates.append(shutil.which("nvcc"))
    for c in candidates:
        if c and Path(c).is_file() and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (set CUDA_HOME or AKAS_B200_NVCC); the kernels cannot be compiled")


_nvcc_version_cache: Dict[str, str] = {}


def _nvcc_version(nvcc: str) -> str:
    if nvcc not in _nvcc_version_cache:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
        _nvcc_version_cache[nvcc] = out.strip().splitlines()[-1] if out.strip() else "unknown"
    return _nvcc_version_cache[nvcc]


def _flags(name: str) -> List[str]:
    return ARCH_FLAGS + BASE_FLAGS + LINK_FLAGS.get(name, [])


def _digest(name: str, nvcc: str) -> str:
    h = hashlib.sha256()
    h.update((CSRC / f"{name}.cu").read_bytes())
    for header in sorted(CSRC.glob("*.cuh")):
        h.update(header.read_bytes())
    h.update(" ".join(_flags(name)).encode())
    h.update(_nvcc_version(nvcc).encode())
    return h.hexdigest()[:16]


def build_dirs() -> List[Path]:
    dirs = []
    if os.environ.get("AKAS_B200_BUILD_DIR"):
        dirs.append(Path(os.environ["AKAS_B200_BUILD_DIR"]))
    dirs.append(CSRC.parent / "_build")
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(Path(tempfile.gettempdir()) / f"akas_b200-build-{uid}")
    return dirs


def _existing(name: str, digest: str):
    for d in build_dirs():
        path = d / f"{name}-{digest}.so"
        if path.is_file():
            return path
    return None


def _writable_dir() -> Path:
    for d in build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe-{os.getpid()}-{threading.get_ident()}"
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(d) for d in build_dirs()]}")


def _compile(name: str, nvcc: str, digest: str, out_dir: Path, verbose: bool = False) -> Path:
    target = out_dir / f"{name}-{digest}.so"
    tmp = out_dir / f".{name}-{digest}.{os.getpid()}.so"
    cmd = [nvcc, *_flags(name), "-I", str(CSRC), "-o", str(tmp), str(CSRC / f"{name}.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {name}.cu:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        _say(proc.stderr)
    os.replace(tmp, target)
    for old in out_dir.glob(f"{name}-*.so"):  # earlier builds of this source
        if old != target and len(old.stem) == len(target.stem):
            try:
                old.unlink()
            except OSError:
                pass
    return target


def ensure_built(names: Iterable[str], verbose: bool = False) -> Dict[str, Path]:
    """Builds what is missing of ``names`` (in parallel) and returns name -> path of the library."""
    names = list(dict.fromkeys(names))
    paths: Dict[str, Path] = {}
    todo = []
    nvcc = None
    for name in names:
        if not (CSRC / f"{name}.cu").is_file():
            raise BuildError(f"no kernel source {name}.cu in {CSRC}")
        if nvcc is None:
            nvcc = find_nvcc()
        digest = _digest(name, nvcc)
        found = None if verbose else _existing(name, digest)
        if found is not None:
            paths[name] = found
        else:
            todo.append((name, digest))
    if todo:
        start = time.time()
        out_dir = _writable_dir()
        _say(f"compiling {', '.join(n + '.cu' for n, _ in todo)} for sm_100a with {nvcc} ...")
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2)) as pool:
            futures = {name: pool.submit(_compile, name, nvcc, digest, out_dir, verbose) for name, digest in todo}
            pending = set(futures)
            while pending:
                time.sleep(0.2)
                for name in list(pending):
                    if futures[name].done():
                        pending.discard(name)
                        paths[name] = futures[name].result()
                        _say(f"  {name}.cu done ({time.time() - start:.0f} s, {len(pending)} left)")
                if pending and int(time.time() - start) % 10 == 0 and time.time() - start > 1:
                    _say(f"  still compiling {', '.join(sorted(pending))} ({time.time() - start:.0f} s)")
                    time.sleep(1.0)
        _say(f"kernels built in {time.time() - start:.0f} s")
    return paths


def library(name: str) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu``, built first if need be."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = ensure_built([name])[name]
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
    return lib


def loaded_libraries() -> Dict[str, str]:
    return {name: lib._name for name, lib in _loaded.items()}
