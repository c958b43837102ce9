"""Compiles the CUDA sources beside this file for sm_100a and loads them with ctypes.

Each `<name>.cu` becomes one shared library `_build/<name>-<hash>.so`, where the hash
covers the source, the shared header and the compiler flags, so an edited source is
rebuilt and an unchanged one is loaded as it is.  A library is compiled the first time
one of its functions is asked for; `build_all()` compiles every source ahead of time.
The build folder is `csrc/_build` if that can be written, else a per-user folder under
the system's temporary folder (a read-only checkout, an empty HOME and a user without
a home folder all work).  While nvcc runs, a line is printed to stderr now and then.

There is no fallback: if nvcc is missing or a source does not compile, the error is
raised to the caller.
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

SRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]
HEADERS = sorted(p.name for p in SRC_DIR.glob("*.cuh"))     # every shared header counts for every hash
# further files that a source includes (they count for its hash)
DEPENDS = {"attn_decode_static": ["attn_mma.cu", "attn_decode_static.h"]}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def kernel_names() -> list[str]:
    return sorted(p.stem for p in SRC_DIR.glob("*.cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA kernels of this engine cannot be built and there is no fallback")


_dir_cache: list = []


def _build_dir() -> Path:
    with _dir_lock:
        if not _dir_cache:
            _dir_cache.append(_find_build_dir())
        return _dir_cache[0]


def _find_build_dir() -> Path:
    env = os.environ.get("JAX_VLLM_B200_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands.append(SRC_DIR / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"jax_vllm_b200_build_{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".probe"):
                pass
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in cands]}")


def _extra_flags(name: str) -> list[str]:
    return []


def _hash(name: str) -> str:
    h = hashlib.sha256()
    for f in [f"{name}.cu", *HEADERS, *DEPENDS.get(name, [])]:
        h.update((SRC_DIR / f).read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + _extra_flags(name)).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path:
    return _build_dir() / f"{name}-{_hash(name)}.so"


def _compile(name: str, out: Path) -> None:
    src = SRC_DIR / f"{name}.cu"
    if not src.is_file():
        raise BuildError(f"no kernel source {src}")
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *_extra_flags(name), "-I", str(SRC_DIR), "-o", str(tmp), str(src)]
    env = dict(os.environ)
    env.setdefault("TMPDIR", str(out.parent))  # nvcc's intermediates: somewhere writable
    t0 = time.time()
    print(f"[jax-vllm_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            print(f"[jax-vllm_b200]   still compiling {src.name} ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed on {src.name}:\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"{name}-*"):          # libraries of earlier versions of this source
        if old.stem != out.stem:
            old.unlink(missing_ok=True)
    print(f"[jax-vllm_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def build(name: str) -> Path:
    """Compiles `<name>.cu` unless its library is already there; returns the library."""
    out = library_path(name)
    if out.is_file():
        return out
    lock = out.with_suffix(".lock")
    import fcntl

    with open(lock, "w") as lf:
        fcntl.flock(lf, fcntl.LOCK_EX)
        try:
            if not out.is_file():
                _compile(name, out)
        finally:
            fcntl.flock(lf, fcntl.LOCK_UN)
    return out


def build_all(names=None, jobs: int | None = None) -> list[Path]:
    """Compiles the given sources (all of them by default), several at a time."""
    names = list(names) if names is not None else kernel_names()
    todo = [n for n in names if not library_path(n).is_file()]
    if todo:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 1)) as ex:
            list(ex.map(build, todo))
    return [library_path(n) for n in names]


def load(name: str) -> ctypes.CDLL:
    """The shared library of `<name>.cu`, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(build(name)))
            _loaded[name] = lib
        return lib
