"""Compiles the CUDA sources of ``csrc/`` into shared libraries, one per source file, and loads
them with ctypes.

Each library is built the first time something asks for it, with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and nothing else from outside the package: no
torch headers (a file compiles in seconds), no network, no per-user cache.  The libraries live in
``<package>/_build/`` when that folder can be written, else in a folder under the system's
temporary directory; the file name carries a hash of the source, of the headers it includes and of
the flags, so a stale library is never loaded.  While nvcc runs, a line is printed every few
seconds so that a first call does not look hung.

There is no fallback: if nvcc is missing or a source does not compile, ``BuildError`` is raised and
nothing runs.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PACKAGE_DIR, "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=default"]

# every source file of the package; `build_all` compiles all of them
SOURCES = ("embedding", "norm", "rope_cache", "attention_simt", "attention_decode", "attention_decode_static", "attention_prefill",
           "attention_prefill_tc",
           "activation", "gemm_simt", "gemm_tcgen05", "gemm_chain", "gemm_pair_tc",
           "sampling")

_libs: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the CUDA kernels of "
                     "this package cannot be built and there is no other code path")


_build_dir_cache: list = []


def _build_dir() -> str:
    if _build_dir_cache:
        return _build_dir_cache[0]
    cands = [os.environ.get("MIE_B200_BUILD_DIR"), os.path.join(PACKAGE_DIR, "_build"),
             os.path.join(tempfile.gettempdir(), f"mini_inference_engine_b200_build_{os.getuid()}")]
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(dir=d, prefix=".probe")
            os.close(fd)
            os.unlink(probe)
            _build_dir_cache.append(d)
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for the compiled kernels (tried " + ", ".join(c for c in cands if c) + ")")


def _source_hash(name: str, extra_flags: tuple) -> str:
    h = hashlib.sha256()
    files = [os.path.join(CSRC, name + ".cu")] + sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for f in files:
        with open(f, "rb") as fh:
            h.update(os.path.basename(f).encode())
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + list(extra_flags)).encode())
    return h.hexdigest()[:16]


def _extra_flags(name: str) -> tuple:
    return ()


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"lib{name}-{_source_hash(name, _extra_flags(name))}.so")


def _compile(name: str, out: str, verbose: bool) -> None:
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no such kernel source: {src}")
    tmp = f"{out}.{os.getpid()}.tmp.so"
    cmd = [_nvcc()] + ARCH_FLAGS + COMMON_FLAGS + list(_extra_flags(name)) + ["-I", CSRC, "-o", tmp, src]
    t0 = time.time()
    if verbose:
        print(f"[mini_inference_engine_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env,
                            cwd=os.path.dirname(out))
    while True:
        try:
            output, _ = proc.communicate(timeout=8)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[mini_inference_engine_b200]   still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    for old in os.listdir(os.path.dirname(out)):          # libraries of earlier versions of this source
        if old.startswith(f"lib{name}-") and old.endswith(".so") and old != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), old))
            except OSError:
                pass
    if verbose:
        print(f"[mini_inference_engine_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> str:
    """Makes sure the library of ``csrc/<name>.cu`` exists and returns its path."""
    out = library_path(name)
    if os.path.isfile(out):
        return out
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)          # another process may be building the same file
        try:
            if not os.path.isfile(out):
                _compile(name, out, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    try:
        os.unlink(lock_path)
    except OSError:
        pass
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu`` (built first if need be)."""
    with _lock:
        lib = _libs.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            _libs[name] = lib
        return lib


def prepare(names, verbose: bool = True) -> None:
    """Compiles those of ``names`` that are not built yet, side by side: a model that needs nine
    libraries waits for the slowest of them at its first load, not for their sum."""
    missing = [n for n in sorted(set(names)) if n not in _libs and not os.path.isfile(library_path(n))]
    if len(missing) > 1:
        build_all(verbose, missing)


def build_all(verbose: bool = True, sources=SOURCES) -> list[str]:
    """Compiles every source (in parallel processes of nvcc) and returns the library paths."""
    errors: list = []
    paths: dict = {}

    def work(n):
        try:
            paths[n] = build(n, verbose)
        except Exception as e:          # noqa: BLE001 - reported below, all at once
            errors.append((n, e))

    threads = [threading.Thread(target=work, args=(n,)) for n in sources]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise BuildError("\n".join(f"{n}: {e}" for n, e in errors))
    return [paths[n] for n in sources]
