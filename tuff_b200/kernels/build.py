"""Compiles the CUDA sources under `tuff_b200/csrc` for sm_100a, one shared
library per source file, on first use.

A library is named after a hash of its source, the shared headers and the
compiler flags, so an edited kernel is rebuilt and an unchanged one is found
again.  Libraries go to `csrc/_build/` inside the package when that folder can
be written, else to a per-user folder under the system's temporary directory;
no home directory is needed.  While nvcc runs, a line is printed to stderr every
few seconds.  There is no fallback: if a library cannot be built or loaded the
caller gets a `KernelBuildError`.
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

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]
LINK_LIBS: dict[str, list[str]] = {}
# TUFF_DEBUG_BOUNDS=1 in the environment builds (under names of their own) and loads the variants of these
# libraries whose kernels range-check every table row, page id and state slot they are given and leave a
# code in the status word instead of making the access (csrc/index.cuh).
CHECKED_LIBS = ("attention_plain", "attention_flash", "attention_tc", "shortconv", "gemm_stream")


def _flags(name: str) -> list[str]:
    extra = ["-DTUFF_DEBUG_BOUNDS"] if name in CHECKED_LIBS and os.environ.get("TUFF_DEBUG_BOUNDS", "0") not in ("", "0") else []
    # TUFF_NVCC_EXTRA: further flags (-D...) for experiments with a kernel's compile-time choices
    return NVCC_FLAGS + extra + os.environ.get("TUFF_NVCC_EXTRA", "").split()

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def sources() -> list[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    cand = os.environ.get("TUFF_NVCC") or shutil.which("nvcc")
    if not cand:
        for p in ("/usr/local/cuda/bin/nvcc",):
            if os.path.isfile(p):
                cand = p
                break
    if not cand:
        raise KernelBuildError("nvcc was not found (PATH, TUFF_NVCC, /usr/local/cuda/bin); the CUDA "
                               "kernels of tuff_b200 cannot be compiled and there is no fallback")
    return cand


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")) or f == name + ".cu":
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + _flags(name) + LINK_LIBS.get(name, [])).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> list[str]:
    dirs = []
    if os.environ.get("TUFF_BUILD_DIR"):
        dirs.append(os.environ["TUFF_BUILD_DIR"])
    dirs.append(os.path.join(CSRC, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"tuff_b200-build-{os.getuid()}"))
    return dirs


def _writable_dir() -> str:
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".probe-"):
                pass
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for compiled kernels: tried " + ", ".join(_build_dirs()))


def library_path(name: str, must_exist: bool = False) -> str | None:
    fname = f"{name}-{_digest(name)}.so"
    for d in _build_dirs():
        p = os.path.join(d, fname)
        if os.path.isfile(p):
            return p
    if must_exist:
        return None
    return os.path.join(_writable_dir(), fname)


def compile_library(name: str, verbose: bool = True) -> str:
    """Builds `csrc/<name>.cu` if its library is not there yet; returns the path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    found = library_path(name, must_exist=True)
    if found:
        return found
    out = library_path(name)
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + _flags(name) + ["-I", CSRC, "-o", tmp, src] + LINK_LIBS.get(name, [])
    t0 = time.time()
    if verbose:
        print(f"[tuff_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    result: list[str] = []
    reader = threading.Thread(target=lambda: result.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[tuff_b200] ... still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    reader.join()
    log = result[0] if result else ""
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    if verbose:
        print(f"[tuff_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, jobs: int | None = None, checked: bool = False) -> list[str]:
    """Compiles every source (in parallel); used by the build check.  `checked`: the range-checking
    variants of `CHECKED_LIBS` instead (what TUFF_DEBUG_BOUNDS=1 loads)."""
    names = sources()
    if checked:
        before = os.environ.get("TUFF_DEBUG_BOUNDS")
        os.environ["TUFF_DEBUG_BOUNDS"] = "1"
        try:
            return _build(list(CHECKED_LIBS), verbose, jobs)
        finally:
            if before is None:
                del os.environ["TUFF_DEBUG_BOUNDS"]
            else:
                os.environ["TUFF_DEBUG_BOUNDS"] = before
    return _build(names, verbose, jobs)


def _build(names: list[str], verbose: bool, jobs: int | None) -> list[str]:
    jobs = jobs or min(len(names), max(1, (os.cpu_count() or 2)))
    out: dict[str, str] = {}
    errs: list[BaseException] = []

    def work(n: str) -> None:
        try:
            out[n] = compile_library(n, verbose)
        except BaseException as e:  # noqa: BLE001 - reported below
            errs.append(e)

    pending = list(names)
    while pending:
        batch, pending = pending[:jobs], pending[jobs:]
        threads = [threading.Thread(target=work, args=(n,)) for n in batch]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    if errs:
        raise errs[0]
    return [out[n] for n in names]
