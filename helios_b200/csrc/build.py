"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each ``.cu`` file becomes one shared library, loaded with ``ctypes``; its
launchers are plain C functions that take device pointers and a stream.  A
library is compiled at the first call that needs it (a float32 run never
compiles the bfloat16 tensor-core kernels) and kept under ``_build/`` beside the
sources, named by a hash of source, headers and flags, so a changed file is
compiled again and an unchanged one is loaded as it is.  If that folder cannot
be written, a per-user folder under the system's temporary directory is used.
While nvcc runs, a line is printed to stderr every few seconds.

There is no fallback: if nvcc is missing or a compile fails, ``KernelBuildError``
is raised with the compiler's output.
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
from typing import Dict, List, Optional

_SRC_DIR = Path(__file__).resolve().parent

# library name -> source file.  Headers every library depends on are listed once.
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "attention_generic": "attention_generic.cu",
    "attention_bf16": "attention_bf16.cu",
    "attention_tc": "attention_tc.cu",
    "attention_pair": "attention_pair.cu",
    "gemm_f32": "gemm_f32.cu",
    "gemm_bf16": "gemm_bf16.cu",
    "gemm_bf16_noalloc": "gemm_bf16_noalloc.cu",
    "sampling": "sampling.cu",
}
_HEADERS = ["common.cuh", "tcgen05.cuh"]
# further files a library's source includes
_INCLUDES: Dict[str, List[str]] = {"gemm_bf16_noalloc": ["gemm_bf16.cu", "gemm_bf16_noalloc.h"],
                                   "attention_bf16": ["attention_mma.cuh"]}

NVCC_FLAGS = [
    "-O3", "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
]


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return str(Path(cand) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise KernelBuildError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                           "the CUDA kernels of helios_b200 cannot be built")


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("HELIOS_B200_BUILD_DIR")
    if override and _writable_dir(Path(override)):
        return Path(override)
    local = _SRC_DIR / "_build"
    if _writable_dir(local):
        return local
    fallback = Path(tempfile.gettempdir()) / f"helios_b200-build-{os.getuid()}"
    if _writable_dir(fallback):
        return fallback
    raise KernelBuildError(f"neither {local} nor {fallback} can be written")


def _digest(name: str, extra_flags: List[str]) -> str:
    h = hashlib.sha256()
    for f in [LIBRARIES[name]] + _HEADERS + _INCLUDES.get(name, []):
        h.update(f.encode())
        h.update((_SRC_DIR / f).read_bytes())
    h.update(" ".join(NVCC_FLAGS + extra_flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path:
    return build_dir() / f"{name}.{_digest(name, _extra_flags(name))}.so"


def _extra_flags(name: str) -> List[str]:
    """Per-library flags."""
    return list(EXTRA_FLAGS.get(name, []))


EXTRA_FLAGS: Dict[str, List[str]] = {}


def _compile(name: str, out: Path, verbose: bool) -> None:
    nvcc = _find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc] + NVCC_FLAGS + _extra_flags(name) + ["-o", str(tmp), str(_SRC_DIR / LIBRARIES[name])]
    t0 = time.time()
    print(f"[helios_b200] compiling {LIBRARIES[name]} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=str(_SRC_DIR))
    done = threading.Event()

    def _tick():
        while not done.wait(8.0):
            print(f"[helios_b200] still compiling {LIBRARIES[name]} ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)

    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        output, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {LIBRARIES[name]}:\n{' '.join(cmd)}\n"
                               + output.decode(errors="replace"))
    os.replace(tmp, out)
    if verbose:
        print(output.decode(errors="replace"), file=sys.stderr)
    print(f"[helios_b200] compiled {LIBRARIES[name]} in {time.time() - t0:.1f} s -> {out}",
          file=sys.stderr, flush=True)


def load_library(name: str, verbose: bool = False) -> ctypes.CDLL:
    """The loaded library ``name``, compiled first if it is not there yet."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        if name not in LIBRARIES:
            raise KernelBuildError(f"unknown kernel library {name!r}")
        out = library_path(name)
        if not out.exists():
            _compile(name, out, verbose)
        try:
            lib = ctypes.CDLL(str(out))
        except OSError as exc:
            raise KernelBuildError(f"cannot load {out}: {exc}") from None
        _loaded[name] = lib
        return lib


def build_all(names: Optional[List[str]] = None, verbose: bool = False) -> List[Path]:
    """Compile every library (in parallel processes) without loading any."""
    names = list(names or LIBRARIES)
    todo = [(n, library_path(n)) for n in names]
    todo = [(n, p) for n, p in todo if not p.exists()]
    errors: List[str] = []

    def _one(n, p):
        try:
            _compile(n, p, verbose)
        except KernelBuildError as exc:
            errors.append(str(exc))

    threads = [threading.Thread(target=_one, args=t) for t in todo]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise KernelBuildError("\n".join(errors))
    return [library_path(n) for n in names]
