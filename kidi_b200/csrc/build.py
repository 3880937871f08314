"""Compiles the CUDA sources of this folder for sm_100a and loads them.

The kernels are plain CUDA with a C interface: no framework headers, so a file
compiles in seconds with `nvcc` alone. A library is a set of sources plus
preprocessor definitions; its shared object is named by a hash of everything that
goes into it (sources, headers, flags), is built at the first call that needs it
and is found again by later calls and other processes. Sources that are specialised
by a size (a head width, say) are compiled for the sizes a loaded model has, not
for every size there could be.

The shared objects live in `build/` beside the sources when that folder can be
written, otherwise under the user's cache folder or the temporary folder. While a
compilation runs, a line is printed to stderr now and then so that a first call
does not look hung. If no compiler is found or a compilation fails, an error is
raised: there is no fallback path.
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
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Mapping, Optional, Sequence, Tuple

from ..errors import runtime_error

SOURCE_DIR = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden"]

# The libraries of the package: name -> sources. Definitions are added per request.
LIBRARIES: Dict[str, Tuple[str, ...]] = {
    "core": ("elementwise.cu", "gemm_simt.cu", "gemm_skinny.cu", "gemm_tcgen05.cu", "attention_generic.cu",
             "sampling.cu"),
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _say(message: str) -> None:
    print(f"[kidi_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("KIDI_B200_NVCC")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(os.path.join(home, "bin", "nvcc"))
    candidates.append(shutil.which("nvcc"))
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise runtime_error("the CUDA kernels have to be compiled and no nvcc was found "
                        "(looked at KIDI_B200_NVCC, CUDA_HOME, /usr/local/cuda/bin and PATH)")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = tempfile.NamedTemporaryFile(dir=path, prefix=".probe", delete=True)
        probe.close()
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("KIDI_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(SOURCE_DIR, "build"))
    cache_home = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    candidates.append(os.path.join(cache_home, "kidi_b200"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"kidi_b200-{os.getuid()}"))
    for candidate in candidates:
        if candidate and _writable_dir(candidate):
            return candidate
    raise runtime_error("no folder to build the CUDA kernels in can be written")


def _headers() -> Sequence[str]:
    return sorted(name for name in os.listdir(SOURCE_DIR) if name.endswith((".cuh", ".h")))


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    digest = hashlib.sha256()
    for name in list(sources) + list(_headers()):
        digest.update(name.encode())
        with open(os.path.join(SOURCE_DIR, name), "rb") as handle:
            digest.update(handle.read())
    # The include path is where this checkout lies: a library built in one place is the same
    # library in a copy of the tree elsewhere.
    digest.update("\0".join(flag for flag in flags if flag != SOURCE_DIR).encode())
    return digest.hexdigest()[:16]


def library_flags(defines: Optional[Mapping[str, object]] = None) -> Sequence[str]:
    flags = list(ARCH_FLAGS) + list(COMMON_FLAGS) + ["-I", SOURCE_DIR]
    for key, value in sorted((defines or {}).items()):
        flags.append(f"-D{key}={value}")
    return flags


def _compile(nvcc: str, source: str, obj: str, flags: Sequence[str]) -> None:
    command = [nvcc, *flags, "-c", os.path.join(SOURCE_DIR, source), "-o", obj]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise runtime_error(f"nvcc failed on {source}:\n{' '.join(command)}\n{result.stdout}\n{result.stderr}")


def _remove_older_builds(folder: str, name: str, keep: str) -> None:
    """Drops the shared objects of earlier versions of a library's sources (a process that
    has one loaded keeps its mapping) and the lock files left from building them."""
    kept_tag = os.path.basename(keep)[len(f"libkidi_{name}_"):-3]
    for prefix, suffix in ((f"libkidi_{name}_", ".so"), (f".{name}_", ".lock")):
        for entry in os.listdir(folder):
            stem = entry[len(prefix):-len(suffix)] if entry.startswith(prefix) and entry.endswith(suffix) else ""
            if stem != kept_tag and len(stem) == 16 and all(c in "0123456789abcdef" for c in stem):
                try:
                    os.remove(os.path.join(folder, entry))
                except OSError:
                    pass


def build_library(name: str, sources: Sequence[str], defines: Optional[Mapping[str, object]] = None,
                  verbose_ptxas: bool = False) -> str:
    """Builds (if it is not there yet) and returns the path of the shared object."""
    flags = list(library_flags(defines))
    if verbose_ptxas:
        flags += ["-Xptxas", "-v"]
    tag = _digest(sources, flags)
    folder = build_dir()
    target = os.path.join(folder, f"libkidi_{name}_{tag}.so")
    if os.path.exists(target):
        return target
    nvcc = find_nvcc()
    with open(os.path.join(folder, f".{name}_{tag}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(target):  # another process built it meanwhile
                return target
            started = time.time()
            _say(f"compiling library '{name}' for sm_100a ({len(sources)} source files; first use only)")
            stop = threading.Event()

            def heartbeat() -> None:
                while not stop.wait(10.0):
                    _say(f"still compiling '{name}' ({time.time() - started:.0f} s)")

            ticker = threading.Thread(target=heartbeat, daemon=True)
            ticker.start()
            work = tempfile.mkdtemp(prefix=f"{name}_{tag}_", dir=folder)
            try:
                objects = [os.path.join(work, os.path.splitext(source)[0] + ".o") for source in sources]
                with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 4)) as pool:
                    list(pool.map(lambda pair: _compile(nvcc, pair[0], pair[1], flags), zip(sources, objects)))
                partial = os.path.join(work, "lib.so")
                link = [nvcc, *ARCH_FLAGS, "-shared", "-o", partial, *objects, "-lcudart"]
                result = subprocess.run(link, capture_output=True, text=True)
                if result.returncode != 0:
                    raise runtime_error(f"linking '{name}' failed:\n{result.stdout}\n{result.stderr}")
                os.replace(partial, target)
                _remove_older_builds(folder, name, keep=target)
            finally:
                stop.set()
                shutil.rmtree(work, ignore_errors=True)
            _say(f"library '{name}' ready after {time.time() - started:.0f} s: {target}")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return target


def load_library(name: str, sources: Optional[Sequence[str]] = None,
                 defines: Optional[Mapping[str, object]] = None) -> ctypes.CDLL:
    """The loaded shared object of a library, compiled first if need be."""
    sources = tuple(sources) if sources is not None else LIBRARIES[name]
    key = name + "|" + ",".join(f"{k}={v}" for k, v in sorted((defines or {}).items()))
    with _lock:
        library = _loaded.get(key)
        if library is None:
            path = build_library(name, sources, defines)
            try:
                library = ctypes.CDLL(path)
            except OSError as error:
                raise runtime_error(f"cannot load {path}: {error}") from None
            _loaded[key] = library
        return library
