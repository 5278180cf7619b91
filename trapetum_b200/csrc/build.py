"""Compiling and loading the kernel libraries.

Each ``.cu`` file of this folder becomes one shared library for sm_100a, built
with nvcc at its first use and kept under ``_build/`` beside the sources (or in
a per-user temporary folder when the source tree cannot be written).  The file
name carries a hash of the source, of the shared headers and of the flags, so an
edited kernel is rebuilt and a stale library is never loaded.  The libraries
export plain C functions and are loaded with ctypes; they do not link against
torch.  There is no fallback: if a library cannot be built or loaded, the call
raises.
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
from typing import Dict, Iterable, List

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]

# every kernel file of the package; build_all() compiles them all.  A name of the form
# "file@MACRO=value" is the file compiled with -DMACRO=value (one library per value).
SOURCES = ["embed", "norm", "rope_kv", "activation", "gemm_simt", "gemm_tc", "attention_simt", "attention_decode", "sampling", "random_init"] + \
    [f"attention_prefill@TB_HD={hd}" for hd in (16, 32, 48, 64, 128, 256)] + \
    [f"attention_prefill_tc@TB_HD={hd}" for hd in (64, 128, 256)]


class KernelBuildError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("TRAPETUM_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $TRAPETUM_NVCC, $CUDA_HOME/bin, PATH and "
                           "/usr/local/cuda/bin); the CUDA kernels cannot be built and there is no fallback")


_build_dir_cached = None


def _build_dir() -> str:
    """The folder the libraries live in; decided once per process."""
    global _build_dir_cached
    if _build_dir_cached is None:
        with _dir_lock:
            if _build_dir_cached is None:
                _build_dir_cached = _pick_build_dir()
    return _build_dir_cached


def _pick_build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"trapetum_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _split(name: str):
    """"file@MACRO=value" -> (file, ["-DMACRO=value"], "file_MACROvalue")."""
    if "@" not in name:
        return name, [], name
    base, macro = name.split("@", 1)
    return base, ["-D" + macro], base + "_" + macro.replace("=", "")


def _digest(name: str) -> str:
    name, defines, _ = _split(name)
    h = hashlib.sha256()
    h.update(" ".join(defines).encode())
    headers = sorted(fn for fn in os.listdir(_HERE) if fn.endswith((".cuh", ".h")))
    for fn in [name + ".cu"] + headers:
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"tb_{_split(name)[2]}-{_digest(name)}.so")


def _say(msg: str) -> None:
    print(f"[trapetum_b200] {msg}", file=sys.stderr, flush=True)


def _compile(name: str) -> str:
    out = library_path(name)
    if os.path.exists(out):
        return out
    base, defines, _ = _split(name)
    src = os.path.join(_HERE, base + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no kernel source {src}")
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + NVCC_FLAGS + defines + ["-I", _HERE, "-o", tmp, src]
    _say(f"compiling {base}.cu {' '.join(defines)} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=os.path.dirname(out))
    while True:
        try:
            log, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {base}.cu ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise KernelBuildError(f"nvcc failed on {base}.cu {' '.join(defines)}:\n{log}")
    os.replace(tmp, out)
    _say(f"  built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def require(names: Iterable[str]) -> None:
    """Build (in parallel) whatever of ``names`` is not built yet."""
    todo = [n for n in dict.fromkeys(names) if n not in _libs and not os.path.exists(library_path(n))]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
        list(ex.map(_compile, todo))
    write_manifest()


def write_manifest() -> str:
    """``manifest.json`` in the build folder: kernel library name -> file, for every library that is built.
    The native host finds the kernels through it (the file names carry source hashes)."""
    import json
    entries = {n: os.path.basename(library_path(n)) for n in SOURCES if os.path.exists(library_path(n))}
    path = os.path.join(_build_dir(), "manifest.json")
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump(entries, f, indent=1, sort_keys=True)
    os.replace(tmp, path)
    return path


# ---------------------------------------------------------------------------
# The native host: libtrapetum_b200.so (C interface, see native/trapetum_b200.h) and the gemma_run binary
# ---------------------------------------------------------------------------
_NATIVE = os.path.join(os.path.dirname(_HERE), "native")
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function"]


def _native_digest() -> str:
    h = hashlib.sha256()
    for fn in sorted(os.listdir(_NATIVE)):
        if fn.endswith((".hpp", ".cpp", ".h")):
            with open(os.path.join(_NATIVE, fn), "rb") as f:
                h.update(fn.encode() + f.read())
    with open(os.path.join(_HERE, "decode_args.h"), "rb") as f:
        h.update(f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:16]


def native_library_path() -> str:
    return os.path.join(_build_dir(), f"libtrapetum_b200-{_native_digest()}.so")


def native_binary_path() -> str:
    return os.path.join(_build_dir(), f"gemma_run-{_native_digest()}")


def _host_compiler() -> str:
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise KernelBuildError("no C++ compiler (g++) was found; the native host cannot be built")
    return cxx


def _run(cmd, what: str) -> None:
    _say(f"compiling {what} ...")
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"building {what} failed:\n{proc.stdout}")
    _say(f"  built {what} in {time.time() - t0:.1f} s")


def build_native() -> str:
    """Compile the native host library and the ``gemma_run`` binary (once per source state); returns the
    library's path.  Stable names (``libtrapetum_b200.so``, ``gemma_run``) point at the current builds."""
    lib, exe = native_library_path(), native_binary_path()
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    with _lock:
        if not os.path.exists(lib):
            tmp = f"{lib}.{os.getpid()}.tmp"
            _run([_host_compiler()] + HOST_FLAGS + ["-shared", "-I", os.path.join(cuda, "include"),
                  os.path.join(_NATIVE, "c_api.cpp"), "-o", tmp, "-L", os.path.join(cuda, "lib64"),
                  "-lcudart_static", "-ldl", "-lrt", "-lpthread"], "the native host library")
            os.replace(tmp, lib)
        if not os.path.exists(exe):
            tmp = f"{exe}.{os.getpid()}.tmp"
            _run([_host_compiler()] + HOST_FLAGS + [os.path.join(_NATIVE, "gemma_run.cpp"), "-o", tmp, lib,
                  "-Wl,-rpath,$ORIGIN", "-ldl", "-lpthread"], "the gemma_run binary")
            os.replace(tmp, exe)
        for target, name in ((lib, "libtrapetum_b200.so"), (exe, "gemma_run")):
            link = os.path.join(_build_dir(), name)
            try:
                if os.path.lexists(link):
                    os.unlink(link)
                os.symlink(os.path.basename(target), link)
            except OSError:
                pass
    write_manifest()
    return lib


def load(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _libs.get(name)
        if lib is not None:
            return lib
        path = _compile(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        lib.tb_error.restype = ctypes.c_char_p
        _libs[name] = lib
        return lib


def loaded() -> List[str]:
    """Names of the kernel libraries this process has loaded so far."""
    return list(_libs)


def prune() -> int:
    """Remove libraries of earlier source states from the build folder (their names carry other hashes)."""
    keep = {os.path.basename(library_path(n)) for n in SOURCES}
    keep |= {os.path.basename(native_library_path()), os.path.basename(native_binary_path()), "manifest.json",
             "libtrapetum_b200.so", "gemma_run"}
    n = 0
    for fn in os.listdir(_build_dir()):
        if fn not in keep and (fn.startswith(("tb_", "libtrapetum_b200-", "gemma_run-")) or fn.endswith(".tmp")):
            try:
                os.unlink(os.path.join(_build_dir(), fn))
                n += 1
            except OSError:
                pass
    return n


def build_all() -> List[str]:
    require(SOURCES)
    write_manifest()
    out = [library_path(n) for n in SOURCES] + [build_native(), native_binary_path()]
    prune()
    return out
