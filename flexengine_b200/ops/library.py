"""Building and loading the CUDA kernel libraries.

The kernels are plain ``extern "C"`` entry points compiled by nvcc for sm_100a into
shared libraries that live inside the package (``_build/``), loaded with ctypes.  A
library is compiled on first use when no build that matches its sources exists, with a
line of progress per file; there is no fallback of any kind: if the compiler or the
GPU is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--compiler-options", "-fPIC", "-Xptxas", "-v"]

# library -> its sources; each library is what one kind of work needs, so that a first call
# compiles only that
GROUPS = {
    "core": ["errors.cu", "elementwise.cu", "attention_simt.cu", "gemm_fp32.cu", "sampling.cu"],
    # elementwise.cu once more: the layer executor launches its kernels from inside this library
    "bf16": ["errors.cu", "attention_mma.cu", "attention_tcgen05.cu", "gemm_skinny.cu", "gemm_tcgen05.cu", "elementwise.cu",
             "layer_executor.cu"],
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelLibraryError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[flexengine_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("FLEXENGINE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelLibraryError("nvcc was not found (looked at FLEXENGINE_NVCC, PATH, CUDA_HOME, /usr/local/cuda); "
                             "the CUDA kernels cannot be built and there is no other path")


def build_root() -> str:
    env = os.environ.get("FLEXENGINE_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(os.path.dirname(CSRC), "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"flexengine_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _sources_hash(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    names = sorted(GROUPS[group]) + sorted(n for n in os.listdir(CSRC) if n.endswith((".cuh", ".h")))
    for name in names:
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def library_path(group: str) -> str:
    return os.path.join(build_root(), f"libflexengine_{group}.{_sources_hash(group)}.so")


def build(group: str, force: bool = False, verbose: bool = True) -> str:
    """Compile library ``group`` if no build of its current sources exists; returns its path."""
    path = library_path(group)
    if os.path.isfile(path) and not force:
        return path
    nvcc = find_nvcc()
    root = os.path.dirname(path)
    with open(os.path.join(root, f".{group}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if os.path.isfile(path) and not force:
            return path
        objdir = os.path.join(root, f"obj_{group}_{_sources_hash(group)}")
        os.makedirs(objdir, exist_ok=True)
        sources = GROUPS[group]
        started = time.time()
        if verbose:
            _log(f"compiling the '{group}' kernels for sm_100a ({len(sources)} files, first call only) ...")
        done = []

        def compile_one(name: str) -> str:
            obj = os.path.join(objdir, name.replace(".cu", ".o"))
            cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise KernelLibraryError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
            with open(obj + ".log", "w") as f:
                f.write(proc.stderr)
            done.append(name)
            if verbose:
                _log(f"  compiled {name} ({len(done)}/{len(sources)}, {time.time() - started:.0f} s)")
            return obj

        stop = threading.Event()

        def heartbeat():
            while not stop.wait(15.0):
                _log(f"  still compiling ... {time.time() - started:.0f} s")

        beat = threading.Thread(target=heartbeat, daemon=True)
        if verbose:
            beat.start()
        try:
            with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2)) as pool:
                objects = list(pool.map(compile_one, sources))
            tmp = path + f".tmp{os.getpid()}"
            proc = subprocess.run([nvcc, "-shared", "-o", tmp, *objects, "-ldl"], capture_output=True, text=True)
            if proc.returncode != 0:
                raise KernelLibraryError(f"linking {group} failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp, path)
            _prune(root, group, keep=_sources_hash(group))
        finally:
            stop.set()
        if verbose:
            _log(f"built {os.path.basename(path)} in {time.time() - started:.0f} s")
    return path


def _prune(root: str, group: str, keep: str) -> None:
    """Remove builds of ``group`` made from older sources."""
    for name in os.listdir(root):
        stale_lib = name.startswith(f"libflexengine_{group}.") and name.endswith(".so") and keep not in name
        stale_obj = name.startswith(f"obj_{group}_") and keep not in name
        if stale_lib:
            try:
                os.remove(os.path.join(root, name))
            except OSError:
                pass
        elif stale_obj:
            shutil.rmtree(os.path.join(root, name), ignore_errors=True)


_PROTOTYPE = re.compile(r'extern\s+"C"\s+((?:const\s+)?[\w ]+?\s*\*?)\s*(fe_\w+)\s*\(([^)]*)\)', re.S)


def _ctype(decl: str, what: str):
    """The ctypes type of one C parameter or return declaration of an entry point."""
    text = decl.replace("const", " ").replace("__restrict__", " ").strip()
    if "*" in text:
        return ctypes.c_char_p if what == "return" and "char" in text else ctypes.c_void_p
    words = text.split()
    if what == "parameter" and len(words) > 1:
        words = words[:-1]                       # the parameter's name
    kind = " ".join(words)
    table = {"int": ctypes.c_int, "long long": ctypes.c_longlong, "float": ctypes.c_float,
             "cudaStream_t": ctypes.c_void_p, "void": None}
    if kind not in table:
        raise KernelLibraryError(f"entry point declares a type this loader does not know: '{decl.strip()}'")
    return table[kind]


def prototypes(group: str) -> dict:
    """{entry point: (return type, [parameter types])} read from the ``extern "C"`` declarations of the group's
    sources, so that the types ctypes converts to are the ones the C side declares (and a call with the wrong
    number of arguments is refused before it reaches the device)."""
    found = {}
    for name in GROUPS[group]:
        with open(os.path.join(CSRC, name)) as f:
            text = f.read()
        for ret, fn, params in _PROTOTYPE.findall(text):
            params = params.strip()
            args = [] if params in ("", "void") else [_ctype(a, "parameter") for a in params.split(",")]
            found[fn] = (_ctype(ret, "return"), args)
    return found


def load(group: str) -> ctypes.CDLL:
    """The loaded library ``group``; builds it first when needed.  Raises when it cannot be had."""
    with _lock:
        if group in _loaded:
            return _loaded[group]
        path = build(group)
        try:
            lib = ctypes.CDLL(path)
        except OSError as ex:
            raise KernelLibraryError(f"cannot load {path}: {ex}") from ex
        for fn, (restype, argtypes) in prototypes(group).items():
            entry = getattr(lib, fn)
            entry.restype, entry.argtypes = restype, argtypes
        # programmatic dependent launch (a kernel's preamble overlaps the tail of the one before): off unless
        # FLEXENGINE_PDL names classes of kernels (a sum of 1 streaming products, 2 decode attention, 4 elementwise,
        # 8 sampling, 16 decode attention in clusters, 128 the rest)
        lib.fe_set_pdl(ctypes.c_int(int(os.environ.get("FLEXENGINE_PDL", "0") or 0)))
        _loaded[group] = lib
        return lib


def build_all(force: bool = False) -> list[str]:
    return [build(g, force=force) for g in GROUPS]
