"""Compiling the CUDA sources under csrc/ for sm_100a and loading them through ctypes.

Each .cu file becomes one shared library, built with nvcc alone (no torch
headers: a library compiles in seconds). A library is compiled at its first
use, so a model compiles what it needs; `build_all` compiles everything.
Built libraries go to csrc/_build/ inside the package when that is writable,
else to a per-user folder under the system's temporary directory. A library is
rebuilt when its source, a header or the flags change.

There is no fallback: if a library is neither built nor buildable, loading it
raises KernelBuildError.
"""
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
MODULES = ("elementwise", "gemm_simt", "gemm_tc", "attention_generic", "attention_decode", "attention_mma", "gemm_rows",
           "sampling", "attention_decode_static", "attention_decode_ring", "attention_tc", "utility", "step")


# ABACUS_TRACE=1 builds every library with the launch-timeline records of csrc/common.cuh compiled in
TRACE = os.environ.get("ABACUS_TRACE", "0") not in ("", "0")


def _module_flags(module):
    return [f"-DABK_TRACE={MODULES.index(module)}"] if TRACE else []


class KernelBuildError(RuntimeError):
    pass


_loaded = {}
_lock = threading.Lock()


def available_modules():
    return [m for m in MODULES if os.path.exists(os.path.join(CSRC, m + ".cu"))]


def _nvcc():
    for cand in (os.environ.get("ABACUS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


_build_dir_found = None


def _build_dir():
    """Where built libraries go: csrc/_build/ if it can be written, else a per-user folder under the system's
    temporary directory. Decided once per process (threads that compile side by side must agree)."""
    global _build_dir_found
    if _build_dir_found is not None:
        return _build_dir_found
    inside = os.path.join(CSRC, "_build")
    try:
        os.makedirs(inside, exist_ok=True)
        fd, probe = tempfile.mkstemp(prefix=".w", dir=inside)
        os.close(fd)
        os.remove(probe)
        found = inside
    except OSError:
        found = os.path.join(tempfile.gettempdir(), f"abacus_b200-build-{os.getuid()}")
        os.makedirs(found, exist_ok=True)
    _build_dir_found = found
    return found


def _fingerprint(module):
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + _module_flags(module)).encode())
    with open(os.path.join(CSRC, module + ".cu")) as f:
        included = {line.split('"')[1] for line in f if line.startswith("#include \"") and line.count('"') >= 2}
    for name in sorted(os.listdir(CSRC)):
        if name == module + ".cu" or name.endswith((".cuh", ".h")) or name in included:
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    return h.hexdigest()


def library_path(module):
    return os.path.join(_build_dir(), f"libabacus_{module}.so")


def _is_current(module):
    path = library_path(module)
    try:
        with open(path + ".stamp") as f:
            return os.path.exists(path) and f.read().strip() == _fingerprint(module)
    except OSError:
        return False


def compile_module(module, verbose=True, extra_flags=()):
    """Compile csrc/<module>.cu into its shared library; returns the path."""
    src = os.path.join(CSRC, module + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no kernel source {src}")
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelBuildError(f"the kernel library for {module!r} is not built and nvcc was not found "
                               "(set ABACUS_NVCC or put nvcc on PATH)")
    out = library_path(module)
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *_module_flags(module), *extra_flags, "-I", CSRC, "-o", tmp, src]
    if verbose:
        print(f"abacus_b200: compiling {module}.cu for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def progress():
        while not done.wait(10.0):
            if verbose:
                print(f"abacus_b200: still compiling {module}.cu ({time.time() - start:.0f} s)", file=sys.stderr,
                      flush=True)

    ticker = threading.Thread(target=progress, daemon=True)
    ticker.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {module}.cu:\n{log}")
    os.replace(tmp, out)
    with open(out + ".stamp", "w") as f:
        f.write(_fingerprint(module))
    if verbose:
        print(f"abacus_b200: compiled {module}.cu in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
    return out


def load_module(module):
    """The ctypes library of csrc/<module>.cu, compiled first if it is missing or stale."""
    with _lock:
        if module in _loaded:
            return _loaded[module]
        if not _is_current(module):
            compile_module(module)
        try:
            lib = ctypes.CDLL(library_path(module))
        except OSError as e:
            raise KernelBuildError(f"cannot load {library_path(module)}: {e}") from None
        lib.abk_last_error.restype = ctypes.c_char_p
        _loaded[module] = lib
        return lib


def build_all(verbose=True):
    """Compile every kernel source that is missing or stale, a few at a time."""
    todo = [m for m in available_modules() if not _is_current(m)]
    errors = []

    def work(m):
        try:
            compile_module(m, verbose)
        except KernelBuildError as e:
            errors.append(str(e))

    threads = [threading.Thread(target=work, args=(m,)) for m in todo]
    for i in range(0, len(threads), 4):
        for t in threads[i:i + 4]:
            t.start()
        for t in threads[i:i + 4]:
            t.join()
    if errors:
        raise KernelBuildError("\n".join(errors))
    return [library_path(m) for m in available_modules()]
