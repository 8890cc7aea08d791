"""Builds and loads the CUDA extension ``_C`` for sm_100a.

The reference builds its extension with a setup.py CUDAExtension for sm_86
(setup.py:7-31).  Here the same sources are compiled either ahead of time
(``python setup.py build_ext --inplace`` or :func:`build`) or at the first call that needs
a kernel: each ``.cu`` file goes through ``nvcc -gencode arch=compute_100a,code=sm_100a``
in parallel, ``bindings.cpp`` through the host compiler, and the objects are linked into
``_C.so`` next to this package (or, when the package folder is read-only, under the
system's temporary folder).  A stamp of the sources' hash decides whether the library on
disk is current, so a built library that was copied along with the sources is loaded as
is.  There is no fallback: if the extension cannot be built or loaded, the call fails.
"""

from __future__ import annotations

import fcntl
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(PACKAGE_DIR, "csrc")
MODULE_NAME = "ampere_kv_engine_b200._C"
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

_loaded = None
_lock = threading.Lock()


class ExtensionError(RuntimeError):
    """The CUDA extension is missing and could not be built, or failed to load."""


def _sources() -> list[str]:
    names = sorted(n for n in os.listdir(CSRC_DIR) if n.endswith((".cu", ".cpp")))
    return [os.path.join(CSRC_DIR, n) for n in names]


def _headers() -> list[str]:
    return [os.path.join(CSRC_DIR, n) for n in sorted(os.listdir(CSRC_DIR)) if n.endswith((".h", ".cuh"))]


def _flags_signature() -> str:
    import torch
    return f"torch={torch.__version__};py={sys.version_info[:2]};arch={NVCC_ARCH};v=3"


def source_hash() -> str:
    digest = hashlib.sha256(_flags_signature().encode())
    for path in _sources() + _headers():
        digest.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            digest.update(handle.read())
    return digest.hexdigest()[:16]


def _find_nvcc() -> str:
    for candidate in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if candidate and os.path.isfile(os.path.join(candidate, "bin", "nvcc")):
            return os.path.join(candidate, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise ExtensionError("nvcc not found (looked in CUDA_HOME, /usr/local/cuda and PATH); "
                         "the engine's kernels cannot be built")


def _writable(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _candidate_dirs(digest: str) -> list[tuple[str, str]]:
    """(folder of the .so, folder of the objects) in order of preference."""
    out = [(PACKAGE_DIR, os.path.join(PACKAGE_DIR, "_build"))]
    tmp = os.path.join(tempfile.gettempdir(), f"ampere_kv_engine_b200_{os.getuid()}_{digest}")
    out.append((tmp, os.path.join(tmp, "_build")))
    return out


def _stamp_path(so_dir: str) -> str:
    return os.path.join(so_dir, "_build", "stamp") if so_dir == PACKAGE_DIR else os.path.join(so_dir, "stamp")


def _is_current(so_dir: str, digest: str) -> bool:
    so = os.path.join(so_dir, "_C.so")
    stamp = _stamp_path(so_dir)
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp, "r", encoding="utf-8") as handle:
        return handle.read().strip() == digest


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise ExtensionError(f"building the CUDA extension failed at {what}:\n$ {' '.join(cmd)}\n{proc.stdout}")


def _say(verbose: bool, message: str) -> None:
    if verbose:
        print(f"[ampere_kv_engine_b200] {message}", file=sys.stderr, flush=True)


def _compile(so_dir: str, obj_dir: str, digest: str, verbose: bool, extra_nvcc: list[str]) -> str:
    import torch
    from torch.utils import cpp_extension

    nvcc = _find_nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    os.makedirs(obj_dir, exist_ok=True)
    includes = [f"-I{CSRC_DIR}", f"-I{os.path.join(cuda_home, 'include')}"]
    torch_includes = [f"-isystem{p}" for p in cpp_extension.include_paths()]
    torch_includes.append(f"-isystem{sysconfig.get_paths()['include']}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    host_cxx = os.environ.get("CXX", "g++")
    jobs: list[tuple[list[str], str, str]] = []
    objects: list[str] = []
    for src in _sources():
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objects.append(obj)
        if src.endswith(".cu"):
            cmd = [nvcc, "-O3", "-std=c++17", *NVCC_ARCH, "-lineinfo", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", *extra_nvcc, *includes, "-c", src, "-o", obj]
        else:
            cmd = [host_cxx, "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                   "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", *includes, *torch_includes,
                   "-c", src, "-o", obj]
        jobs.append((cmd, os.path.basename(src), obj))

    started = time.time()
    _say(verbose, f"compiling {len(jobs)} sources for sm_100a into {obj_dir} (first call only; about a minute)")
    done = []

    def work(job):
        cmd, name, _ = job
        _run(cmd, name)
        done.append(name)
        _say(verbose, f"  compiled {name} ({len(done)}/{len(jobs)}, {time.time() - started:.0f}s)")

    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
        futures = [pool.submit(work, job) for job in jobs]
        while True:
            pending = [f for f in futures if not f.done()]
            if not pending:
                break
            time.sleep(1.0)
            if int(time.time() - started) % 15 == 0:
                _say(verbose, f"  still compiling ({len(pending)} of {len(jobs)} left, {time.time() - started:.0f}s)")
        for f in futures:
            f.result()

    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    so_tmp = os.path.join(so_dir, f"_C.so.tmp{os.getpid()}")
    link = [host_cxx, "-shared", *objects, "-o", so_tmp, f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart"]
    _run(link, "link")
    os.replace(so_tmp, os.path.join(so_dir, "_C.so"))
    stamp = _stamp_path(so_dir)
    os.makedirs(os.path.dirname(stamp), exist_ok=True)
    with open(stamp, "w", encoding="utf-8") as handle:
        handle.write(digest)
    _say(verbose, f"built {os.path.join(so_dir, '_C.so')} in {time.time() - started:.0f}s")
    return os.path.join(so_dir, "_C.so")


def build(verbose: bool = True, force: bool = False, extra_nvcc: list[str] | None = None) -> str:
    """Make sure a current ``_C.so`` exists; returns its path.  Safe to call from several processes."""
    digest = source_hash()
    last_error: Exception | None = None
    for so_dir, obj_dir in _candidate_dirs(digest):
        if not force and _is_current(so_dir, digest):
            return os.path.join(so_dir, "_C.so")
        if not _writable(so_dir) or not _writable(obj_dir):
            continue
        lock_path = os.path.join(obj_dir, "lock")
        with open(lock_path, "w") as lock_file:
            fcntl.flock(lock_file, fcntl.LOCK_EX)
            try:
                if not force and _is_current(so_dir, digest):
                    return os.path.join(so_dir, "_C.so")
                return _compile(so_dir, obj_dir, digest, verbose, extra_nvcc or [])
            except ExtensionError as exc:
                last_error = exc
                raise
            finally:
                fcntl.flock(lock_file, fcntl.LOCK_UN)
    raise ExtensionError(f"no writable folder to build the CUDA extension in ({last_error})")


def load(verbose: bool = True):
    """The extension module ``_C``; built first if it is missing or stale.  Raises if it cannot be had."""
    global _loaded
    if _loaded is not None:
        return _loaded
    with _lock:
        if _loaded is not None:
            return _loaded
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        path = build(verbose=verbose)
        spec = importlib.util.spec_from_file_location(MODULE_NAME, path)
        if spec is None or spec.loader is None:
            raise ExtensionError(f"cannot load {path}")
        module = importlib.util.module_from_spec(spec)
        try:
            spec.loader.exec_module(module)
        except ImportError as exc:
            raise ExtensionError(f"the CUDA extension {path} failed to load: {exc}") from exc
        sys.modules[MODULE_NAME] = module
        _loaded = module
        return module
