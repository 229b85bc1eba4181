"""Builds and loads the CUDA extension (sm_100a only), in the tree.

The library's name carries a hash of the sources, the flags and the torch version, so a
built library is loaded as it is when nothing changed (no rebuild on a machine that
received the tree with the library in it) and rebuilt when anything did.  The build
folder is ``csrc/_build`` inside the package; if that cannot be written (a read-only
checkout) a folder under the system's temporary directory is used.  Nothing is read
from or written to the home directory.  While compiling, a line is printed every few
seconds so that a first call does not look hung.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))

SOURCES = [
    "binding.cpp",
    "elementwise.cu",
    "gemm_simt.cu",
    "attention_simt.cu",
    "attention_mma.cu",
    "attention_decode.cu",
    "attention_decode_boxes.cu",
    "attention_tc.cu",
    "gemm_skinny.cu",
    "gemm_tc.cu",
    "gemm_tc_pair.cu",
    "attention_noalloc.cu",
    "sampling.cu",
]
HEADERS = ["common.cuh", "kernels.h", "launch.cuh", "tc_common.cuh", "gemm_epilogue.cuh", "attention_mma.cuh", "attention_decode.cuh", "attention_noalloc.h"]

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17"]

_loaded = None


def _hash() -> str:
    import torch
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(CUDA_FLAGS + CXX_FLAGS).encode())
    h.update(torch.__version__.encode())
    return h.hexdigest()[:12]


def _build_root() -> str:
    for root in (os.path.join(_HERE, "_build"),
                 os.path.join(tempfile.gettempdir(), f"vt_transformer_b200_build_{os.getuid()}")):
        try:
            os.makedirs(root, exist_ok=True)
            probe = os.path.join(root, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return root
        except OSError:
            continue
    raise RuntimeError("no writable folder to build the CUDA extension in")


def extension_name() -> str:
    return f"vtb200_ext_{_hash()}"


def find_built():
    """Path of the built library for the present sources, or None."""
    name = extension_name()
    for root in (os.path.join(_HERE, "_build"),
                 os.path.join(tempfile.gettempdir(), f"vt_transformer_b200_build_{os.getuid()}")):
        path = os.path.join(root, name, name + ".so")
        if os.path.isfile(path):
            return path
    return None


def _import(path: str, name: str):
    import torch  # noqa: F401  (its libraries must be loaded first)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load(verbose: bool = False):
    """The extension module; compiled first if no built library matches the sources."""
    global _loaded
    if _loaded is not None:
        return _loaded
    name = extension_name()
    path = find_built()
    if path is None:
        path = _compile(name, verbose)
    _loaded = _import(path, name)
    return _loaded


def _compile(name: str, verbose: bool) -> str:
    from torch.utils import cpp_extension
    if cpp_extension.CUDA_HOME is None:
        raise RuntimeError("the CUDA extension has to be compiled but no CUDA toolkit (nvcc) was found; "
                           "there is no CPU path")
    build_dir = os.path.join(_build_root(), name)
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 1)))
    stop = threading.Event()
    t0 = time.time()

    def _tick():
        while not stop.wait(10.0):
            print(f"[vt_transformer_b200] compiling CUDA kernels for sm_100a ... {time.time() - t0:.0f} s",
                  file=sys.stderr, flush=True)

    print(f"[vt_transformer_b200] compiling CUDA kernels for sm_100a into {build_dir} (first call only)",
          file=sys.stderr, flush=True)
    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        cpp_extension.load(
            name=name,
            sources=[os.path.join(_HERE, s) for s in SOURCES],
            extra_cflags=CXX_FLAGS,
            extra_cuda_cflags=CUDA_FLAGS,
            extra_include_paths=[_HERE],
            build_directory=build_dir,
            verbose=verbose,
            is_python_module=False,
        )
    finally:
        stop.set()
    path = os.path.join(build_dir, name + ".so")
    if not os.path.isfile(path):
        raise RuntimeError(f"the build finished but {path} is missing")
    print(f"[vt_transformer_b200] compiled in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    _remove_stale(os.path.dirname(build_dir), name)
    return path


def _remove_stale(root: str, keep: str, prefix: str = "vtb200_ext_") -> None:
    """Deletes the builds of earlier sources beside the one just made."""
    import shutil
    for entry in os.listdir(root):
        if entry.startswith(prefix) and entry != keep:
            shutil.rmtree(os.path.join(root, entry), ignore_errors=True)


# ---- the host-side module: C++ without CUDA, compiled with the host compiler alone -------------------------

HOST_SOURCE = "host_runtime.cpp"
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]
_host = None


def _host_name() -> str:
    h = hashlib.sha256()
    with open(os.path.join(_HERE, HOST_SOURCE), "rb") as f:
        h.update(f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    h.update(sys.version.encode())
    return f"vtb200_host_{h.hexdigest()[:12]}"


def load_host():
    """The module of ``host_runtime.cpp`` (the cache manager's bookkeeping and the packing of a step's
    description); compiled with the host compiler at the first call, into the same build folder."""
    global _host
    if _host is not None:
        return _host
    name = _host_name()
    path = None
    for root in (os.path.join(_HERE, "_build"),
                 os.path.join(tempfile.gettempdir(), f"vt_transformer_b200_build_{os.getuid()}")):
        cand = os.path.join(root, name, name + ".so")
        if os.path.isfile(cand):
            path = cand
            break
    if path is None:
        path = _compile_host(name)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _host = mod
    return mod


def _compile_host(name: str) -> str:
    import shutil
    import subprocess
    import sysconfig
    try:
        import pybind11
        pybind_include = pybind11.get_include()
    except ImportError:                       # the headers that come with torch
        import torch
        pybind_include = os.path.join(os.path.dirname(torch.__file__), "include")
    compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        raise RuntimeError("the host-side module has to be compiled but no C++ compiler (g++) was found")
    build_dir = os.path.join(_build_root(), name)
    os.makedirs(build_dir, exist_ok=True)
    out = os.path.join(build_dir, name + ".so")
    tmp = out + f".tmp{os.getpid()}"
    cmd = [compiler, *HOST_FLAGS, f"-DVTB_HOST_MODULE_NAME={name}", "-I", pybind_include,
           "-I", sysconfig.get_paths()["include"], os.path.join(_HERE, HOST_SOURCE), "-o", tmp]
    print(f"[vt_transformer_b200] compiling the host-side module into {build_dir} (first call only)",
          file=sys.stderr, flush=True)
    t0 = time.time()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("compiling host_runtime.cpp failed:\n" + " ".join(cmd) + "\n" + res.stderr[-4000:])
    os.replace(tmp, out)
    print(f"[vt_transformer_b200] compiled in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    _remove_stale(os.path.dirname(build_dir), name, prefix="vtb200_host_")
    return out
