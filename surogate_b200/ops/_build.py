"""Build / load the in-tree CUDA extension (sm_100a only).

``build()`` compiles every ``.cu`` / ``.cpp`` under ``csrc/`` with
``-gencode arch=compute_100a,code=sm_100a`` into ``surogate_b200/_ext/`` (kept in
the source tree so a snapshot of the repository carries the binary).
``load()`` imports the prebuilt module, building it first only when it is missing
or older than its sources.  On a machine with a GPU a missing extension is an
error: the CUDA ops never fall back silently to PyTorch.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
EXT_DIR = os.path.join(os.path.dirname(_HERE), "_ext")
EXT_NAME = "sg_b200_ext"
_lock = threading.Lock()
_module = None

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
              "-U__CUDA_NO_HALF2_OPERATORS__"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _so_path():
    return os.path.join(EXT_DIR, EXT_NAME + ".so")


def _stale() -> bool:
    so = _so_path()
    if not os.path.exists(so):
        return True
    t = os.path.getmtime(so)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False):
    """Compile the extension for sm_100a (works without a GPU: nvcc cross-compiles)."""
    from torch.utils import cpp_extension

    os.makedirs(EXT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    if force and os.path.exists(_so_path()):
        os.remove(_so_path())
    return cpp_extension.load(name=EXT_NAME, sources=sources(), extra_cuda_cflags=NVCC_FLAGS, extra_cflags=["-O2", "-std=c++17"],
                              extra_ldflags=["-lcuda"] if os.path.exists("/usr/lib/x86_64-linux-gnu/libcuda.so") else [],
                              build_directory=EXT_DIR, with_cuda=True, verbose=verbose)


def load():
    """Return the extension module (import the prebuilt .so; build when missing or stale)."""
    global _module
    with _lock:
        if _module is not None:
            return _module
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        if _stale() and os.environ.get("SUROGATE_NO_BUILD", "0") != "1":
            _module = build()
            return _module
        spec = importlib.util.spec_from_file_location(EXT_NAME, _so_path())
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[EXT_NAME] = mod
        _module = mod
        return _module


def available() -> bool:
    try:
        load()
        return True
    except Exception:  # noqa: BLE001
        return False
