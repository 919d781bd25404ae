"""Builds and loads the native sm_100a extension (`_b200ep_C`) IN-TREE.

The shared object lives under `gpu_data_transfer_profile_b200/_C_build/` so that it travels
with the source tree; a content hash of the sources is stored beside it and a stale or
missing object is rebuilt (nvcc cross-compiles without a GPU). There is no Python fallback
for the kernels: on a machine with a GPU a missing extension is an error, not a slow path.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = REPO_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_C_build"
NAME = "_b200ep_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]

_lock = threading.Lock()
_mod = None


def sources():
    out = [CSRC / "bindings.cpp"]
    out += sorted(CSRC.glob("*/*.cu")) + sorted(CSRC.glob("*/*.cpp"))
    return [p for p in out if p.exists()]


def _all_inputs():
    return sorted(set(sources()) | set(CSRC.glob("**/*.h")) | set(CSRC.glob("**/*.cuh"))
                  | set(CSRC.glob("**/*.inc")))


def source_hash() -> str:
    h = hashlib.sha256()
    for p in _all_inputs():
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return BUILD_DIR / f"{NAME}.so"


def is_built() -> bool:
    stamp = BUILD_DIR / "source.sha256"
    return _so_path().exists() and stamp.exists() and stamp.read_text().strip() == source_hash()


def build(verbose: bool = False):
    """Compile every CUDA/C++ source for sm_100a and return the loaded module."""
    import torch  # noqa: F401
    from torch.utils import cpp_extension
    BUILD_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    inc = [str(CSRC)]
    cutlass = cutlass_include_dir()
    if cutlass:
        inc.append(cutlass)
    mod = cpp_extension.load(
        name=NAME, sources=[str(s) for s in sources()], build_directory=str(BUILD_DIR),
        extra_include_paths=inc, extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS, extra_ldflags=["-lcuda"], verbose=verbose)
    (BUILD_DIR / "source.sha256").write_text(source_hash())
    return mod


def cutlass_include_dir():
    """CUTLASS/CuTe headers vendored inside an installed Python package, if any."""
    for base in sys.path:
        for rel in ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include"):
            p = Path(base) / rel
            if (p / "cute" / "tensor.hpp").exists():
                return str(p)
    return None


def _import_so():
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location(NAME, str(_so_path()))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[NAME] = mod
    return mod


def load():
    """Return the native module, building it when missing or stale."""
    global _mod
    with _lock:
        if _mod is None:
            if is_built():
                _mod = _import_so()
            else:
                _mod = build()
        return _mod


def loaded_path() -> str:
    return str(_so_path())
