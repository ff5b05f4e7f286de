"""In-tree build of the native extension (sm_100a only).

The extension is compiled into ``teramoe_b200/_ext/`` next to the sources, so the built ``.so``
travels with the source tree (no JIT cache outside the tree is involved).  ``load_ext()`` imports
the existing ``.so`` when its recorded source hash matches the current sources and rebuilds it
otherwise; a rebuild needs ``nvcc`` but no GPU.

Reference counterpart: setup.py:1-140 (torch CUDAExtension build with arch 9.0;10.0 and build-time
macros).  Here there is one target architecture and no build-time feature macro.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_EXT_DIR = _PKG / "_ext"
_NAME = "teramoe_b200_C"
_LOCK = threading.Lock()
_MOD = None

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17"]


def sources() -> list[Path]:
    return sorted(list(_CSRC.glob("*.cu")) + list(_CSRC.glob("*.cpp")))


def _source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(list(_CSRC.glob("*.cu")) + list(_CSRC.glob("*.cpp")) + list(_CSRC.glob("*.h")) + list(_CSRC.glob("*.cuh"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return _EXT_DIR / f"{_NAME}.so"


def _stamp_path() -> Path:
    return _EXT_DIR / f"{_NAME}.hash"


def is_built() -> bool:
    return _so_path().exists() and _stamp_path().exists() and _stamp_path().read_text().strip() == _source_hash()


def build(verbose: bool = False) -> Path:
    """Compile the extension for sm_100a into ``_ext/`` (no-op when up to date)."""
    if is_built():
        return _so_path()
    from torch.utils import cpp_extension

    _EXT_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=_NAME,
        sources=[str(p) for p in sources()],
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=CUDA_FLAGS,
        extra_include_paths=[str(_CSRC)],
        build_directory=str(_EXT_DIR),
        with_cuda=True,
        is_python_module=True,
        verbose=verbose,
    )
    _stamp_path().write_text(_source_hash())
    return _so_path()


def _rank_serialised_build() -> None:
    """Several ranks of one job may import at once; only local rank 0 compiles."""
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if local_rank == 0 or "LOCAL_RANK" not in os.environ:
        build()
        return
    import time

    for _ in range(1800):
        if is_built():
            return
        time.sleep(1.0)
    raise RuntimeError("teramoe_b200: timed out waiting for local rank 0 to build the native extension")


def load_ext():
    """Return the native module, building it first if needed.  Raises if it cannot be produced."""
    global _MOD
    with _LOCK:
        if _MOD is not None:
            return _MOD
        if not is_built():
            _rank_serialised_build()
        import torch  # noqa: F401  (the extension links against libtorch)

        spec = importlib.util.spec_from_file_location(_NAME, str(_so_path()))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[_NAME] = mod
        _MOD = mod
        return mod


def so_path() -> Path:
    return _so_path()
