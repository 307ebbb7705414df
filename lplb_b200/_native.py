"""Build and load the native sm_100a extension.

The shared object is built in-tree (``lplb_b200/_build/``) ahead of time with
``nvcc -gencode arch=compute_100a,code=sm_100a`` through ``torch.utils.cpp_extension``;
nothing is compiled at run time on the GPU host.  This replaces the reference's NVRTC +
nvJitLink run-time compilation and on-disk cubin cache
(reference ``csrc/plugin.cpp:149-327``) and its ``setup.py`` (reference ``setup.py:1-50``).

A fingerprint of the sources is stored next to the binary; ``load()`` uses the existing
binary when the fingerprint matches and rebuilds otherwise (when a compiler is present).

``LPLB_B200_DEBUG_BOUNDS=1`` selects the bounds-checking variant: the same sources compiled
with ``-DLPLB_BOUNDS_CHECK`` into a build directory of their own (``_build_bounds/``).  In that
variant every data-dependent shared- or global-memory index of the planner and MoE support
kernels is range-checked; a violation is recorded in the status block and the access is
skipped.  It stands in for a memory checker where none can be run.
"""

from __future__ import annotations

import hashlib
import importlib.util
import logging
import os
import sys
from pathlib import Path

log = logging.getLogger("lplb_b200")

_ROOT = Path(__file__).resolve().parent
_CSRC = _ROOT / "csrc"
# Where the binary and its fingerprint live.  LPLB_B200_CACHE_PATH relocates it (the
# reference's LPLB_CACHE_PATH does the same for its JIT cache, reference csrc/plugin.cpp:207-214).
BOUNDS_CHECK = os.environ.get("LPLB_B200_DEBUG_BOUNDS") == "1"
_BUILD = Path(os.environ["LPLB_B200_CACHE_PATH"]) if os.environ.get("LPLB_B200_CACHE_PATH") else _ROOT / "_build"
_NAME = "lplb_b200_native"
if BOUNDS_CHECK:
    _BUILD = _BUILD.with_name(_BUILD.name + "_bounds")
    _NAME = "lplb_b200_native_bounds"

SOURCES = [
    "binding.cpp",
    "planner_launch.cu",
    "count_noalloc.cu",
    "moe_binding.cpp",
    "moe_launch.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
] + (["-DLPLB_BOUNDS_CHECK"] if BOUNDS_CHECK else [])

_module = None


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sorted(_CSRC.iterdir()):
        if path.suffix in (".cu", ".cuh", ".h", ".cpp"):
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return _BUILD / f"{_NAME}.so"


def is_built() -> bool:
    stamp = _BUILD / "fingerprint"
    return _so_path().exists() and stamp.exists() and stamp.read_text().strip() == _fingerprint()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA/C++ source for sm_100a into ``_build/`` (no GPU needed)."""
    if is_built() and not force:
        return _so_path()
    from torch.utils import cpp_extension

    _BUILD.mkdir(exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=_NAME,
        sources=[str(_CSRC / s) for s in SOURCES],
        extra_cflags=["-O2", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(_CSRC)],
        build_directory=str(_BUILD),
        verbose=verbose,
        is_python_module=False,
    )
    (_BUILD / "fingerprint").write_text(_fingerprint())
    return _so_path()


def load():
    """Import the extension module, building it first if that is possible and needed."""
    global _module
    if _module is not None:
        return _module
    so = _so_path()
    if not is_built():
        if so.exists() and os.environ.get("LPLB_B200_NO_REBUILD") == "1":
            log.warning("native extension is older than its sources; using it as is")
        else:
            try:
                build()
            except Exception as exc:  # no compiler, no nvcc, ...
                if not so.exists():
                    raise ImportError(f"lplb_b200 native extension is not built and cannot be built here: {exc}") from exc
                log.warning("rebuild failed (%s); using the existing binary", exc)
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(_NAME, so)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[_NAME] = module
    _module = module
    return module


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False
