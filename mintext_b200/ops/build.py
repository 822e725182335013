"""In-tree build of the CUDA/C++ extension for sm_100a.

``python -m mintext_b200.ops.build`` compiles every source under ``csrc/`` into
``mintext_b200/_mt_C.so`` (CUDA kernels + torch bindings), ``mintext_b200/_mt_C_dbg.so`` (the same sources with
``-DMINTEXT_DEBUG_BOUNDS``: data-dependent indices are range-checked, violations are recorded and skipped; selected
at run time with ``MT_DEBUG_BOUNDS=1``) and ``mintext_b200/_mt_io.so`` (host-only C++ runtime pieces).  nvcc cross-compiles without a GPU, so this also serves as the "does it build" check.
"""

from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]
CSRC = REPO_ROOT / "csrc"
PKG = REPO_ROOT / "mintext_b200"

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _cuda_sources() -> list[str]:
    return sorted(str(p) for p in CSRC.rglob("*.cu"))


def build_cuda(verbose: bool = False, debug_bounds: bool = False) -> Path:
    from torch.utils import cpp_extension

    name = "_mt_C_dbg" if debug_bounds else "_mt_C"
    build_dir = REPO_ROOT / "build" / name
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    sources = [str(CSRC / "bindings.cpp")] + _cuda_sources()
    define = ["-DMINTEXT_DEBUG_BOUNDS"] if debug_bounds else []
    cpp_extension.load(
        name=name,
        sources=sources,
        extra_cflags=["-O3", "-std=c++17"] + define,
        extra_cuda_cflags=CUDA_FLAGS + define,
        extra_include_paths=[str(CSRC)],
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=True,
    )
    out = PKG / f"{name}.so"
    shutil.copyfile(build_dir / f"{name}.so", out)
    return out


def build_io(verbose: bool = False) -> Path | None:
    """Host-only C++ runtime (data index builders, mmap reader, async checkpoint writer)."""
    src = sorted(str(p) for p in (CSRC / "io").glob("*.cpp") if p.name != "io_selftest.cpp")  # that one has a main()
    if not src:
        return None
    from torch.utils import cpp_extension

    build_dir = REPO_ROOT / "build" / "_mt_io"
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(
        name="_mt_io",
        sources=src,
        extra_cflags=["-O3", "-std=c++17", "-pthread"],
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=True,
    )
    out = PKG / "_mt_io.so"
    shutil.copyfile(build_dir / "_mt_io.so", out)
    return out


def build_all(verbose: bool = False) -> None:
    build_cuda(verbose)
    build_cuda(verbose, debug_bounds=True)
    build_io(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built:", [p.name for p in PKG.glob("_mt_*.so")])
