"""Build the sm_100a extension in-tree: ``python -m deepfold3_dev_b200.ops.build``.

Sources under ``ops/csrc`` are compiled with ``-gencode arch=compute_100a,code=sm_100a`` (nvcc
cross-compiles without a GPU) and linked into ``ops/_df3_sm100.so``, which ``ops/native.py`` loads
with ``torch.ops.load_library``. Objects are cached under ``ops/_build`` and rebuilt when a source
or header is newer.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")
SO_PATH = os.path.join(HERE, "_df3_sm100.so")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _stale() -> bool:
    if not os.path.exists(SO_PATH):
        return True
    built = os.path.getmtime(SO_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps)


CHECKED_SO_PATH = os.path.join(HERE, "_df3_sm100_checked.so")


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """Compile if needed and return the path of the shared object. ``checked`` builds the debug variant
    (``-DDF3_BOUNDS_CHECK``: index tests around the kernels' global accesses that record a status code instead of
    touching memory out of range) as ``_df3_sm100_checked.so``; ``DF3_BOUNDS_CHECK=1`` makes ``ops/native.py`` load it."""
    if checked:
        return _build_checked(verbose)
    if not force and not _stale():
        return SO_PATH
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    srcs = sources()
    defines = ["-DDF3_WITH_GEMM"] if any(os.path.basename(s) == "gemm_sm100.cu" for s in srcs) else []
    cpp_extension.load(
        name="_df3_sm100",
        sources=srcs,
        extra_cflags=["-O3", "-std=c++17"] + defines,
        extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xptxas", "-v"] + ARCH_FLAGS + defines,
        build_directory=BUILD_DIR,
        is_python_module=False,
        verbose=verbose,
    )
    built = os.path.join(BUILD_DIR, "_df3_sm100.so")
    shutil.copy2(built, SO_PATH)
    return SO_PATH


def _build_checked(verbose: bool) -> str:
    from torch.utils import cpp_extension

    build_dir = BUILD_DIR + "_checked"
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    defines = ["-DDF3_WITH_GEMM", "-DDF3_BOUNDS_CHECK"]
    cpp_extension.load(
        name="_df3_sm100_checked", sources=sources(), extra_cflags=["-O3", "-std=c++17"] + defines,
        extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "--use_fast_math"] + ARCH_FLAGS + defines,
        build_directory=build_dir, is_python_module=False, verbose=verbose,
    )  # fmt: skip
    shutil.copy2(os.path.join(build_dir, "_df3_sm100_checked.so"), CHECKED_SO_PATH)
    return CHECKED_SO_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv, checked="--checked" in sys.argv)
    print(path)
