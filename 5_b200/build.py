"""Builds lib/libhc_cuda.so: the sm_100a kernels plus the C ABI of include/hc-c/Cuda.h.

Usage:  python 5_b200/build.py [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU. The CUDA runtime is linked statically and the
driver library is never linked (the one driver entry point needed is fetched at run time), so
the result loads on a machine that has no GPU driver; NCCL is opened at run time only when
the multi-GPU entry points are used.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
LIB_DIR = PACKAGE_DIR / "lib"
BUILD_DIR = LIB_DIR / "build"
OUTPUT = LIB_DIR / "libhc_cuda.so"
CHECKED_OUTPUT = LIB_DIR / "libhc_cuda_checked.so"

SOURCES = [
    LIB_DIR / "Kernels" / "gemm_dense_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_dense_pair_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_dense_wide_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_dense_cluster_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_skinny_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_tiny_sm100a.cu",
    LIB_DIR / "Kernels" / "repack_sm100a.cu",
    LIB_DIR / "Kernels" / "repack_bytes_sm100a.cu",
    LIB_DIR / "Kernels" / "epilogue_only_sm100a.cu",
    LIB_DIR / "Kernels" / "map_elementwise_sm100a.cu",
    LIB_DIR / "Kernels" / "pairwise_distance_sm100a.cu",
    LIB_DIR / "Kernels" / "row_reduce_sm100a.cu",
    LIB_DIR / "Kernels" / "gemm_skinny_static_sm100a.cu",
    LIB_DIR / "Kernels" / "selftest_sm100a.cu",
    LIB_DIR / "CAPI" / "Cuda.cpp",
]
HEADERS = [
    LIB_DIR / "Kernels" / "gemm_launch.h",
    LIB_DIR / "Kernels" / "sm100_ptx.cuh",
    LIB_DIR / "Kernels" / "gemm_epilogue.cuh",
    LIB_DIR / "Kernels" / "device_checks.cuh",
    REPO_ROOT / "include" / "hc-c" / "Cuda.h",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden,-Wall",
    f"-I{REPO_ROOT / 'include'}",
]


# The pairwise kernel reproduces NumPy's float32 results bit for bit: no multiply may be contracted
# with an addition anywhere in that file. (The flag alone does not stop ptxas from fusing a packed
# float32x2 multiply with the add it feeds; the kernel writes its squares in a form that cannot be.)
EXTRA_FLAGS = {"pairwise_distance_sm100a.cu": ["-fmad=false"]}


def find_nvcc() -> str:
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return nvcc


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def build(*, force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compiles what is out of date and returns the path of the shared library. `checked`: the
    variant with index checks inside the kernels (-DHC_CUDA_CHECKED, lib/libhc_cuda_checked.so)."""
    from concurrent.futures import ThreadPoolExecutor

    nvcc = find_nvcc()
    build_dir = BUILD_DIR.with_name(BUILD_DIR.name + "_checked") if checked else BUILD_DIR
    output = CHECKED_OUTPUT if checked else OUTPUT
    flags = [*NVCC_FLAGS, "-DHC_CUDA_CHECKED=1"] if checked else NVCC_FLAGS
    build_dir.mkdir(parents=True, exist_ok=True)
    objects, commands = [], []
    for src in SOURCES:
        obj = build_dir / (src.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, [src, *HEADERS, Path(__file__)]):
            cmd = [nvcc, *flags, *EXTRA_FLAGS.get(src.name, []), "-x", "cu", "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            commands.append(cmd)
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        for done in pool.map(lambda cmd: subprocess.run(cmd, check=True), commands):
            del done
    if force or _stale(output, objects):
        cmd = [nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", str(output), *map(str, objects), "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return output


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--force", action="store_true", help="rebuild everything")
    parser.add_argument("--verbose", action="store_true", help="print commands and ptxas resource use")
    parser.add_argument("--checked", action="store_true",
                        help="build libhc_cuda_checked.so (index checks inside the kernels) instead")
    args = parser.parse_args(argv)
    print(build(force=args.force, verbose=args.verbose, checked=args.checked))
    return 0


if __name__ == "__main__":
    sys.exit(main())
