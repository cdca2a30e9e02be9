"""hc -- the kernel-DSL surface of the tiled-matmul path, with a B200 launch backend.

The public names are those of the reference package (hc/__init__.py:11-63). `hc.compile`
gains `target="nvidia-sm100a"`, which makes the returned handle launch hand-written sm_100a
kernels through the C ABI of include/hc-c/Cuda.h; `hc.cuda` exposes that ABI (contexts,
device buffers, pinned arrays) and `hc.distributed` the N-sharding helpers;
`hc.simulator.launch(fn, *args)`, the reference's launch entry point, runs the kernel on the GPU
through the same handle. `hc.symbols`, `hc.cuda` and the others load lazily, as `symbols` does in
the reference.
"""

from __future__ import annotations

import importlib
from typing import Any

from . import core as _core
from ._compile import CompiledKernel, compile

# The definition surface, re-exported under the names kernels import from `hc`.
for _name in _core.__all__:
    if not _name.endswith("Metadata"):
        globals()[_name] = getattr(_core, _name)
del _name
from .errors import DeviceError, LaunchError, SimulatorError

__all__ = [
    "Buffer", "BufferSpec", "CompiledKernel", "CurrentGroup", "DeviceError", "IdxTypeSpec",
    "IndexMap", "LaunchError", "Result", "Scope", "SimulatorError", "SubGroup", "Symbol",
    "TensorTypeSpec", "UndefTypeSpec", "VectorTypeSpec", "WorkGroup", "WorkItem", "as_layout",
    "compile", "cuda", "distributed", "idx_type", "index_map", "kernel", "simulator", "sym", "symbols",
    "tensor_type", "undef_type", "vector_type",
]

_LAZY_MODULES = {"symbols", "cuda", "distributed", "simulator"}


def __getattr__(name: str) -> Any:
    if name in _LAZY_MODULES:
        return importlib.import_module(f".{name}", __name__)
    if name in ("Symbol", "sym"):
        return getattr(importlib.import_module(".symbols", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted(__all__)
