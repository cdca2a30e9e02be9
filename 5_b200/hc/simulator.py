"""`hc.simulator.launch` -- the reference's launch entry point, served by the B200 backend.

In the reference this module is the NumPy/greenlet host simulator and `launch(fn, *args)` is the
only way a kernel ever executes (hc/simulator.py:165-186; the example calls it as
`sim.launch(tiled_gfx11_wmma_matmul, a, b, c)`, examples/amdgpu_gfx11_wmma_matmul.py:338-348).
Here the same call runs the kernel on the GPU: the function is compiled once for the
`"nvidia-sm100a"` target (`hc.compile`) and the handle is called with the arguments, so code written
against the reference -- its example module included -- runs unchanged with this package first on
the import path. Same contract: arguments are bound and checked with the simulator's rules and
`LaunchError` messages (`hc._launch`), buffers are updated in place, the call returns None when the
result is complete, a zero-sized work shape launches nothing.

There is no simulator behind it and no CPU fallback: a kernel the target does not recognise raises
`NotImplementedError` with the recogniser's diagnostics, and a missing CUDA library or device
raises from `hc.cuda`.
"""

from __future__ import annotations

import threading
from typing import Any, Callable

from ._compile import CompiledKernel, compile as _compile
from ._pipeline import NVIDIA_SM100A
from .errors import LaunchError, SimulatorError

__all__ = ["LaunchError", "SimulatorError", "compiled", "launch", "run"]

_HANDLES: dict[int, tuple[Any, CompiledKernel]] = {}
_LOCK = threading.Lock()


def compiled(fn: Callable[..., Any]) -> CompiledKernel:
    """The handle `launch` uses for `fn` (compiled on first use, kept for the life of `fn`)."""
    if getattr(fn, "__hc_kernel__", None) is None:
        raise LaunchError("launch() expects a function decorated with @kernel")
    with _LOCK:
        entry = _HANDLES.get(id(fn))
        if entry is None or entry[0] is not fn:
            entry = (fn, _compile(fn, target=NVIDIA_SM100A))
            _HANDLES[id(fn)] = entry
        return entry[1]


def launch(fn: Callable[..., Any], *args: Any, target: Any = None, **kwargs: Any) -> None:
    """Runs `fn(group, *args, **kwargs)` for every workgroup of its launch geometry -- on the GPU.

    `target=` is the reference's simulator-target argument (group-size limits of the host
    simulator, hc/simulator.py:61-80); it has no meaning here and must be left at None."""
    if target is not None:
        raise LaunchError("hc.simulator.launch on the nvidia-sm100a backend takes no simulator target")
    compiled(fn)(*args, **kwargs)


run = launch
