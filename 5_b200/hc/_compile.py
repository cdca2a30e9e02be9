"""`hc.compile`: turn a `@kernel` function into a handle, and -- new here -- launch it.

Signature, argument checks and the handle's fields follow the reference
(hc/_compile.py:41-150): `compile(kernel_fn, symbols=None, *, schedule=None)` returns a
frozen `CompiledKernel` carrying the kernel, the normalised literal bindings and the IR
fields. Two things differ:

  * `target=` selects a backend. With `target="nvidia-sm100a"` the handle's `__call__`
    runs the kernel on a B200 through include/hc-c/Cuda.h instead of raising
    `NotImplementedError` (hc/_compile.py:57-62). The call takes the kernel's arguments
    without the group (doc/langref.md:133-142), writes C in place and returns None once
    the result is complete, like `hc.simulator.launch` (hc/simulator.py:165-186).
  * The MLIR front half is not part of this package: `front_ir`/`hc_ir` stay None and
    `pipeline_diagnostics` says so, the same non-fatal convention the reference uses when
    its pipeline fails (hc/_pipeline.py:100-108). `schedule=` is accepted and recorded.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from ._launch import PreparedLaunch, prepare_launch
from ._map_kernels import MapContract
from ._pairwise_kernels import PairwiseContract
from ._reduce_kernels import RowSumContract
from ._pipeline import GemmContract, ScheduleSource, lower_for_target
from .errors import LaunchError

__all__ = ["CompiledKernel", "ScheduleSource", "compile"]

_NO_MLIR = ("hc_front / hc MLIR is not produced by this package: the MLIR front half of hc is "
            "outside the B200 launch path")


@dataclass(frozen=True)
class CompiledKernel:
    """Handle returned by `hc.compile`."""

    kernel: Any
    bindings: Mapping[str, int]
    front_ir: Any = None
    front_ir_text: str | None = None
    front_ir_symbols: tuple[str, ...] = field(default=())
    hc_ir: Any | None = field(default=None)
    hc_ir_text: str | None = field(default=None)
    pipeline_diagnostics: tuple[str, ...] = field(default=())
    # Extensions of the NVIDIA path.
    target: str | None = field(default=None)
    plan: GemmContract | MapContract | PairwiseContract | None = field(default=None)
    schedule: ScheduleSource = field(default=None)
    device: int | None = field(default=None)

    # -- launch -------------------------------------------------------------------------
    def __call__(self, *args: Any, **kwargs: Any) -> None:
        if self.target is None:
            raise NotImplementedError(
                "this handle was compiled without a target; pass target='nvidia-sm100a' to "
                "hc.compile to get a launchable kernel")
        if self.plan is None:
            reasons = "; ".join(self.pipeline_diagnostics) or "kernel not recognised"
            raise NotImplementedError(
                f"target {self.target!r} cannot launch {self._name()}: {reasons}")
        launch = prepare_launch(self.kernel, args, kwargs, dict(self.bindings))
        if launch.is_empty:
            return None
        if isinstance(self.plan, MapContract):
            self._launch_map(launch)
        elif isinstance(self.plan, PairwiseContract):
            self._launch_pairwise(launch)
        elif isinstance(self.plan, RowSumContract):
            self._launch_row_sum(launch)
        else:
            self._launch_gemm(launch)
        return None

    def prepare(self, *args: Any, **kwargs: Any) -> PreparedLaunch:
        """Binding and geometry of a call, without launching (symbols, work/group shape)."""
        return prepare_launch(self.kernel, args, kwargs, dict(self.bindings))

    def _launch_gemm(self, launch: PreparedLaunch) -> None:
        from . import cuda  # imported on first launch so that compile() needs no CUDA library

        plan = self.plan
        assert plan is not None
        a, b, c = (launch.arguments[p] for p in (plan.a_param, plan.b_param, plan.c_param))
        variant = {"auto": cuda.VARIANT_AUTO, "dense": cuda.VARIANT_DENSE, "skinny": cuda.VARIANT_SKINNY,
                   "tiny": cuda.VARIANT_TINY}[
            (plan.lowering or {}).get("variant", "auto")]
        bias = launch.arguments[plan.bias_param] if plan.bias_param is not None else None
        buffers = (a, b, c) if bias is None else (a, b, c, bias)
        on_device = [type(x).__name__ == "DeviceBuffer" for x in buffers]
        if any(on_device) and not all(on_device):
            raise LaunchError("buffers must be all numpy.ndarray or all DeviceBuffer")
        options = dict(variant=variant, b_transposed=plan.b_transposed, accumulate=plan.accumulate,
                       epilogue=plan.epilogue)
        if all(on_device):
            ctx = a.ctx
            if any(x.ctx is not ctx for x in buffers):
                raise LaunchError("device buffers must belong to one context")
            ctx.gemm(a, b, c, bias=bias, **options)
            ctx.synchronize()
            return
        ctx = cuda.default_context(self.device)
        a_host = _row_major(a)
        b_host = _row_major(b)
        bias_host = None if bias is None else np.ascontiguousarray(bias)
        if _is_row_major(c) and c.flags.writeable:
            ctx.gemm_host(a_host, b_host, c, bias=bias_host, **options)
            return
        if not c.flags.writeable:
            raise LaunchError(f"{plan.c_param} must be writeable")
        # C's previous contents start the sums of an accumulating kernel.
        staged = np.array(c, order="C") if plan.accumulate else np.empty(c.shape, c.dtype)
        ctx.gemm_host(a_host, b_host, staged, bias=bias_host, **options)
        c[...] = staged

    def _launch_map(self, launch: PreparedLaunch) -> None:
        """out[i] = ops(x[i] [, y[i]]) for a recognised element-wise kernel."""
        from . import cuda

        plan = self.plan
        assert isinstance(plan, MapContract)
        names = [plan.x_param] + ([plan.other_param] if plan.other_param else []) + [plan.out_param]
        buffers = [launch.arguments[name] for name in names]
        for name, buf in zip(names, buffers):
            if buf.dtype != np.float32:
                raise LaunchError(f"{name} dtype expected float32, got {buf.dtype.name}: target {self.target!r} runs "
                                  f"element-wise kernels on float32 buffers")
        x, out = buffers[0], buffers[-1]
        other = buffers[1] if plan.other_param else None
        on_device = [type(buf).__name__ == "DeviceBuffer" for buf in buffers]
        if any(on_device) and not all(on_device):
            raise LaunchError("buffers must be all numpy.ndarray or all DeviceBuffer")
        if all(on_device):
            ctx = x.ctx
            if any(buf.ctx is not ctx for buf in buffers):
                raise LaunchError("device buffers must belong to one context")
            if plan.rank == 2:
                # The function is element-wise, so a matrix is its elements in row-major order.
                for name, buf in zip(names, buffers):
                    if buf.ld != buf.shape[1]:
                        raise LaunchError(f"{name}: a two-dimensional element-wise kernel needs device matrices "
                                          f"without row padding (pitch {buf.ld} for {buf.shape[1]} columns)")
                flat = [type(buf).wrap(ctx, buf.ptr, (buf.shape[0] * buf.shape[1],), buf.dtype) for buf in buffers]
                x, out = flat[0], flat[-1]
                other = flat[1] if plan.other_param else None
            ctx.map(x, out, plan.ops, other=other)
            ctx.synchronize()
            return
        if not out.flags.writeable:
            raise LaunchError(f"{plan.out_param} must be writeable")
        ctx = cuda.default_context(self.device)
        # Inputs that are the output array itself (in place) stay that array; everything else that
        # is not contiguous is staged through a contiguous copy.
        direct = out.flags.c_contiguous
        staged = out if direct else np.empty(out.shape, np.float32)

        def host(arr: np.ndarray) -> np.ndarray:
            if arr is out:
                if not direct:
                    staged[...] = out
                return staged.reshape(-1)
            return np.ascontiguousarray(arr).reshape(-1)  # (a matrix goes as its elements in row-major order)

        ctx.map_host(host(x), staged.reshape(-1), plan.ops, other=None if other is None else host(other))
        if not direct:
            out[...] = staged

    def _launch_pairwise(self, launch: PreparedLaunch) -> None:
        """out[i, j] = [sqrt] sum_h (x1[i, h] - x2[j, h])^2 for a recognised pairwise kernel."""
        from . import cuda

        plan = self.plan
        assert isinstance(plan, PairwiseContract)
        names = [plan.lhs_param, plan.rhs_param, plan.out_param]
        x1, x2, out = (launch.arguments[name] for name in names)
        for name, buf in zip(names, (x1, x2, out)):
            if buf.dtype != np.float32:
                raise LaunchError(f"{name} dtype expected float32, got {buf.dtype.name}: target {self.target!r} runs "
                                  f"pairwise kernels on float32 buffers")
        on_device = [type(buf).__name__ == "DeviceBuffer" for buf in (x1, x2, out)]
        if any(on_device) and not all(on_device):
            raise LaunchError("buffers must be all numpy.ndarray or all DeviceBuffer")
        if all(on_device):
            ctx = x1.ctx
            if x2.ctx is not ctx or out.ctx is not ctx:
                raise LaunchError("device buffers must belong to one context")
            ctx.pairwise(x1, x2, out, take_sqrt=plan.take_sqrt)
            ctx.synchronize()
            return
        if not out.flags.writeable:
            raise LaunchError(f"{plan.out_param} must be writeable")
        ctx = cuda.default_context(self.device)
        direct = _is_row_major(out)
        # (Only the w1 x w2 results are written, so a staged copy starts from out's contents when h == 0.)
        staged = out if direct else np.array(out, order="C")
        ctx.pairwise_host(_row_major(x1), _row_major(x2), staged, take_sqrt=plan.take_sqrt)
        if not direct:
            out[...] = staged

    def _launch_row_sum(self, launch: PreparedLaunch) -> None:
        """out[i] = [sqrt] sum_h x[i, h] [squared] for a recognised row-sum kernel."""
        from . import cuda

        plan = self.plan
        assert isinstance(plan, RowSumContract)
        names = [plan.in_param, plan.out_param]
        x, out = (launch.arguments[name] for name in names)
        for name, buf in zip(names, (x, out)):
            if buf.dtype != np.float32:
                raise LaunchError(f"{name} dtype expected float32, got {buf.dtype.name}: target {self.target!r} runs "
                                  f"row sums on float32 buffers")
        on_device = [type(buf).__name__ == "DeviceBuffer" for buf in (x, out)]
        if any(on_device) and not all(on_device):
            raise LaunchError("buffers must be all numpy.ndarray or all DeviceBuffer")
        if all(on_device):
            ctx = x.ctx
            if out.ctx is not ctx:
                raise LaunchError("device buffers must belong to one context")
            ctx.row_sum(x, out, square=plan.square, take_sqrt=plan.take_sqrt)
            ctx.synchronize()
            return
        if not out.flags.writeable:
            raise LaunchError(f"{plan.out_param} must be writeable")
        ctx = cuda.default_context(self.device)
        direct = out.ndim == 1 and (out.shape[0] <= 1 or out.strides[0] == out.itemsize)
        # (Only the w results are written, so a staged copy starts from out's contents when h == 0.)
        staged = out if direct else np.array(out, order="C")
        ctx.row_sum_host(_row_major(x), staged, square=plan.square, take_sqrt=plan.take_sqrt)
        if not direct:
            out[...] = staged

    # -- text ---------------------------------------------------------------------------
    def _name(self) -> str:
        return getattr(self.kernel, "__name__", "<kernel>")

    def __repr__(self) -> str:
        joined = ", ".join(f"{k}={v}" for k, v in sorted(self.bindings.items()))
        if self.target is not None:
            stage = self.target if self.plan is not None else f"{self.target}:unsupported"
        else:
            stage = "hc" if self.hc_ir_text is not None else "hc_front"
        return f"CompiledKernel({self._name()}, {{{joined}}}, stage={stage})"


def _is_row_major(x: np.ndarray) -> bool:
    """Rows contiguous, row pitch a whole non-negative number of elements."""
    if x.ndim != 2:
        return False
    if x.shape[0] == 0 or x.shape[1] == 0:
        return True
    item = x.itemsize
    inner_ok = x.shape[1] == 1 or x.strides[1] == item
    outer_ok = x.shape[0] == 1 or (x.strides[0] % item == 0 and x.strides[0] >= x.shape[1] * item)
    return inner_ok and outer_ok


def _row_major(x: np.ndarray) -> np.ndarray:
    return x if _is_row_major(x) else np.ascontiguousarray(x)


def compile(  # noqa: A001 - public name fixed by the reference API
    kernel_fn: Any,
    symbols: Mapping[Any, int] | None = None,
    *,
    schedule: ScheduleSource = None,
    target: str | None = None,
    device: int | None = None,
) -> CompiledKernel:
    """Compile a `@kernel` function.

    `symbols` binds literal symbols (keys: `Symbol` or `str`; values: `int`). Keys must be in
    the kernel's `literals=` set when it declared one. With `target="nvidia-sm100a"` the
    returned handle is callable; bound symbols are checked against the buffer shapes of
    every call. `device` picks the GPU for NumPy-buffer launches (default `$HC_CUDA_DEVICE`
    or 0).
    """
    metadata = getattr(kernel_fn, "__hc_kernel__", None)
    if metadata is None or not hasattr(metadata, "work_shape"):
        raise TypeError(f"hc.compile expects a @kernel-decorated function, got {kernel_fn!r}")
    if symbols is None:
        symbols = {}
    elif not isinstance(symbols, Mapping):
        raise TypeError(f"symbols must be a Mapping, got {type(symbols).__name__}")
    bindings = normalise_bindings(symbols, metadata)

    diagnostics = [_NO_MLIR]
    plan = None
    if target is not None:
        result = lower_for_target(kernel_fn, target)
        plan = result.plan
        diagnostics.extend(result.diagnostics)
    return CompiledKernel(
        kernel=kernel_fn,
        bindings=bindings,
        pipeline_diagnostics=tuple(diagnostics),
        target=target,
        plan=plan,
        schedule=schedule,
        device=device,
    )


def symbol_name(obj: Any) -> str:
    if isinstance(obj, str):
        return obj
    name = getattr(obj, "name", None)
    if isinstance(name, str) and hasattr(obj, "free_symbols"):
        return name
    raise TypeError(f"cannot interpret {obj!r} as a symbol name")


def normalise_bindings(symbols: Mapping[Any, int], metadata: Any) -> dict[str, int]:
    """`symbols=` -> {name: int}; same rules and messages as hc/_compile.py:153-181."""
    allowed = {symbol_name(s) for s in metadata.literals}
    out: dict[str, int] = {}
    for key, value in symbols.items():
        name = symbol_name(key)
        if allowed and name not in allowed:
            raise ValueError(
                f"'{name}' is not a declared literal symbol; kernel declares {sorted(allowed)}")
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError(
                f"literal symbol '{name}' must bind to an int, got {type(value).__name__}")
        if name in out and out[name] != value:
            raise ValueError(
                f"literal symbol '{name}' bound twice with conflicting values "
                f"({out[name]!r} and {value!r})")
        out[name] = value
    return out
