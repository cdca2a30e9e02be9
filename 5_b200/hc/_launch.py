"""Launch preparation for compiled kernels: argument binding, symbol binding, geometry checks.

Mirrors what the reference simulator does before it runs a workgroup
(`_prepare_launch`, hc/simulator.py:189-229): bind the call's arguments to the kernel's
parameters minus the leading group (:664-672), derive symbol values from buffer shapes with
conflict detection (`_bind_buffer`, :752-768), evaluate `work_shape` / `group_shape` /
`subgroup_size` (:797-855) and validate them (`_validate_launch`, :858-900). Messages are
the reference's, so a caller sees the same text from the simulator and from the GPU path.
The one extension: a buffer may also be a `hc.cuda.DeviceBuffer`, which stands for an
ndarray of the same shape and dtype that already lives on the GPU.
"""

from __future__ import annotations

import functools
import inspect
from dataclasses import dataclass
from typing import Any

import numpy as np

from ._pipeline import resolved_annotations
from .errors import LaunchError
from .symbols import Bindings, Expr, Symbol, SymbolError

__all__ = ["PreparedLaunch", "prepare_launch"]


@dataclass(frozen=True)
class PreparedLaunch:
    arguments: dict[str, Any]
    symbols: dict[str, int]
    work_shape: tuple[int, ...]
    group_shape: tuple[int, ...]
    subgroup_size: int | None

    @property
    def is_empty(self) -> bool:
        """A zero-sized work shape launches nothing (hc/simulator.py:175-176)."""
        return any(extent == 0 for extent in self.work_shape)

    @property
    def group_counts(self) -> tuple[int, ...]:
        return tuple(-(-w // g) for w, g in zip(self.work_shape, self.group_shape))


def _is_device_buffer(value: Any) -> bool:
    return type(value).__name__ == "DeviceBuffer" and hasattr(value, "ptr")


def _is_symbol(dim: Any) -> bool:
    return isinstance(dim, Symbol) or (
        isinstance(getattr(dim, "name", None), str) and hasattr(dim, "free_symbols")
        and getattr(dim, "op", "sym") == "sym")


class _ForeignBindings:
    """Binding store for symbols of another `hc` package (keyed by name)."""

    def __init__(self) -> None:
        self.values: dict[str, int] = {}
        self.sources: dict[str, str | None] = {}

    def bind(self, name: str, value: int, source: str | None) -> None:
        known = self.values.get(name)
        if known is not None and known != value:
            raise LaunchError(
                f"conflicting binding for {name}: {known} from {self.sources.get(name)!r} vs "
                f"{value} from {source!r}")
        self.values[name] = value
        self.sources[name] = source


def _bind_dimension(store: _ForeignBindings, dim: Any, value: int, source: str) -> None:
    if isinstance(dim, bool):
        return
    if isinstance(dim, int):
        if dim != value:
            raise LaunchError(f"{source} expected {dim}, got {value}")
        return
    if _is_symbol(dim):
        store.bind(dim.name, value, source)
        return
    evaluate = getattr(dim, "eval", None)
    if evaluate is not None:
        try:
            actual = int(evaluate(dict(store.values)))
        except Exception as exc:  # unbound symbols, non-integer value
            raise LaunchError(str(exc)) from exc
        if actual != value:
            raise LaunchError(f"requirement failed at {source!r}: expected {dim} == {value}, got {actual}")


def _bind_buffer(store: _ForeignBindings, spec: Any, value: Any, source: str) -> None:
    if not isinstance(value, np.ndarray) and not _is_device_buffer(value):
        raise LaunchError(f"{source} must be a numpy.ndarray buffer")
    if value.ndim != len(spec.dimensions):
        raise LaunchError(f"{source} rank does not match its Buffer annotation")
    if spec.dtype is not None:
        expected = np.dtype(spec.dtype)
        if value.dtype != expected:
            raise LaunchError(f"{source} dtype expected {expected.name}, got {value.dtype.name}")
    for index, dim in enumerate(spec.dimensions):
        _bind_dimension(store, dim, int(value.shape[index]), f"{source}.shape[{index}]")


def _resolve_dim(value: Any, names: dict[str, int], what: str) -> int:
    if isinstance(value, bool):
        raise LaunchError(f"{what} must be an integer")
    if isinstance(value, (int, np.integer)):
        return int(value)
    evaluate = getattr(value, "eval", None)
    if evaluate is None:
        raise LaunchError(f"{what} must be an integer expression")
    try:
        return int(evaluate(names))
    except SymbolError as exc:
        raise LaunchError(str(exc)) from exc
    except Exception as exc:  # a foreign symbol engine's own error types
        raise LaunchError(str(exc)) from exc


def _resolve_shape(spec: Any, names: dict[str, int], what: str) -> tuple[int, ...]:
    values = spec if isinstance(spec, tuple) else (spec,)
    return tuple(_resolve_dim(v, names, what) for v in values)


@functools.lru_cache(maxsize=256)
def _launch_signature(kernel_fn: Any) -> tuple[inspect.Signature | None, dict[str, Any]]:
    """Signature without the group parameter, and resolved annotations; fixed per kernel."""
    params = list(inspect.signature(kernel_fn).parameters.values())
    if not params:
        return None, {}
    return inspect.Signature(params[1:]), resolved_annotations(kernel_fn)


def prepare_launch(kernel_fn: Any, args: tuple[Any, ...], kwargs: dict[str, Any],
                   literal_bindings: dict[str, int] | None = None) -> PreparedLaunch:
    """Binds a call to `kernel_fn` (without the group parameter) and checks its geometry."""
    meta = getattr(kernel_fn, "__hc_kernel__", None)
    if meta is None:
        raise LaunchError("launch() expects a function decorated with @kernel")
    signature, annotations = _launch_signature(kernel_fn)
    if signature is None:
        raise LaunchError("kernel must accept a CurrentGroup parameter")
    try:
        bound = signature.bind(*args, **kwargs)
    except TypeError as exc:
        raise LaunchError(str(exc)) from exc

    store = _ForeignBindings()
    for name, value in (literal_bindings or {}).items():
        store.bind(name, int(value), "hc.compile(symbols=...)")
    for name, value in bound.arguments.items():
        spec = annotations.get(name)
        if type(spec).__name__ == "BufferSpec":
            _bind_buffer(store, spec, value, name)

    names = dict(store.values)
    if meta.work_shape is None:
        raise LaunchError("kernel metadata is missing required work_shape")
    work_shape = _resolve_shape(meta.work_shape, names, "shape")
    subgroup = None if meta.subgroup_size is None else _resolve_dim(meta.subgroup_size, names, "subgroup_size")
    if meta.group_shape is None:
        group_shape = tuple(max(1, w) for w in work_shape)
    else:
        group_shape = _resolve_shape(meta.group_shape, names, "shape")

    if len(work_shape) != len(group_shape):
        raise LaunchError("work_shape and group_shape must have the same rank")
    if any(w < 0 for w in work_shape):
        raise LaunchError("work_shape values must be non-negative")
    if any(g <= 0 for g in group_shape):
        raise LaunchError("group_shape values must be positive")
    if subgroup is not None:
        if subgroup <= 0:
            raise LaunchError("subgroup_size must be positive")
        if group_shape and group_shape[0] % subgroup != 0:
            raise LaunchError("group_shape[0] must be divisible by subgroup_size")
    return PreparedLaunch(dict(bound.arguments), names, work_shape, group_shape, subgroup)


# `Bindings` / `Expr` are re-exported for callers that build launch environments by hand.
_ = (Bindings, Expr)
