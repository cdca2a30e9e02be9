"""Kernel-definition surface of hc, as far as the tiled-matmul path uses it.

This is a from-scratch mirror of the decorator/metadata layer of the reference
(hc/core.py): `@kernel`, `@kernel.func`, `@kernel.intrinsic` (+ `.lower/.verify/.infer`
hooks), `Buffer[...]`, the scopes and the type-spec constructors. Like there, decorating only
records metadata on the function object; nothing is executed or compiled at decoration time.

The attribute names and dataclass field names are the drop-in contract: the NVIDIA target
(`hc._pipeline`) reads `__hc_kernel__`, `__hc_func__`, `__hc_intrinsic__`,
`__hc_lowerings__` and the `Buffer` annotations by duck typing, so a kernel decorated with the
reference's own `hc` package is accepted unchanged.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from collections.abc import Callable, Sequence
from dataclasses import dataclass, field
from typing import Any

__all__ = [
    "Buffer",
    "BufferSpec",
    "CurrentGroup",
    "FuncMetadata",
    "IdxTypeSpec",
    "IndexMap",
    "IntrinsicMetadata",
    "KernelMetadata",
    "Result",
    "Scope",
    "SubGroup",
    "TensorTypeSpec",
    "UndefTypeSpec",
    "VectorTypeSpec",
    "WorkGroup",
    "WorkItem",
    "as_layout",
    "idx_type",
    "index_map",
    "kernel",
    "tensor_type",
    "undef_type",
    "vector_type",
]


def _dtype_name(value: Any) -> str:
    """NumPy spelling of a dtype ("float16", "bfloat16", "float32", ...); hc/core.py:89-92."""
    import numpy as np

    return str(np.dtype(value).name)


def _looks_like_dtype(value: Any) -> bool:
    import numpy as np

    return isinstance(value, np.dtype) or (isinstance(value, type) and issubclass(value, np.generic))


# ------------------------------------------------------------------ type specs ----------


@dataclass(frozen=True)
class BufferSpec:
    """`Buffer[M, K, np.float16]`: symbolic extents plus an optional element type."""

    dimensions: tuple[Any, ...]
    dtype: str | None = None

    def __repr__(self) -> str:
        items = [str(d) for d in self.dimensions]
        if self.dtype is not None:
            items.append(self.dtype)
        return "Buffer[" + ", ".join(items) + "]"


class Buffer:
    """Annotation factory: `Buffer[dims..., dtype]` -> BufferSpec (hc/core.py:68-76).

    A trailing NumPy dtype (or scalar type, including ml_dtypes.bfloat16) is taken as the
    element type, but only when at least one extent precedes it.
    """

    def __class_getitem__(cls, item: Any) -> BufferSpec:
        items = item if isinstance(item, tuple) else (item,)
        if len(items) >= 2 and _looks_like_dtype(items[-1]):
            return BufferSpec(tuple(items[:-1]), _dtype_name(items[-1]))
        return BufferSpec(tuple(items), None)


@dataclass(frozen=True)
class TensorTypeSpec:
    dimensions: tuple[Any, ...]
    dtype: str


@dataclass(frozen=True)
class VectorTypeSpec:
    dimensions: tuple[Any, ...]
    dtype: str


@dataclass(frozen=True)
class IdxTypeSpec:
    expr: Any = None


@dataclass(frozen=True)
class UndefTypeSpec:
    pass


def tensor_type(shape: Sequence[Any], dtype: Any) -> TensorTypeSpec:
    return TensorTypeSpec(tuple(shape), _dtype_name(dtype))


def vector_type(shape: Sequence[Any], dtype: Any) -> VectorTypeSpec:
    return VectorTypeSpec(tuple(shape), _dtype_name(dtype))


def idx_type(expr: Any = None) -> IdxTypeSpec:
    return IdxTypeSpec(expr)


def undef_type() -> UndefTypeSpec:
    return UndefTypeSpec()


@dataclass(frozen=True)
class Result:
    type: Any
    mask: Any = None
    layout: Any = None


@dataclass(frozen=True)
class IndexMap:
    params: Callable[..., Any] | None
    storage_size: Callable[..., Any]
    offset: Callable[..., Any]


def index_map(*, params: Callable[..., Any] | None = None, storage_size: Callable[..., Any],
              offset: Callable[..., Any]) -> IndexMap:
    return IndexMap(params, storage_size, offset)


def as_layout(value: Any, layout: Any = None) -> Any:
    hook = getattr(value, "as_layout", None)
    if hook is None:
        raise TypeError("as_layout() expects a layout-aware value")
    return hook(layout)


# ------------------------------------------------------------------ scopes --------------


@dataclass(frozen=True)
class Scope:
    name: str

    def __str__(self) -> str:
        return self.name

    __repr__ = __str__


WorkGroup = Scope("WorkGroup")


def _backend_only(what: str) -> NotImplementedError:
    return NotImplementedError(f"{what} is implemented by runtime backends")


class CurrentGroup:
    """Static stand-in for the group handle a kernel body receives (hc/core.py:395-453)."""

    def __init__(self, *, group_id: tuple[int, ...] = (), shape: tuple[int, ...] = (),
                 work_shape: tuple[int, ...] = (), work_offset: tuple[int, ...] = ()) -> None:
        self.group_id = group_id
        self.shape = shape
        self.work_shape = work_shape
        self.work_offset = work_offset

    @property
    def size(self) -> int:
        total = 1
        for extent in self.shape:
            total *= extent
        return total

    def subgroups(self, fn: Callable[..., Any]) -> Callable[..., Any]:
        return fn

    def workitems(self, fn: Callable[..., Any]) -> Callable[..., Any]:
        return fn

    def barrier(self) -> None:
        raise _backend_only("barrier")


def _make_group_stub(name: str) -> Callable[..., Any]:
    def stub(self: Any, *args: Any, **kwargs: Any) -> Any:
        raise _backend_only(name)

    stub.__name__ = name
    return stub


for _name in ("load", "vload", "store", "empty", "zeros", "ones", "full", "vzeros", "vones", "vfull"):
    setattr(CurrentGroup, _name, _make_group_stub(_name))
del _name


class SubGroup:
    def subgroup_id(self) -> int:
        raise _backend_only("subgroup_id")

    def size(self) -> int:
        raise _backend_only("size")


class WorkItem:
    def global_id(self) -> tuple[int, ...]:
        raise _backend_only("global_id")

    def local_id(self) -> tuple[int, ...]:
        raise _backend_only("local_id")


# ------------------------------------------------------------------ metadata ------------


@dataclass(frozen=True)
class KernelMetadata:
    work_shape: Any = None
    group_shape: Any = None
    subgroup_size: Any = None
    literals: frozenset[Any] = field(default_factory=frozenset)


@dataclass(frozen=True)
class FuncMetadata:
    scope: Any = None


@dataclass(frozen=True)
class IntrinsicMetadata:
    scope: Any = None
    effects: Any = None
    const_attrs: frozenset[str] = field(default_factory=frozenset)
    operand_types: tuple[Any, ...] | None = None
    result_types: tuple[Any, ...] = ()


def _has_fallback_body(fn: Callable[..., Any]) -> bool:
    """True when the intrinsic's Python body does something (a simulator fallback).

    A body that is empty, `pass`, `...` or only a docstring declares a device-only intrinsic
    (hc/core.py:211-259). When the source cannot be read the body is assumed to be real.
    """
    try:
        tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    except (OSError, TypeError, SyntaxError):
        return True
    if not tree.body or not isinstance(tree.body[0], (ast.FunctionDef, ast.AsyncFunctionDef)):
        return True
    for stmt in tree.body[0].body:
        if isinstance(stmt, ast.Pass):
            continue
        if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant) and (
            stmt.value.value is Ellipsis or isinstance(stmt.value.value, str)
        ):
            continue
        return True
    return False


def _install_intrinsic_hooks(fn: Any) -> None:
    """`.lower(target=...)`, `.verify`, `.infer` registration decorators (hc/core.py:282-307)."""
    fn.__hc_lowerings__ = {}
    fn.__hc_verify__ = None
    fn.__hc_infer__ = None
    fn.__hc_has_fallback__ = _has_fallback_body(fn)

    def lower(*, target: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def register(callback: Callable[..., Any]) -> Callable[..., Any]:
            fn.__hc_lowerings__[target] = callback
            return callback

        return register

    def verify(callback: Callable[..., Any]) -> Callable[..., Any]:
        fn.__hc_verify__ = callback
        return callback

    def infer(callback: Callable[..., Any]) -> Callable[..., Any]:
        fn.__hc_infer__ = callback
        return callback

    fn.lower = lower
    fn.verify = verify
    fn.infer = infer


def _apply(fn: Callable[..., Any] | None, decorate: Callable[[Any], Any]) -> Any:
    """Supports both `@decorator` and `@decorator(...)` spellings."""
    return decorate if fn is None else decorate(fn)


class _KernelNamespace:
    """The `kernel` object: callable decorator with `.func` and `.intrinsic` members."""

    def __call__(self, fn: Callable[..., Any] | None = None, *, work_shape: Any = None,
                 group_shape: Any = None, subgroup_size: Any = None,
                 literals: set[Any] | frozenset[Any] | None = None) -> Any:
        meta = KernelMetadata(work_shape, group_shape, subgroup_size,
                              frozenset(literals) if literals is not None else frozenset())

        def decorate(target: Any) -> Any:
            target.__hc_kernel__ = meta
            return target

        return _apply(fn, decorate)

    def func(self, fn: Callable[..., Any] | None = None, *, scope: Any = None) -> Any:
        meta = FuncMetadata(scope)

        def decorate(target: Any) -> Any:
            target.__hc_func__ = meta
            return target

        return _apply(fn, decorate)

    def intrinsic(self, fn: Callable[..., Any] | None = None, *, scope: Any = None,
                  effects: Any = None, const_attrs: set[str] | frozenset[str] | None = None,
                  operand_types: Sequence[Any] | None = None,
                  result_types: Sequence[Any] | Any = ()) -> Any:
        if result_types is None:
            results: tuple[Any, ...] = ()
        elif isinstance(result_types, Sequence) and not isinstance(result_types, (str, bytes)):
            results = tuple(result_types)
        else:
            results = (result_types,)
        meta = IntrinsicMetadata(
            scope=scope,
            effects=effects,
            const_attrs=frozenset(const_attrs) if const_attrs is not None else frozenset(),
            operand_types=tuple(operand_types) if operand_types is not None else None,
            result_types=results,
        )

        def decorate(target: Any) -> Any:
            target.__hc_intrinsic__ = meta
            _install_intrinsic_hooks(target)
            return target

        return _apply(fn, decorate)


kernel = _KernelNamespace()
