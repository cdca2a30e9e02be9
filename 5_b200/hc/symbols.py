"""Integer symbols for launch shapes: `sym.M`, `ceil_div(M, 16) * 32`, bindings, evaluation.

The reference wraps a third-party computer-algebra engine here (hc/symbols.py on top of
`ixsimpl`). The matmul path needs none of the algebra -- only to name extents in `Buffer`
annotations, to write a launch shape as an expression of them, to bind them from array
shapes with conflict detection (`Bindings.bind`, hc/symbols.py:408-418) and to evaluate the
shape to integers (`Expr.eval`, hc/symbols.py:226-230). This module provides exactly that
with exact rational arithmetic and no simplifier. Names, exception classes and error texts
follow the reference so that launch errors read the same.
"""

from __future__ import annotations

import math
from collections.abc import Iterator, Mapping
from fractions import Fraction
from typing import Any

__all__ = [
    "Bindings",
    "Env",
    "Expr",
    "NonConstantError",
    "Symbol",
    "SymbolConflictError",
    "SymbolError",
    "UnboundSymbolError",
    "ceil",
    "ceil_div",
    "const",
    "floor",
    "floor_div",
    "max_",
    "min_",
    "mod",
    "sym",
]


class SymbolError(RuntimeError):
    pass


class SymbolConflictError(SymbolError):
    pass


class UnboundSymbolError(SymbolError):
    pass


class NonConstantError(SymbolError):
    pass


class Expr:
    """Immutable expression tree over integer symbols and rational constants."""

    __slots__ = ("_op", "_args", "_free")

    def __init__(self, op: str, args: tuple[Any, ...]) -> None:
        self._op = op
        self._args = args
        self._free: frozenset[Symbol] | None = None  # filled on first use; nodes are immutable

    # -- structure ----------------------------------------------------------------------
    @property
    def op(self) -> str:
        return self._op

    @property
    def children(self) -> tuple["Expr", ...]:
        return tuple(arg for arg in self._args if isinstance(arg, Expr))

    def free_symbols(self) -> frozenset["Symbol"]:
        if self._free is not None:
            return self._free
        found: set[Symbol] = set()
        stack: list[Expr] = [self]
        while stack:
            node = stack.pop()
            if isinstance(node, Symbol):
                found.add(node)
            stack.extend(node.children)
        self._free = frozenset(found)
        return self._free

    def _key(self) -> tuple[Any, ...]:
        return (self._op, tuple(a._key() if isinstance(a, Expr) else a for a in self._args))

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Expr) and self._key() == other._key()

    def __hash__(self) -> int:
        return hash(self._key())

    def __bool__(self) -> bool:
        raise TypeError("symbolic expressions do not define truthiness; use eval()")

    # -- evaluation ---------------------------------------------------------------------
    def _value(self, names: Mapping[str, int]) -> Fraction:
        op, args = self._op, self._args
        if op == "const":
            return args[0]
        if op == "sym":
            return Fraction(names[args[0]])
        vals = [arg._value(names) for arg in args]
        if op == "add":
            return vals[0] + vals[1]
        if op == "mul":
            return vals[0] * vals[1]
        if op == "div":
            if vals[1] == 0:
                raise SymbolError("division by zero in a symbolic expression")
            return vals[0] / vals[1]
        if op == "floor":
            return Fraction(math.floor(vals[0]))
        if op == "ceil":
            return Fraction(math.ceil(vals[0]))
        if op == "mod":
            if vals[1] == 0:
                raise SymbolError("modulo by zero in a symbolic expression")
            return vals[0] - vals[1] * math.floor(vals[0] / vals[1])
        if op == "min":
            return min(vals)
        if op == "max":
            return max(vals)
        raise SymbolError(f"unknown expression node {op!r}")

    def eval(self, env: "Env | Mapping[Any, int]") -> int:
        """Value under `env` (an Env, or a mapping keyed by Symbol or name)."""
        names = _names_of(env)
        missing = sorted(s.name for s in self.free_symbols() if s.name not in names)
        if missing:
            raise UnboundSymbolError(f"missing bindings for symbols: {', '.join(missing)}")
        value = self._value(names)
        if value.denominator != 1:
            raise NonConstantError(f"expression is not an integer: {self} = {value}")
        return int(value)

    eval_int = eval

    def try_eval(self, env: "Env | Mapping[Any, int]") -> int | None:
        try:
            return self.eval(env)
        except SymbolError:
            return None

    def is_constant(self) -> bool:
        return not self.free_symbols()

    # -- arithmetic ---------------------------------------------------------------------
    def __add__(self, other: Any) -> "Expr":
        return Expr("add", (self, _coerce(other)))

    def __radd__(self, other: Any) -> "Expr":
        return Expr("add", (_coerce(other), self))

    def __sub__(self, other: Any) -> "Expr":
        return Expr("add", (self, Expr("mul", (const(-1), _coerce(other)))))

    def __rsub__(self, other: Any) -> "Expr":
        return Expr("add", (_coerce(other), Expr("mul", (const(-1), self))))

    def __mul__(self, other: Any) -> "Expr":
        return Expr("mul", (self, _coerce(other)))

    def __rmul__(self, other: Any) -> "Expr":
        return Expr("mul", (_coerce(other), self))

    def __truediv__(self, other: Any) -> "Expr":
        return Expr("div", (self, _coerce(other)))

    def __rtruediv__(self, other: Any) -> "Expr":
        return Expr("div", (_coerce(other), self))

    def __floordiv__(self, other: Any) -> "Expr":
        return floor_div(self, other)

    def __rfloordiv__(self, other: Any) -> "Expr":
        return floor_div(other, self)

    def __mod__(self, other: Any) -> "Expr":
        return mod(self, other)

    def __neg__(self) -> "Expr":
        return Expr("mul", (const(-1), self))

    # -- text ---------------------------------------------------------------------------
    def __str__(self) -> str:
        op, args = self._op, self._args
        if op == "const":
            return str(args[0])
        if op == "sym":
            return args[0]
        if op in ("add", "mul", "div"):
            sign = {"add": " + ", "mul": "*", "div": "/"}[op]
            return "(" + sign.join(str(a) for a in args) + ")"
        name = {"ceil": "ceiling", "mod": "Mod", "min": "Min", "max": "Max"}.get(op, op)
        return f"{name}({', '.join(str(a) for a in args)})"

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self})"


class Symbol(Expr):
    __slots__ = ()

    def __init__(self, name: str) -> None:
        super().__init__("sym", (name,))

    @property
    def name(self) -> str:
        return self._args[0]


def const(value: int | Fraction) -> Expr:
    return Expr("const", (Fraction(value),))


def _coerce(value: Any) -> Expr:
    if isinstance(value, Expr):
        return value
    if isinstance(value, bool):
        raise TypeError("boolean values are not valid symbolic expressions")
    if isinstance(value, (int, Fraction)):
        return const(value)
    raise TypeError(f"cannot use {type(value).__name__} in a symbolic expression")


def floor(expr: Any) -> Expr:
    return Expr("floor", (_coerce(expr),))


def ceil(expr: Any) -> Expr:
    return Expr("ceil", (_coerce(expr),))


def floor_div(a: Any, b: Any) -> Expr:
    return floor(_coerce(a) / _coerce(b))


def ceil_div(a: Any, b: Any) -> Expr:
    """ceil(a / b), as used for tile counts (hc/symbols.py:499-501)."""
    return ceil(_coerce(a) / _coerce(b))


def mod(a: Any, b: Any) -> Expr:
    return Expr("mod", (_coerce(a), _coerce(b)))


def min_(a: Any, b: Any) -> Expr:
    return Expr("min", (_coerce(a), _coerce(b)))


def max_(a: Any, b: Any) -> Expr:
    return Expr("max", (_coerce(a), _coerce(b)))


class Env(Mapping[Symbol, int]):
    """Frozen symbol -> integer bindings."""

    def __init__(self, bindings: Mapping[Symbol, int] | None = None) -> None:
        self._bindings = dict(bindings or {})

    def __getitem__(self, key: Symbol) -> int:
        return self._bindings[key]

    def __iter__(self) -> Iterator[Symbol]:
        return iter(self._bindings)

    def __len__(self) -> int:
        return len(self._bindings)

    def eval(self, expr: Any) -> int:
        return _coerce(expr).eval(self)

    def names(self) -> dict[str, int]:
        return {symbol.name: value for symbol, value in self._bindings.items()}


def _names_of(env: Env | Mapping[Any, int] | None) -> dict[str, int]:
    if env is None:
        return {}
    if isinstance(env, Env):
        return env.names()
    return {(key.name if isinstance(key, Symbol) else str(key)): int(value) for key, value in env.items()}


class Bindings:
    """Accumulates symbol values and rejects contradictions (hc/symbols.py:402-468)."""

    def __init__(self) -> None:
        self._values: dict[Symbol, int] = {}
        self._sources: dict[Symbol, str | None] = {}

    def bind(self, symbol: Symbol, value: int, *, source: str | None = None) -> None:
        known = self._values.get(symbol)
        if known is not None and known != value:
            raise SymbolConflictError(
                f"conflicting binding for {symbol}: {known} from {self._sources.get(symbol)!r} vs "
                f"{value} from {source!r}"
            )
        self._values[symbol] = value
        self._sources[symbol] = source

    def require(self, expr: Any, value: int, *, source: str | None = None) -> None:
        actual = _coerce(expr).eval(self.freeze())
        if actual != int(value):
            raise SymbolConflictError(
                f"requirement failed at {source!r}: expected {expr} == {value}, got {actual}"
            )

    def get(self, symbol: Symbol) -> int | None:
        return self._values.get(symbol)

    def freeze(self) -> Env:
        return Env(self._values)


class _SymbolNamespace:
    """`sym.M` / `sym["M"]`: interned symbols."""

    def __init__(self) -> None:
        self._cache: dict[str, Symbol] = {}

    def __getitem__(self, name: str) -> Symbol:
        symbol = self._cache.get(name)
        if symbol is None:
            symbol = self._cache[name] = Symbol(name)
        return symbol

    def __getattr__(self, name: str) -> Symbol:
        if name.startswith("_"):
            raise AttributeError(name)
        return self[name]

    def __repr__(self) -> str:
        return "sym"


sym = _SymbolNamespace()
