"""Stand-in for the third-party `ixsimpl` symbolic engine (test infrastructure only).

The reference project takes its integer-expression engine from a git submodule
(third_party/ixsimpl -> Hardcode84/4, .gitmodules:5-7) that is not vendored; its pinned
revision cannot be recovered. This module implements just the interface that
hc/_symbols_backend.py:11-73 declares and the node attributes hc/symbols.py touches, with
exact `fractions.Fraction` arithmetic and eager constant folding. It exists so that the
UNMODIFIED reference simulator can evaluate launch-shape integers such as
`ceil_div(M, 16) * 32` while golden fixtures are generated. None of the matmul arithmetic
passes through it. It does not reproduce the real engine's simplifier or its string
rendering, and nothing in the product imports it.
"""

from __future__ import annotations

import math
from fractions import Fraction

(INT, RAT, SYM, ADD, MUL, FLOOR, CEIL, MOD, PIECEWISE, MAX, MIN, XOR, CMP, AND, OR, NOT, TRUE,
 FALSE) = range(18)

_CMP_OPS = {
    "<": lambda a, b: a < b,
    "<=": lambda a, b: a <= b,
    ">": lambda a, b: a > b,
    ">=": lambda a, b: a >= b,
    "==": lambda a, b: a == b,
    "!=": lambda a, b: a != b,
}


class Node:
    __slots__ = ("tag", "children", "value", "sym_name", "cmp_op")

    is_error = False
    is_parse_error = False
    is_domain_error = False

    def __init__(self, tag, children=(), value=None, sym_name=None, cmp_op=None):
        self.tag = tag
        self.children = tuple(children)
        self.value = value
        self.sym_name = sym_name
        self.cmp_op = cmp_op

    # -- structure ------------------------------------------------------------------
    def _key(self):
        return (self.tag, self.value, self.sym_name, self.cmp_op,
                tuple(child._key() for child in self.children))

    def __eq__(self, other):
        return isinstance(other, Node) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    @property
    def free_symbols(self):
        if self.tag == SYM:
            return frozenset({self})
        found = frozenset()
        for child in self.children:
            found |= child.free_symbols
        return found

    def _const(self):
        if self.tag in (INT, RAT):
            return self.value
        return None

    # -- evaluation -----------------------------------------------------------------
    def subs(self, mapping):
        by_name = {}
        for key, value in mapping.items():
            name = key.sym_name if isinstance(key, Node) else str(key)
            by_name[name] = value if isinstance(value, Node) else _number(value)
        return self._subs(by_name)

    def _subs(self, by_name):
        if self.tag == SYM:
            return by_name.get(self.sym_name, self)
        if not self.children:
            return self
        return _build(self.tag, [child._subs(by_name) for child in self.children], self.cmp_op)

    def simplify(self, assumptions=None):
        return self

    def __int__(self):
        value = self._const()
        if value is None or value.denominator != 1:
            raise TypeError("expression is not a constant integer")
        return int(value)

    # -- arithmetic -----------------------------------------------------------------
    def __add__(self, other):
        return _build(ADD, [self, _node(other)])

    def __sub__(self, other):
        return _build(ADD, [self, _build(MUL, [_number(-1), _node(other)])])

    def __mul__(self, other):
        return _build(MUL, [self, _node(other)])

    def __truediv__(self, other):
        other = _node(other)
        value = other._const()
        if value is None:
            raise TypeError("the ixsimpl stand-in only divides by constants")
        if value == 0:
            raise ZeroDivisionError("division by zero")
        return _build(MUL, [self, _number(1 / value)])

    def __neg__(self):
        return _build(MUL, [_number(-1), self])

    def __lt__(self, other):
        return _build(CMP, [self, _node(other)], "<")

    def __le__(self, other):
        return _build(CMP, [self, _node(other)], "<=")

    def __gt__(self, other):
        return _build(CMP, [self, _node(other)], ">")

    def __ge__(self, other):
        return _build(CMP, [self, _node(other)], ">=")

    def to_c(self):
        return str(self)

    def __str__(self):
        if self.tag in (INT, RAT):
            return str(self.value)
        if self.tag == SYM:
            return self.sym_name
        if self.tag == TRUE:
            return "True"
        if self.tag == FALSE:
            return "False"
        names = {ADD: "add", MUL: "mul", FLOOR: "floor", CEIL: "ceiling", MOD: "Mod", MAX: "Max",
                 MIN: "Min", XOR: "xor", CMP: f"cmp[{self.cmp_op}]", AND: "and", OR: "or",
                 NOT: "not", PIECEWISE: "piecewise"}
        inner = ", ".join(str(child) for child in self.children)
        return f"{names[self.tag]}({inner})"


def _number(value):
    value = Fraction(value)
    return Node(INT if value.denominator == 1 else RAT, value=value)


def _node(value):
    if isinstance(value, Node):
        return value
    if isinstance(value, bool):
        return Node(TRUE if value else FALSE)
    return _number(value)


def _build(tag, children, cmp_op=None):
    children = [_node(child) for child in children]
    consts = [child._const() for child in children]
    if all(value is not None for value in consts):
        if tag == ADD:
            return _number(sum(consts))
        if tag == MUL:
            return _number(math.prod(consts))
        if tag == FLOOR:
            return _number(math.floor(consts[0]))
        if tag == CEIL:
            return _number(math.ceil(consts[0]))
        if tag == MOD:
            return _number(consts[0] - consts[1] * math.floor(consts[0] / consts[1]))
        if tag == MAX:
            return _number(max(consts))
        if tag == MIN:
            return _number(min(consts))
        if tag == XOR:
            return _number(int(consts[0]) ^ int(consts[1]))
        if tag == CMP:
            return Node(TRUE if _CMP_OPS[cmp_op](consts[0], consts[1]) else FALSE)
    truth = [child.tag for child in children]
    if tag == NOT and truth[0] in (TRUE, FALSE):
        return Node(FALSE if truth[0] == TRUE else TRUE)
    if tag == AND and all(t in (TRUE, FALSE) for t in truth):
        return Node(TRUE if all(t == TRUE for t in truth) else FALSE)
    if tag == OR and all(t in (TRUE, FALSE) for t in truth):
        return Node(TRUE if any(t == TRUE for t in truth) else FALSE)
    if tag == PIECEWISE:
        for index in range(0, len(children), 2):
            cond = children[index + 1]
            if cond.tag == TRUE:
                return children[index]
            if cond.tag != FALSE:
                break
    return Node(tag, children, cmp_op=cmp_op)


class Context:
    def __init__(self):
        self.errors = []

    def sym(self, name):
        return Node(SYM, sym_name=str(name))

    def int_(self, value):
        return _number(int(value))

    def rat(self, num, den):
        return _number(Fraction(int(num), int(den)))

    def true_(self):
        return Node(TRUE)

    def false_(self):
        return Node(FALSE)

    def parse(self, text):
        raise NotImplementedError("the ixsimpl stand-in does not parse text")

    def eq(self, lhs, rhs):
        return _build(CMP, [lhs, rhs], "==")

    def ne(self, lhs, rhs):
        return _build(CMP, [lhs, rhs], "!=")

    def check(self, expr, assumptions=None):
        if expr.tag == TRUE:
            return True
        if expr.tag == FALSE:
            return False
        return None


def same_node(lhs, rhs):
    return lhs == rhs


def and_(lhs, rhs):
    return _build(AND, [lhs, rhs])


def or_(lhs, rhs):
    return _build(OR, [lhs, rhs])


def not_(value):
    return _build(NOT, [value])


def floor(value):
    return _build(FLOOR, [value])


def ceil(value):
    return _build(CEIL, [value])


def mod(lhs, rhs):
    return _build(MOD, [lhs, rhs])


def min_(lhs, rhs):
    return _build(MIN, [lhs, rhs])


def max_(lhs, rhs):
    return _build(MAX, [lhs, rhs])


def xor_(lhs, rhs):
    return _build(XOR, [lhs, rhs])


def pw(*branches):
    flat = []
    for value, cond in branches:
        flat.extend([value, cond])
    return _build(PIECEWISE, flat)
