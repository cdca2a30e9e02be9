"""Recogniser of the second kernel class the NVIDIA target runs: the masked element-wise map.

The class is the one-dimensional load / compute / store kernel of the reference simulator's own
tests (tests/test_simulator.py:210-224):

    @kernel(work_shape=(W,), group_shape=(4,))
    def add_vec(group, x: Buffer[W], y: Buffer[W]) -> None:
        gid = group.work_offset[0]
        vec = group.vload(x[gid:], shape=(4,))
        group.store(y[gid:], vec + 2)

Every workgroup loads the `G` elements that start at its work offset (elements past the end of
the buffer are inactive, hc/simulator.py:1338-1357), applies element-wise arithmetic, and stores
the active elements that fall inside the output (hc/simulator.py:1441-1458). With
work_shape=(W,), group_shape=(G,) and a load of exactly G elements the groups tile [0, W) once,
so the kernel computes out[i] = f(x[i] [, y[i]]) for i < W and touches nothing else. The group
size is not observable (doc/langref.md:694-697); the GPU kernel re-tiles to 128-bit vectors.
The two-dimensional form is the same with one offset, one slice and one group extent per axis
(`r0, c0 = group.work_offset`, `group.load(x[r0:, c0:], shape=(GM, GN))`, work_shape=(M, N)):
the (GM, GN) workgroups tile the matrix once (hc/simulator.py:914-920), the function is
element-wise, so the launch runs over the M * N elements in row-major order.

As for the matmul family the body is matched statement by statement and anything else is refused
with a diagnostic. `f` must be a chain of at most eight float32 operations, each with a constant
or with the element of one second input: `*`, `+`, `-` (either way round), `np.maximum`,
`np.minimum`, unary minus. Constants must be Python numbers or `np.float32(...)`: NumPy then
computes in float32 (a Python scalar never widens an array), one rounding per operation, which
is what the CUDA kernel does, so results are bit-identical to the simulator's. A float64
constant would make NumPy compute in float64 and is refused.
"""

from __future__ import annotations

import ast
from dataclasses import dataclass
from typing import Any

import numpy as np

__all__ = ["MapContract", "recognise_elementwise_map"]

MAX_MAP_OPS = 8


@dataclass(frozen=True)
class MapContract:
    """What the recogniser established about an element-wise kernel."""

    kernel_name: str
    x_param: str                 # the input the chain starts from
    other_param: str | None      # the second input, if any operation uses it
    out_param: str               # the buffer that is stored to (may be an input: in place)
    extent: Any                  # symbol name (str) or fixed int extent of all buffers; a pair for rank 2
    group_size: Any              # G of the kernel as written (not observable on the GPU); a pair for rank 2
    ops: tuple[tuple, ...]       # ("scale", c) ("add", c) ("max", c) ("min", c) ("rsub", c) ("rmax", c)
    #                              ("rmin", c) ("add_other",) ("sub_other",) ("rsub_other",) ("mul_other",)
    #                              ("max_other",) ("min_other",) ("rmax_other",) ("rmin_other",), in order
    dtype: str = "float32"
    rank: int = 1                # 1: vectors; 2: matrices tiled by (GM, GN) workgroups, elements in row-major order


@dataclass(frozen=True)
class _Chain:
    base: str            # input parameter the value starts from
    ops: tuple[tuple, ...]
    other: str | None    # second input parameter used so far


def _const(node: ast.AST, consts: dict[str, Any]) -> float | None:
    """A constant NumPy combines with a float32 array in float32: a Python number (literal or
    module-level / closure name), `np.float32(<that>)`, or its negation."""
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)):
        inner = _const(node.operand, consts)
        if inner is None:
            return None
        return -inner if isinstance(node.op, ast.USub) else inner
    if isinstance(node, ast.Call) and len(node.args) == 1 and not node.keywords:
        func = node.func
        name = func.attr if isinstance(func, ast.Attribute) else (func.id if isinstance(func, ast.Name) else None)
        return _const(node.args[0], consts) if name == "float32" else None
    if isinstance(node, ast.Constant):
        value = node.value
    elif isinstance(node, ast.Name):
        value = consts.get(node.id)
    else:
        return None
    if isinstance(value, bool):
        return None
    if isinstance(value, np.float32) or type(value) in (int, float):
        with np.errstate(over="ignore"):
            value = float(np.float32(value))
        return value if np.isfinite(value) else None
    return None


_BINARY = {ast.Mult: ("scale", "scale", "mul_other", "mul_other"),
           ast.Add: ("add", "add", "add_other", "add_other"),
           ast.Sub: ("add", "rsub", "sub_other", "rsub_other")}  # (v op c, c op v, v op w, w op v)
# np.maximum / np.minimum return their second operand when neither is greater (zeros of opposite
# sign), so the operand order is kept: "r..." has the chain as the second operand.
_CALLS = {"maximum": ("max", "rmax", "max_other", "rmax_other"), "minimum": ("min", "rmin", "min_other", "rmin_other")}


class _Expressions:
    def __init__(self, consts: dict[str, Any]) -> None:
        self.consts = consts
        self.env: dict[str, _Chain] = {}
        self.why: str | None = None

    def fail(self, text: str) -> None:
        if self.why is None:
            self.why = text
        return None

    def chain(self, node: ast.AST) -> _Chain | None:
        if isinstance(node, ast.Name):
            found = self.env.get(node.id)
            return found if found is not None else self.fail(f"`{node.id}` is not a loaded vector")
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
            inner = self.chain(node.operand)
            return None if inner is None else _Chain(inner.base, inner.ops + (("scale", -1.0),), inner.other)
        if isinstance(node, ast.BinOp) and type(node.op) in _BINARY:
            return self._combine(node, node.left, node.right, _BINARY[type(node.op)],
                                 negate_const=isinstance(node.op, ast.Sub))
        if isinstance(node, ast.Call) and not node.keywords:
            func = node.func
            name = func.attr if isinstance(func, ast.Attribute) else (func.id if isinstance(func, ast.Name) else None)
            if name in _CALLS and len(node.args) == 2:
                return self._combine(node, node.args[0], node.args[1], _CALLS[name], negate_const=False)
            if (name == "astype" and isinstance(func, ast.Attribute) and len(node.args) == 1
                    and ast.unparse(node.args[0]).split(".")[-1] == "float32"):
                return self.chain(func.value)
        return self.fail(f"`{ast.unparse(node)}` is not element-wise arithmetic this target runs (`*`, `+`, `-`, "
                         f"np.maximum, np.minimum with a constant or a second loaded vector)")

    def _combine(self, node: ast.AST, left: ast.AST, right: ast.AST, kinds: tuple[str, str, str, str],
                 negate_const: bool) -> _Chain | None:
        v_c, c_v, v_w, w_v = kinds
        left_const, right_const = _const(left, self.consts), _const(right, self.consts)
        if right_const is not None and left_const is None:
            inner = self.chain(left)
            if inner is None:
                return None
            value = -right_const if negate_const else right_const  # v - c == v + (-c), exactly
            return _Chain(inner.base, inner.ops + ((v_c, value),), inner.other)
        if left_const is not None and right_const is None:
            inner = self.chain(right)
            return None if inner is None else _Chain(inner.base, inner.ops + ((c_v, left_const),), inner.other)
        if left_const is not None:
            return self.fail(f"`{ast.unparse(node)}` has no vector operand")
        lhs, rhs = self.chain(left), self.chain(right)
        if lhs is None or rhs is None:
            return None
        # One side must be a second input exactly as it was loaded.
        for main, bare, kind in ((lhs, rhs, v_w), (rhs, lhs, w_v)):
            if bare.ops == () and bare.base != main.base and main.other in (None, bare.base):
                return _Chain(main.base, main.ops + ((kind,),), bare.base)
        return self.fail(f"`{ast.unparse(node)}` combines two computed vectors; one operand of a vector-vector "
                         f"operation must be a second input as loaded")


def _dim_key(dim: Any) -> Any:
    if isinstance(dim, bool):
        return None
    if isinstance(dim, int):
        return int(dim)
    name = getattr(dim, "name", None)
    return name if isinstance(name, str) and hasattr(dim, "free_symbols") else None


def _evaluate(expr: Any, names: dict[str, int]) -> int | None:
    if isinstance(expr, bool):
        return None
    if isinstance(expr, int):
        return int(expr)
    evaluate = getattr(expr, "eval", None)
    try:
        return None if evaluate is None else int(evaluate(names))
    except Exception:
        return None


def recognise_elementwise_map(kernel_fn: Any) -> tuple[MapContract | None, list[str]]:
    """Decides whether `kernel_fn` is a masked element-wise map. Returns (contract, diagnostics)."""
    from ._pipeline import _function_consts, _function_node, _without_docstring, resolved_annotations
    import inspect

    name = getattr(kernel_fn, "__name__", "<kernel>")
    meta = getattr(kernel_fn, "__hc_kernel__", None)
    if meta is None:
        return None, [f"{name}: not a @kernel function"]

    def refuse(text: str) -> tuple[None, list[str]]:
        return None, [f"{name}: {text}"]

    try:
        params = list(inspect.signature(kernel_fn).parameters)
    except (TypeError, ValueError):
        return refuse("signature is not inspectable")
    if len(params) not in (2, 3, 4):
        return refuse(f"an element-wise map takes (group, x) in place, (group, x, out) or (group, x, y, out); "
                      f"found {len(params)} parameters")
    group = params[0]
    annotations = resolved_annotations(kernel_fn)
    extents: tuple | None = None
    for param in params[1:]:
        spec = annotations.get(param)
        if type(spec).__name__ != "BufferSpec" or len(spec.dimensions) not in (1, 2):
            return refuse(f"parameter `{param}` must be annotated as a rank-1 or rank-2 Buffer")
        keys = tuple(_dim_key(d) for d in spec.dimensions)
        if None in keys or (extents is not None and keys != extents):
            return refuse("all buffers of an element-wise map must have the same extents (the same symbols or integers)")
        extents = keys
        if spec.dtype not in (None, "float32"):
            return refuse(f"`{param}` is Buffer[..., {spec.dtype}]; this target runs element-wise kernels on float32")
    assert extents is not None
    rank = len(extents)

    # Geometry: work_shape == the buffers' extents, group_shape constant, one axis per buffer axis.
    work, group_shape = meta.work_shape, meta.group_shape
    work = work if isinstance(work, tuple) else (work,)
    group_shape = group_shape if isinstance(group_shape, tuple) else (group_shape,)
    if len(work) != rank or len(group_shape) != rank:
        return refuse("work_shape and group_shape of an element-wise map must have one axis per buffer axis")
    group_sizes = tuple(_evaluate(g, {}) for g in group_shape)
    if any(g is None or g <= 0 for g in group_sizes):
        return refuse("group_shape must be a positive constant")
    for probe in ((1, 3), (5, 1), (4096, 17), (1000003, 2)):
        names = {key: probe[axis] for axis, key in enumerate(extents) if isinstance(key, str)}
        for axis, key in enumerate(extents):
            want = names[key] if isinstance(key, str) else key
            if _evaluate(work[axis], names) != want:
                return refuse(f"work_shape must be the buffers' extent, one workitem per element (axis {axis} evaluates "
                              f"to {_evaluate(work[axis], names)} for an extent of {want})")

    fn_node = _function_node(kernel_fn)
    if fn_node is None:
        return refuse("kernel source is unavailable, so its body cannot be checked")
    consts = _function_consts(kernel_fn)
    body = _without_docstring(list(fn_node.body))
    if body and isinstance(body[-1], ast.Return) and (body[-1].value is None or (
            isinstance(body[-1].value, ast.Constant) and body[-1].value.value is None)):
        body = body[:-1]

    # The same kernel written one element per work-item (tests/test_simulator.py:901-917):
    #
    #     @group.workitems
    #     def inner(wi) -> None:
    #         gid = wi.global_id()[0]
    #         vec = group.vload(src[gid:], shape=(1,))
    #         group.store(dst[gid:], vec + 2)
    #     inner()
    #
    # Every work-item of every group runs the body once with its own global id (ids past the end of
    # the buffers load nothing and store nothing), so it is the map with windows of one element.
    workitem: str | None = None
    if (len(body) == 2 and isinstance(body[0], ast.FunctionDef) and isinstance(body[1], ast.Expr)
            and isinstance(body[1].value, ast.Call) and isinstance(body[1].value.func, ast.Name)
            and body[1].value.func.id == body[0].name and not body[1].value.args and not body[1].value.keywords):
        inner = body[0]
        decorators = [ast.unparse(d) for d in inner.decorator_list]
        inner_args = inner.args
        if (decorators == [f"{group}.workitems"] and len(inner_args.args) == 1 and not inner_args.vararg
                and not inner_args.kwarg and not inner_args.kwonlyargs and not inner_args.posonlyargs):
            workitem = inner_args.args[0].arg
            body = _without_docstring(list(inner.body))
            if body and isinstance(body[-1], ast.Return) and (body[-1].value is None or (
                    isinstance(body[-1].value, ast.Constant) and body[-1].value.value is None)):
                body = body[:-1]
            group_sizes = (1,) * rank  # the window a work-item loads and stores

    offset_names: dict[str, int] = {}  # name -> axis of group.work_offset it holds
    exprs = _Expressions(consts)
    out_param: str | None = None
    result: _Chain | None = None
    shape_text = "(" + ", ".join(str(g) for g in group_sizes) + ("," if rank == 1 else "") + ")"
    window_text = "buf[" + ", ".join(f"o{axis}:" for axis in range(rank)) + "]" if rank > 1 else "buf[gid:]"

    def window_of(node: ast.AST) -> str | None:
        """`buf[gid:]` / `buf[gid:gid + G]` (one slice per axis, each from that axis' work offset) -> buf."""
        if not (isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name) and node.value.id in params[1:]):
            return None
        parts = list(node.slice.elts) if isinstance(node.slice, ast.Tuple) else [node.slice]
        if len(parts) != rank:
            return None
        for axis, part in enumerate(parts):
            if not (isinstance(part, ast.Slice) and part.step is None and isinstance(part.lower, ast.Name)
                    and offset_names.get(part.lower.id) == axis):
                return None
            upper = part.upper
            if upper is not None:
                ok = (isinstance(upper, ast.BinOp) and isinstance(upper.op, ast.Add)
                      and isinstance(upper.left, ast.Name) and upper.left.id == part.lower.id
                      and _const(upper.right, consts) == group_sizes[axis])
                if not ok:
                    return None
        return node.value.id

    def work_offset_axis(value: ast.AST | None) -> int | None:
        """`group.work_offset[axis]` (or, in a work-item body, `wi.global_id()[axis]`) -> axis."""
        if workitem is not None:
            if (isinstance(value, ast.Subscript) and isinstance(value.slice, ast.Constant)
                    and isinstance(value.slice.value, int) and not isinstance(value.slice.value, bool)
                    and 0 <= value.slice.value < rank and ast.unparse(value.value) == f"{workitem}.global_id()"):
                return value.slice.value
            return None
        if (isinstance(value, ast.Subscript) and isinstance(value.value, ast.Attribute)
                and value.value.attr == "work_offset" and isinstance(value.value.value, ast.Name)
                and value.value.value.id == group and isinstance(value.slice, ast.Constant)
                and isinstance(value.slice.value, int) and 0 <= value.slice.value < rank):
            return value.slice.value
        return None

    for stmt in body:
        text = ast.unparse(stmt)
        if out_param is not None:
            return refuse(f"`{text}` follows the store; an element-wise map ends with it")
        target = (stmt.targets[0].id if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1
                  and isinstance(stmt.targets[0], ast.Name) else None)
        value = stmt.value if isinstance(stmt, (ast.Assign, ast.Expr)) else None
        # gid = group.work_offset[axis]   (or `r0, c0 = group.work_offset` for two axes)
        if target and work_offset_axis(value) is not None:
            offset_names[target] = work_offset_axis(value)
            continue
        if (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Tuple)
                and len(stmt.targets[0].elts) == rank and all(isinstance(e, ast.Name) for e in stmt.targets[0].elts)
                and ((workitem is None and isinstance(value, ast.Attribute) and value.attr == "work_offset"
                      and isinstance(value.value, ast.Name) and value.value.id == group)
                     or (workitem is not None and value is not None and ast.unparse(value) == f"{workitem}.global_id()"))):
            for axis, elt in enumerate(stmt.targets[0].elts):
                offset_names[elt.id] = axis
            continue
        call = value if isinstance(value, ast.Call) else None
        func = call.func if call is not None else None
        on_group = (isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name) and func.value.id == group)
        # vec = group.vload(x[gid:], shape=(G,))   (or group.load)
        if target and on_group and func.attr in ("vload", "load"):
            source = window_of(call.args[0]) if len(call.args) == 1 else None
            keywords = {kw.arg: kw.value for kw in call.keywords}
            shape = keywords.get("shape")
            shape_ok = (set(keywords) == {"shape"} and isinstance(shape, ast.Tuple) and len(shape.elts) == rank
                        and tuple(_const(elt, consts) for elt in shape.elts) == group_sizes)
            if source is None or not shape_ok:
                return refuse(f"`{text}` must load the group's own window, `{group}.vload({window_text}, shape={shape_text})` "
                              f"with the offsets taken from {group}.work_offset and the group shape as shape")
            exprs.env[target] = _Chain(source, (), None)
            continue
        # group.store(out[gid:], <expression>)
        if isinstance(stmt, ast.Expr) and on_group and func.attr == "store" and len(call.args) == 2 and not call.keywords:
            out_param = window_of(call.args[0])
            if out_param is None:
                return refuse(f"`{text}` must store to the group's own window, `{group}.store(out{window_text[3:]}, vec)`")
            result = exprs.chain(call.args[1])
            if result is None:
                return refuse(exprs.why or "unsupported expression")
            continue
        # vec = <expression>
        if target and value is not None:
            chain = exprs.chain(value)
            if chain is None:
                return refuse(exprs.why or "unsupported expression")
            exprs.env[target] = chain
            continue
        return refuse(f"`{text}` is not part of the load / element-wise / store form")

    if out_param is None or result is None:
        return refuse(f"the kernel must end with `{group}.store(out{window_text[3:]}, vec)`")
    if len(result.ops) > MAX_MAP_OPS:
        return refuse(f"at most {MAX_MAP_OPS} element-wise operations are supported, found {len(result.ops)}")
    return MapContract(kernel_name=name, x_param=result.base, other_param=result.other, out_param=out_param,
                       extent=extents[0] if rank == 1 else extents, group_size=group_sizes[0] if rank == 1 else group_sizes,
                       ops=result.ops, rank=rank), []
