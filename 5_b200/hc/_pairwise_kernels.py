"""Recogniser of the third kernel class the NVIDIA target runs: pairwise distances.

The class is the two-dimensional workgroup kernel that opens the reference simulator's own tests
(tests/test_simulator.py:142-167):

    @kernel(work_shape=(W1, W2), group_shape=(4, 4))
    def pairwise(group, x1: Buffer[W1, H], x2: Buffer[W2, H], out: Buffer[W1, W2]) -> None:
        gid = group.work_offset
        lhs = group.load(x1[gid[0]:], shape=(group.shape[0], x1.shape[1]))
        rhs = group.load(x2[gid[1]:], shape=(group.shape[1], x2.shape[1]))
        diff = ((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2)
        group.store(out[gid[0]:, gid[1]:], np.sqrt(diff))

A workgroup loads the G1 rows of x1 and the G2 rows of x2 that start at its work offsets (rows
past the end of a buffer are inactive, hc/simulator.py:1338-1357), forms all G1 x G2 squared
differences, reduces them over the shared axis and stores the active results that fall inside
`out` (hc/simulator.py:1441-1458). With work_shape=(W1, W2) the groups tile the W1 x W2 outputs
once, so the kernel computes out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h])^2) and touches nothing
else; the group shape is not observable (doc/langref.md:694-697) and the GPU kernel re-tiles.

The body is matched statement by statement against exactly this form (the square root is
optional, the two operands of the subtraction may be swapped, temporaries may be named freely);
anything else is refused with a diagnostic. The arithmetic is float32 with one rounding per
operation and the reduction in the order of NumPy's float32 sum, which the CUDA kernel reproduces
(lib/Kernels/pairwise_distance_sm100a.cu), so results are bit-identical to the simulator's.
"""

from __future__ import annotations

import ast
import copy
from dataclasses import dataclass
from typing import Any

__all__ = ["PairwiseContract", "recognise_pairwise"]


@dataclass(frozen=True)
class PairwiseContract:
    """What the recogniser established about a pairwise-distance kernel."""

    kernel_name: str
    lhs_param: str        # rows follow work axis 0: Buffer[W1, H]
    rhs_param: str        # rows follow work axis 1: Buffer[W2, H]
    out_param: str        # Buffer[W1, W2]
    extents: tuple        # (W1, W2, H): symbol names or fixed integers
    group_shape: tuple    # (G1, G2) of the kernel as written (not observable on the GPU)
    take_sqrt: bool       # np.sqrt of the sum (Euclidean distance) or the sum itself
    dtype: str = "float32"


def _dim_key(dim: Any) -> Any:
    if isinstance(dim, int) and not isinstance(dim, bool):
        return dim
    name = getattr(dim, "name", None)
    return name if isinstance(name, str) else None


class _Substitute(ast.NodeTransformer):
    """Replaces names bound to expressions by those expressions (temporaries inlined)."""

    def __init__(self, env: dict[str, ast.AST]) -> None:
        self.env = env

    def visit_Name(self, node: ast.Name) -> ast.AST:
        if isinstance(node.ctx, ast.Load) and node.id in self.env:
            return copy.deepcopy(self.env[node.id])
        return node


def _dump(source: str) -> str:
    return ast.dump(ast.parse(source, mode="eval").body)


def recognise_pairwise(kernel_fn: Any) -> tuple[PairwiseContract | None, list[str]]:
    """Decides whether `kernel_fn` is the pairwise-distance kernel. Returns (contract, diagnostics)."""
    from ._map_kernels import _evaluate
    from ._pipeline import _function_node, _without_docstring, resolved_annotations
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
    if len(params) != 4:
        return refuse(f"a pairwise kernel takes (group, x1, x2, out); found {len(params)} parameters")
    group = params[0]
    annotations = resolved_annotations(kernel_fn)
    dims: dict[str, tuple] = {}
    for param in params[1:]:
        spec = annotations.get(param)
        if type(spec).__name__ != "BufferSpec" or len(spec.dimensions) != 2:
            return refuse(f"parameter `{param}` must be annotated as a rank-2 Buffer")
        keys = tuple(_dim_key(d) for d in spec.dimensions)
        if None in keys:
            return refuse(f"the extents of `{param}` must be symbols or integers")
        if spec.dtype not in (None, "float32"):
            return refuse(f"`{param}` is Buffer[..., {spec.dtype}]; this target runs pairwise kernels on float32")
        dims[param] = keys

    work, group_shape = meta.work_shape, meta.group_shape
    work = work if isinstance(work, tuple) else (work,)
    group_shape = group_shape if isinstance(group_shape, tuple) else (group_shape,)
    if len(work) != 2 or len(group_shape) != 2:
        return refuse("work_shape and group_shape of a pairwise kernel must have two axes")
    group_sizes = tuple(_evaluate(g, {}) for g in group_shape)
    if any(g is None or g <= 0 for g in group_sizes):
        return refuse("group_shape must be a pair of positive constants")

    fn_node = _function_node(kernel_fn)
    if fn_node is None:
        return refuse("kernel source is unavailable, so its body cannot be checked")
    body = _without_docstring(list(fn_node.body))
    if body and isinstance(body[-1], ast.Return) and (body[-1].value is None or (
            isinstance(body[-1].value, ast.Constant) and body[-1].value.value is None)):
        body = body[:-1]

    whole_offset: set[str] = set()       # names bound to group.work_offset
    axis_offset: dict[str, int] = {}     # names bound to group.work_offset[axis]
    loaded: dict[str, tuple[str, int]] = {}  # name -> (buffer parameter, work axis its rows follow)
    temporaries: dict[str, ast.AST] = {}
    stored: tuple[str, ast.AST] | None = None

    def is_work_offset(node: ast.AST) -> bool:
        return (isinstance(node, ast.Attribute) and node.attr == "work_offset" and isinstance(node.value, ast.Name)
                and node.value.id == group)

    def offset_axis(node: ast.AST | None) -> int | None:
        """`gid[axis]`, `group.work_offset[axis]` or a name bound to one of them -> axis."""
        if isinstance(node, ast.Name):
            return axis_offset.get(node.id)
        if (isinstance(node, ast.Subscript) and isinstance(node.slice, ast.Constant) and node.slice.value in (0, 1)
                and not isinstance(node.slice.value, bool)):
            base = node.value
            if is_work_offset(base) or (isinstance(base, ast.Name) and base.id in whole_offset):
                return int(node.slice.value)
        return None

    def open_slice_from(part: ast.AST) -> int | None:
        """`<offset of an axis>:` -> that axis."""
        if isinstance(part, ast.Slice) and part.upper is None and part.step is None:
            return offset_axis(part.lower)
        return None

    def shape_ok(node: ast.AST | None, param: str, axis: int) -> bool:
        """(group.shape[axis] or the constant G of that axis, <param>.shape[1])"""
        if not (isinstance(node, ast.Tuple) and len(node.elts) == 2):
            return False
        rows, cols = node.elts
        rows_text, cols_text = ast.unparse(rows), ast.unparse(cols)
        rows_ok = rows_text == f"{group}.shape[{axis}]" or rows_text == str(group_sizes[axis])
        return rows_ok and cols_text == f"{param}.shape[1]"

    for stmt in body:
        text = ast.unparse(stmt)
        if stored is not None:
            return refuse(f"`{text}` follows the store; a pairwise kernel ends with it")
        target = (stmt.targets[0].id if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1
                  and isinstance(stmt.targets[0], ast.Name) else None)
        value = stmt.value if isinstance(stmt, (ast.Assign, ast.Expr)) else None
        if target and value is not None and is_work_offset(value):
            whole_offset.add(target)
            continue
        if target and offset_axis(value) is not None and not isinstance(value, ast.Name):
            axis_offset[target] = offset_axis(value)
            continue
        if (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Tuple)
                and len(stmt.targets[0].elts) == 2 and all(isinstance(e, ast.Name) for e in stmt.targets[0].elts)
                and value is not None and is_work_offset(value)):
            for axis, elt in enumerate(stmt.targets[0].elts):
                axis_offset[elt.id] = axis
            continue
        call = value if isinstance(value, ast.Call) else None
        func = call.func if call is not None else None
        on_group = isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name) and func.value.id == group
        if target and on_group and func.attr == "load":
            window = call.args[0] if len(call.args) == 1 else None
            keywords = {kw.arg: kw.value for kw in call.keywords}
            ok = (isinstance(window, ast.Subscript) and isinstance(window.value, ast.Name)
                  and window.value.id in params[1:] and set(keywords) == {"shape"})
            axis = open_slice_from(window.slice) if ok else None
            if axis is None or not shape_ok(keywords.get("shape"), window.value.id, axis):
                return refuse(f"`{text}` must load the group's rows of a buffer, `{group}.load(x[gid[a]:], "
                              f"shape=({group}.shape[a], x.shape[1]))` with gid = {group}.work_offset")
            loaded[target] = (window.value.id, axis)
            continue
        if isinstance(stmt, ast.Expr) and on_group and func.attr == "store" and len(call.args) == 2 and not call.keywords:
            window = call.args[0]
            parts = window.slice.elts if isinstance(window, ast.Subscript) and isinstance(window.slice, ast.Tuple) else []
            if not (isinstance(window, ast.Subscript) and isinstance(window.value, ast.Name)
                    and window.value.id in params[1:] and len(parts) == 2
                    and open_slice_from(parts[0]) == 0 and open_slice_from(parts[1]) == 1):
                return refuse(f"`{text}` must store to the group's own window, `{group}.store(out[gid[0]:, gid[1]:], d)`")
            stored = (window.value.id, call.args[1])
            continue
        if target and value is not None:
            temporaries[target] = _Substitute(temporaries).visit(copy.deepcopy(value))
            continue
        return refuse(f"`{text}` is not part of the load / pairwise difference / store form")

    if stored is None:
        return refuse(f"the kernel must end with `{group}.store(out[gid[0]:, gid[1]:], d)`")
    out_param, expression = stored
    expression = _Substitute(temporaries).visit(copy.deepcopy(expression))
    rows_names = [n for n, (_, axis) in loaded.items() if axis == 0]
    cols_names = [n for n, (_, axis) in loaded.items() if axis == 1]
    found: tuple[str, str, bool] | None = None
    dumped = ast.dump(expression)
    for lhs in rows_names:
        for rhs in cols_names:
            for first, second in ((f"{lhs}[:, None, :]", f"{rhs}[None, :, :]"), (f"{rhs}[None, :, :]", f"{lhs}[:, None, :]")):
                squared = f"(({first} - {second}) ** 2).sum(axis=2)"
                for module in ("np", "numpy"):
                    if dumped == _dump(f"{module}.sqrt({squared})"):
                        found = (lhs, rhs, True)
                if dumped == _dump(squared):
                    found = (lhs, rhs, False)
    if found is None:
        return refuse(f"`{ast.unparse(expression)}` is not `np.sqrt(((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2))` "
                      f"(or that sum without the square root) of a value loaded along work axis 0 and one loaded along axis 1")
    lhs_param, rhs_param = loaded[found[0]][0], loaded[found[1]][0]
    if len({lhs_param, rhs_param, out_param}) != 3:
        return refuse("x1, x2 and out must be three different buffers")
    (w1, h1), (w2, h2), (o1, o2) = dims[lhs_param], dims[rhs_param], dims[out_param]
    if h1 != h2:
        return refuse(f"`{lhs_param}` and `{rhs_param}` must share their second extent (found {h1} and {h2})")
    if (o1, o2) != (w1, w2):
        return refuse(f"`{out_param}` must be Buffer[{w1}, {w2}] (found Buffer[{o1}, {o2}])")
    # work_shape == (W1, W2): one workitem per output.
    for probe in ((1, 3), (5, 1), (4096, 17), (1000003, 2)):
        names = {key: probe[axis] for axis, key in enumerate((w1, w2)) if isinstance(key, str)}
        if isinstance(w1, str) and w1 == w2:
            names[w1] = probe[0]
        for axis, key in enumerate((w1, w2)):
            want = names[key] if isinstance(key, str) else key
            if _evaluate(work[axis], names) != want:
                return refuse(f"work_shape must be the extents of `{out_param}`, one workitem per output (axis {axis} "
                              f"evaluates to {_evaluate(work[axis], names)} for an extent of {want})")
    return PairwiseContract(kernel_name=name, lhs_param=lhs_param, rhs_param=rhs_param, out_param=out_param,
                            extents=(w1, w2, h1), group_shape=group_sizes, take_sqrt=found[2]), []
