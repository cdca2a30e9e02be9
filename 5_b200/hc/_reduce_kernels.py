"""Recogniser of the fourth kernel class the NVIDIA target runs: row sums.

The class is the one-dimensional workgroup kernel that reduces the rows it loads -- the load of the
reference simulator's first test (tests/test_simulator.py:153-154) followed by the reduction of the
simulator's value type (hc/_sim_types.py:338-351, 501-518):

    @kernel(work_shape=(W,), group_shape=(4,))
    def row_sums(group, x: Buffer[W, H], out: Buffer[W]) -> None:
        r0 = group.work_offset[0]
        rows = group.load(x[r0:], shape=(group.shape[0], x.shape[1]))
        group.store(out[r0:], rows.sum(axis=1))

A workgroup loads the G rows of x that start at its work offset (rows past the end of the buffer
are inactive, hc/simulator.py:1338-1357), reduces each over its values (`_reduce_arrays` keeps the
active values of a row and hands them to np.sum, hc/_sim_types.py:1050-1102) and stores the active
results that fall inside `out` (hc/simulator.py:1441-1458). With work_shape=(W,) the groups cover
the W rows once, so the kernel computes out[i] = np.sum(x[i, :]) and touches nothing else; the
group shape is not observable (doc/langref.md:694-697) and the GPU kernel re-tiles.

Two decorations are part of the class: the rows squared before the sum (`rows * rows` or
`rows ** 2`) and `np.sqrt` of the sum -- sums of squares and row norms. The body is matched
statement by statement against exactly these forms (temporaries may be named freely); anything
else, `max` and `min` reductions included, is refused with a diagnostic. The arithmetic is float32
with one rounding per operation and the additions in the order of NumPy's float32 sum, which the
CUDA kernel reproduces (lib/Kernels/row_reduce_sm100a.cu), so results are bit-identical to the
simulator's.
"""

from __future__ import annotations

import ast
import copy
import inspect
from dataclasses import dataclass
from typing import Any

__all__ = ["RowSumContract", "recognise_row_sum"]


@dataclass(frozen=True)
class RowSumContract:
    """What the recogniser established about a row-sum kernel."""

    kernel_name: str
    in_param: str         # Buffer[W, H]
    out_param: str        # Buffer[W]
    extents: tuple        # (W, H): symbol names or fixed integers
    group_rows: int       # G of the kernel as written (not observable on the GPU)
    square: bool          # every value multiplied by itself before the sum
    take_sqrt: bool       # np.sqrt of the sum
    dtype: str = "float32"


def recognise_row_sum(kernel_fn: Any) -> tuple[RowSumContract | None, list[str]]:
    """Decides whether `kernel_fn` is a row-sum kernel. Returns (contract, diagnostics)."""
    from ._map_kernels import _evaluate
    from ._pairwise_kernels import _Substitute, _dim_key, _dump
    from ._pipeline import _function_node, _without_docstring, resolved_annotations

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
    if len(params) != 3:
        return refuse(f"a row-sum kernel takes (group, x, out); found {len(params)} parameters")
    group = params[0]
    annotations = resolved_annotations(kernel_fn)
    dims: dict[str, tuple] = {}
    for param in params[1:]:
        spec = annotations.get(param)
        if type(spec).__name__ != "BufferSpec" or len(spec.dimensions) not in (1, 2):
            return refuse(f"parameter `{param}` must be annotated as a rank-1 or rank-2 Buffer")
        keys = tuple(_dim_key(d) for d in spec.dimensions)
        if None in keys:
            return refuse(f"the extents of `{param}` must be symbols or integers")
        if spec.dtype not in (None, "float32"):
            return refuse(f"`{param}` is Buffer[..., {spec.dtype}]; this target runs row sums on float32")
        dims[param] = keys

    work, group_shape = meta.work_shape, meta.group_shape
    work = work if isinstance(work, tuple) else (work,)
    group_shape = group_shape if isinstance(group_shape, tuple) else (group_shape,)
    if len(work) != 1 or len(group_shape) != 1:
        return refuse("work_shape and group_shape of a row-sum kernel must have one axis")
    group_rows = _evaluate(group_shape[0], {})
    if group_rows is None or group_rows <= 0:
        return refuse("group_shape must be a positive constant")

    fn_node = _function_node(kernel_fn)
    if fn_node is None:
        return refuse("kernel source is unavailable, so its body cannot be checked")
    body = _without_docstring(list(fn_node.body))
    if body and isinstance(body[-1], ast.Return) and (body[-1].value is None or (
            isinstance(body[-1].value, ast.Constant) and body[-1].value.value is None)):
        body = body[:-1]

    whole_offset: set[str] = set()   # names bound to group.work_offset
    row_offset: set[str] = set()     # names bound to group.work_offset[0]
    loaded: dict[str, str] = {}      # name -> buffer parameter whose rows it holds
    temporaries: dict[str, ast.AST] = {}
    stored: tuple[str, ast.AST] | None = None

    def is_work_offset(node: ast.AST) -> bool:
        return (isinstance(node, ast.Attribute) and node.attr == "work_offset" and isinstance(node.value, ast.Name)
                and node.value.id == group)

    def is_row_offset(node: ast.AST | None) -> bool:
        """`group.work_offset[0]`, `gid[0]` with gid = group.work_offset, or a name bound to one of them."""
        if isinstance(node, ast.Name):
            return node.id in row_offset
        if (isinstance(node, ast.Subscript) and isinstance(node.slice, ast.Constant) and node.slice.value == 0
                and not isinstance(node.slice.value, bool)):
            base = node.value
            return is_work_offset(base) or (isinstance(base, ast.Name) and base.id in whole_offset)
        return False

    def open_row_slice(part: ast.AST) -> bool:
        return isinstance(part, ast.Slice) and part.upper is None and part.step is None and is_row_offset(part.lower)

    for stmt in body:
        text = ast.unparse(stmt)
        if stored is not None:
            return refuse(f"`{text}` follows the store; a row-sum kernel ends with it")
        target = (stmt.targets[0].id if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1
                  and isinstance(stmt.targets[0], ast.Name) else None)
        value = stmt.value if isinstance(stmt, (ast.Assign, ast.Expr)) else None
        if target and value is not None and is_work_offset(value):
            whole_offset.add(target)
            continue
        if target and value is not None and not isinstance(value, ast.Name) and is_row_offset(value):
            row_offset.add(target)
            continue
        call = value if isinstance(value, ast.Call) else None
        func = call.func if call is not None else None
        on_group = isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name) and func.value.id == group
        if target and on_group and func.attr == "load":
            window = call.args[0] if len(call.args) == 1 else None
            keywords = {kw.arg: kw.value for kw in call.keywords}
            ok = (isinstance(window, ast.Subscript) and isinstance(window.value, ast.Name)
                  and window.value.id in params[1:] and set(keywords) == {"shape"} and open_row_slice(window.slice))
            shape = keywords.get("shape")
            if ok and isinstance(shape, ast.Tuple) and len(shape.elts) == 2:
                rows_text, cols_text = (ast.unparse(e) for e in shape.elts)
                ok = (rows_text in (f"{group}.shape[0]", str(group_rows))
                      and cols_text == f"{window.value.id}.shape[1]")
            else:
                ok = False
            if not ok:
                return refuse(f"`{text}` must load the group's rows of the buffer, `{group}.load(x[r0:], "
                              f"shape=({group}.shape[0], x.shape[1]))` with r0 = {group}.work_offset[0]")
            loaded[target] = window.value.id
            continue
        if isinstance(stmt, ast.Expr) and on_group and func.attr == "store" and len(call.args) == 2 and not call.keywords:
            window = call.args[0]
            if not (isinstance(window, ast.Subscript) and isinstance(window.value, ast.Name)
                    and window.value.id in params[1:] and open_row_slice(window.slice)):
                return refuse(f"`{text}` must store to the group's own window, `{group}.store(out[r0:], sums)`")
            stored = (window.value.id, call.args[1])
            continue
        if target and value is not None:
            temporaries[target] = _Substitute(temporaries).visit(copy.deepcopy(value))
            continue
        return refuse(f"`{text}` is not part of the load / row sum / store form")

    if stored is None:
        return refuse(f"the kernel must end with `{group}.store(out[r0:], sums)`")
    out_param, expression = stored
    expression = _Substitute(temporaries).visit(copy.deepcopy(expression))
    dumped = ast.dump(expression)
    found: tuple[str, bool, bool] | None = None
    for rows in loaded:
        for square, operand in ((False, rows), (True, f"({rows} * {rows})"), (True, f"({rows} ** 2)")):
            for axis in ("1", "-1"):
                summed = f"{operand}.sum(axis={axis})"
                if dumped == _dump(summed):
                    found = (rows, square, False)
                for module in ("np", "numpy"):
                    if dumped == _dump(f"{module}.sqrt({summed})"):
                        found = (rows, square, True)
    if found is None:
        return refuse(f"`{ast.unparse(expression)}` is not `rows.sum(axis=1)`, `(rows * rows).sum(axis=1)` or "
                      f"`np.sqrt(...)` of one of them, for the rows the kernel loaded (other reductions are not run "
                      f"by this target)")
    in_param = loaded[found[0]]
    if in_param == out_param:
        return refuse("x and out must be two different buffers")
    if len(dims[in_param]) != 2 or len(dims[out_param]) != 1:
        return refuse(f"`{in_param}` must be a rank-2 Buffer and `{out_param}` a rank-1 Buffer")
    (w, h), (o,) = dims[in_param], dims[out_param]
    if o != w:
        return refuse(f"`{out_param}` must be Buffer[{w}] (found Buffer[{o}])")
    # work_shape == (W,): one workitem per row.
    for probe in (1, 5, 4096, 1000003):
        names = {w: probe} if isinstance(w, str) else {}
        want = probe if isinstance(w, str) else w
        if _evaluate(work[0], names) != want:
            return refuse(f"work_shape must be the extent of `{out_param}`, one workitem per row (it evaluates to "
                          f"{_evaluate(work[0], names)} for an extent of {want})")
    return RowSumContract(kernel_name=name, in_param=in_param, out_param=out_param, extents=(w, h),
                          group_rows=int(group_rows), square=found[1], take_sqrt=found[2]), []
