"""Compilation targets of `hc.compile`, and the NVIDIA sm_100a target's kernel recogniser.

In the reference, `hc/_pipeline.py` drives an MLIR transform schedule that lowers the
frontend IR to the `hc` dialect and stops there (run_front_to_hc, hc/_pipeline.py:62-113);
no target can execute anything. Here the module keeps that role -- "turn a decorated kernel
into something a handle can carry" -- for targets that need no MLIR. One target exists:

    "nvidia-sm100a"   maps the tiled WMMA matmul kernel family (this module) and the masked
                      element-wise map (hc._map_kernels) onto the hand-written B200 kernels
                      behind include/hc-c/Cuda.h.

The target does not translate Python to device code. It recognises the kernel: from the
`@kernel` metadata (launch geometry), the `Buffer` annotations (operand roles, extents,
element types), the WMMA intrinsic reachable from the kernel body and its type contract
(`hc._intrinsic_contracts`), and the shape of the body's k-loop, it establishes that the
kernel computes C[M,N] = A[M,K] @ B[K,N] with fp32 accumulation over zero-filled edge
tiles (the contract of examples/amdgpu_gfx11_wmma_matmul.py:301-326). The tile
distribution the kernel spells out (one wave per 16x16 tile, 8 accumulator values per lane)
is, per the language reference, not observable (doc/langref.md:694-697); the plan records it
and the CUDA kernels re-tile to 128x256 CTA tiles with the accumulator in tensor memory.

A kernel that does not match is not an error at compile time: as with a failed MLIR
pipeline in the reference (hc/_pipeline.py:100-108) the handle carries diagnostics and
refuses to launch.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass
from pathlib import Path
from types import FunctionType
from typing import Any

import numpy as np

from ._intrinsic_contracts import serialize_intrinsic_type_spec

__all__ = [
    "NVIDIA_SM100A",
    "GemmContract",
    "LoweringContext",
    "ScheduleSource",
    "TargetResult",
    "known_targets",
    "lower_for_target",
    "recognise_tiled_matmul",
]

ScheduleSource = Path | str | None

NVIDIA_SM100A = "nvidia-sm100a"
_SUPPORTED_INPUT_DTYPES = ("float16", "bfloat16", "float8_e4m3fn", "float8_e5m2")
_SUPPORTED_OUTPUT_DTYPES = ("float32", "float16", "bfloat16")
_PROBE_SHAPES = ((1, 1, 1), (16, 16, 16), (17, 19, 18), (64, 48, 80), (4095, 3073, 1031))


@dataclass(frozen=True)
class GemmContract:
    """What the recogniser established about a kernel."""

    kernel_name: str
    a_param: str
    b_param: str
    c_param: str
    m_dim: Any  # symbol name (str) or fixed int extent
    n_dim: Any
    k_dim: Any
    input_dtype: str  # "float16" | "bfloat16"
    output_dtype: str  # "float32", or "float16" / "bfloat16": the float32 result rounded on store
    tile: tuple[int, int, int]  # WMMA tile (m, n, k) of the kernel as written
    wave_size: int
    accumulators_per_lane: int
    intrinsic_name: str
    intrinsic_const_attrs: tuple[str, ...]
    has_target_lowering: bool  # intrinsic registered `.lower(target="nvidia-sm100a")`
    # What that lowering hook returned (a mapping; see `_run_lowering_hook`), or None.
    lowering: Any = None
    # True when the kernel's b is Buffer[N, K] (B stored transposed) and its k-loop loads
    # b[cols, k0:k0+tk] windows, with the intrinsic's B tile shaped (tn, tk).
    b_transposed: bool = False
    # True when the accumulators are loaded from `c` before the k-loop: C = C + A.B.
    accumulate: bool = False
    # Element-wise statements between the k-loop and the store, in order, as the launcher takes
    # them: ("scale", x), ("add", x), ("max", x), ("min", x), ("bias",).
    epilogue: tuple[tuple, ...] = ()
    # The rank-1 `Buffer[N, float32]` parameter that ("bias",) adds per column, if any.
    bias_param: str | None = None


@dataclass(frozen=True)
class TargetResult:
    target: str
    # GemmContract, hc._map_kernels.MapContract, hc._pairwise_kernels.PairwiseContract,
    # hc._reduce_kernels.RowSumContract, or None
    plan: Any
    diagnostics: tuple[str, ...]


def known_targets() -> tuple[str, ...]:
    return (NVIDIA_SM100A,)


def lower_for_target(kernel_fn: Any, target: str) -> TargetResult:
    """Tries the kernel classes the target runs: the tiled matmul family, then the masked
    element-wise map (`hc._map_kernels`), pairwise distances (`hc._pairwise_kernels`) and row sums
    (`hc._reduce_kernels`). The diagnostics of the class the kernel's signature points at are
    reported when none matches."""
    if target != NVIDIA_SM100A:
        raise ValueError(f"unknown hc.compile target {target!r}; known targets: {list(known_targets())}")
    from ._map_kernels import recognise_elementwise_map
    from ._pairwise_kernels import recognise_pairwise
    from ._reduce_kernels import recognise_row_sum

    plan, diagnostics = recognise_tiled_matmul(kernel_fn)
    if plan is None:
        map_plan, map_diagnostics = recognise_elementwise_map(kernel_fn)
        if map_plan is not None:
            return TargetResult(target, map_plan, ())
        pair_plan, pair_diagnostics = recognise_pairwise(kernel_fn)
        if pair_plan is not None:
            return TargetResult(target, pair_plan, ())
        row_plan, row_diagnostics = recognise_row_sum(kernel_fn)
        if row_plan is not None:
            return TargetResult(target, row_plan, ())
        if _looks_one_dimensional(kernel_fn):
            diagnostics = row_diagnostics if _reduces_without_loop(kernel_fn, 3) else map_diagnostics
        elif _looks_like_pairwise(kernel_fn):
            diagnostics = pair_diagnostics
    return TargetResult(target, plan, tuple(diagnostics))


def _looks_like_pairwise(kernel_fn: Any) -> bool:
    """Three buffers, no k-loop and a reduction of a value (`.sum(...)`): not a member of the matmul family."""
    return _reduces_without_loop(kernel_fn, 4)


def _reduces_without_loop(kernel_fn: Any, parameter_count: int) -> bool:
    """`parameter_count` parameters (the group included), no loop and a reduction of a value
    (`.sum(...)`, `.max(...)`, `.min(...)`)."""
    source = _function_node(kernel_fn)
    if source is None:
        return False
    nodes = list(ast.walk(source))
    has_loop = any(isinstance(node, (ast.For, ast.While)) for node in nodes)
    reduces = any(isinstance(node, ast.Attribute) and node.attr in ("sum", "max", "min") for node in nodes)
    try:
        count = len(inspect.signature(kernel_fn).parameters)
    except (TypeError, ValueError):
        return False
    return count == parameter_count and reduces and not has_loop


def _looks_one_dimensional(kernel_fn: Any) -> bool:
    work = getattr(getattr(kernel_fn, "__hc_kernel__", None), "work_shape", None)
    return not isinstance(work, tuple) or len(work) == 1


# ------------------------------------------------------------------ helpers -------------


def _dim_key(dim: Any) -> Any:
    """Symbol -> its name; integer extent -> int; anything else -> None."""
    if isinstance(dim, bool):
        return None
    if isinstance(dim, int):
        return int(dim)
    name = getattr(dim, "name", None)
    if isinstance(name, str) and hasattr(dim, "free_symbols"):
        return name
    return None


def resolved_annotations(fn: Any) -> dict[str, Any]:
    """Parameter annotations with string forms evaluated in the function's own scope."""
    raw = inspect.get_annotations(fn, eval_str=False)
    if not any(isinstance(value, str) for value in raw.values()):
        return dict(raw)
    scope = dict(getattr(fn, "__globals__", {}))
    try:
        scope.update(inspect.getclosurevars(fn).nonlocals)
    except (TypeError, ValueError):
        pass
    out = {}
    for name, value in raw.items():
        if isinstance(value, str):
            try:
                value = eval(value, scope)  # noqa: S307 - annotations of a user's own kernel
            except Exception:
                value = None
        out[name] = value
    return out


def _reachable_callables(kernel_fn: Any) -> list[Any]:
    """The kernel plus every function it can reach through globals and closure cells.

    Same idea as the reference resolver's dependency walk (hc/_resolve.py:154-189): follow
    names used by a function's code into its globals and closure, and keep going through
    anything that is itself a Python function (decorated helper, intrinsic, or plain
    inline helper).
    """
    seen: dict[int, Any] = {}
    todo = [kernel_fn]
    while todo:
        fn = todo.pop()
        if id(fn) in seen or not isinstance(fn, FunctionType):
            continue
        seen[id(fn)] = fn
        names: set[str] = set()
        codes = [fn.__code__]
        while codes:
            code = codes.pop()
            names.update(code.co_names)
            codes.extend(const for const in code.co_consts if inspect.iscode(const))
        for name in names:
            value = fn.__globals__.get(name)
            if isinstance(value, FunctionType):
                todo.append(value)
        for cell in fn.__closure__ or ():
            try:
                value = cell.cell_contents
            except ValueError:
                continue
            if isinstance(value, FunctionType):
                todo.append(value)
    return list(seen.values())


def _scope_name(scope: Any) -> str:
    return getattr(scope, "__name__", None) or str(scope)


def _int_shape(record: dict[str, object]) -> tuple[int, ...] | None:
    try:
        return tuple(int(extent) for extent in record["shape"])  # type: ignore[union-attr]
    except (KeyError, TypeError, ValueError):
        return None


def _match_mma_contract(fn: Any, input_dtype: str, b_transposed: bool = False) -> tuple[tuple[int, int, int], int] | str:
    """Returns ((tm, tn, tk), accumulators per lane) or a text saying why it does not match."""
    meta = fn.__hc_intrinsic__
    if _scope_name(meta.scope) != "WorkItem":
        return f"scope is {_scope_name(meta.scope)}, expected WorkItem"
    if meta.effects != "pure":
        return f"effects is {meta.effects!r}, expected 'pure'"
    if meta.operand_types is None or len(meta.result_types) != 1:
        return "needs operand_types and exactly one result type"
    try:
        operands = [serialize_intrinsic_type_spec(spec) for spec in meta.operand_types]
        result = serialize_intrinsic_type_spec(meta.result_types[0])
    except RuntimeError as exc:
        return str(exc)
    kinds = [record["kind"] for record in operands]
    if kinds != ["undef", "tensor", "tensor", "vector", "vector", "vector", "idx"]:
        return f"operand kinds {kinds} are not (group, A tile, B tile, A frag, B frag, acc, lane)"
    a_tile, b_tile, a_frag, b_frag, acc = operands[1:6]
    shapes = [_int_shape(record) for record in (a_tile, b_tile, a_frag, b_frag, acc, result)]
    if any(shape is None for shape in shapes):
        return "tile and fragment shapes must be integer literals"
    sa, sb, sfa, sfb, sacc, sres = shapes
    if b_transposed:
        sb = (sb[1], sb[0]) if len(sb) == 2 else sb  # the B tile is declared (tn, tk)
    if len(sa) != 2 or len(sb) != 2 or sa[1] != sb[0]:
        return f"tile shapes {sa} x {sb} do not chain"
    tm, tk, tn = sa[0], sa[1], sb[1]
    if sfa != (tk,) or sfb != (tk,):
        return "lane fragments must be vectors of the tile's k extent"
    if any(record["dtype"] != input_dtype for record in (a_tile, b_tile, a_frag, b_frag)):
        return f"tile/fragment dtypes must all be {input_dtype}"
    if acc != result or acc["dtype"] != "float32" or len(sacc) != 1:
        return "accumulator and result must be the same float32 vector"
    return (tm, tn, tk), sacc[0]


def _evaluate(expr: Any, names: dict[str, int]) -> int | None:
    if isinstance(expr, bool):
        return None
    if isinstance(expr, int):
        return int(expr)
    evaluate = getattr(expr, "eval", None)
    if evaluate is None:
        return None
    try:
        return int(evaluate(names))
    except Exception:
        return None


def _check_geometry(meta: Any, dims: dict[str, Any], tile: tuple[int, int, int],
                    acc_len: int) -> tuple[int, list[str]]:
    """Checks work/group shape against one-wave-per-tile. Returns (wave size, problems)."""
    problems: list[str] = []
    tm, tn, _ = tile
    work, group = meta.work_shape, meta.group_shape
    if not isinstance(work, tuple) or len(work) != 2:
        return 0, ["work_shape must be a pair (tile rows x lanes, tile columns)"]
    if not isinstance(group, tuple) or len(group) != 2:
        return 0, ["group_shape must be a pair (lanes, 1)"]
    wave = _evaluate(group[0], {})
    if wave is None or wave <= 0 or _evaluate(group[1], {}) != 1:
        return 0, ["group_shape must be (wave size, 1) with a constant wave size"]
    subgroup = meta.subgroup_size
    if subgroup is not None and _evaluate(subgroup, {}) != wave:
        problems.append("subgroup_size must equal the wave size")
    if tm * tn != acc_len * wave:
        problems.append(
            f"a {tm}x{tn} tile over {wave} lanes needs {tm * tn // max(wave, 1)} accumulator values per "
            f"lane, the intrinsic carries {acc_len}")
    for m, n, k in _PROBE_SHAPES:
        names = {}
        for key, value in (("m", m), ("n", n), ("k", k)):
            if isinstance(dims[key], str):
                names[dims[key]] = value
        mm = m if isinstance(dims["m"], str) else dims["m"]
        nn = n if isinstance(dims["n"], str) else dims["n"]
        want = (-(-mm // tm) * wave, -(-nn // tn))
        got = (_evaluate(work[0], names), _evaluate(work[1], names))
        if got != want:
            problems.append(
                f"work_shape evaluates to {got} for M={mm}, N={nn}; one wave of {wave} per "
                f"{tm}x{tn} tile needs {want}")
            break
    return wave, problems


def _names_in(node: ast.AST | None) -> set[str]:
    return {n.id for n in ast.walk(node) if isinstance(n, ast.Name)} if node is not None else set()


_MAX_EPILOGUE_OPS = 4

# ---- integer index expressions as affine forms ------------------------------------------------
#
# Tile origins and window bounds are integer expressions over `group.group_id[0]`,
# `group.group_id[1]` and the k-loop variable. They are evaluated to affine forms
# {symbol: coefficient} ("1" is the constant term), so that `row0 : row0 + 16` with
# `row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])` can be compared with what a
# matmul tile needs, whatever the spelling (a helper returning a tuple, two assignments, the
# products written inline).

_GID0, _GID1, _KVAR, _ONE = "group_id[0]", "group_id[1]", "k", "1"
Affine = dict


def _affine_const(value: int) -> Affine:
    return {_ONE: int(value)} if value else {}


def _affine_add(x: Affine, y: Affine, sign: int = 1) -> Affine:
    out = dict(x)
    for key, coeff in y.items():
        out[key] = out.get(key, 0) + sign * coeff
    return {key: coeff for key, coeff in out.items() if coeff}


def _affine_mul(x: Affine, y: Affine) -> Affine | None:
    for scalar, other in ((x, y), (y, x)):
        if set(scalar) <= {_ONE}:
            factor = scalar.get(_ONE, 0)
            return {key: coeff * factor for key, coeff in other.items() if coeff * factor}
    return None


def _affine_text(x: Affine) -> str:
    if not x:
        return "0"
    parts = []
    for key, coeff in sorted(x.items(), key=lambda item: item[0] == _ONE):
        parts.append(str(coeff) if key == _ONE else (key if coeff == 1 else f"{coeff}*{key}"))
    return " + ".join(parts)


def _function_consts(fn: Any) -> dict[str, Any]:
    consts = dict(getattr(fn, "__globals__", {}))
    try:
        consts.update(inspect.getclosurevars(fn).nonlocals)
    except (TypeError, ValueError):
        pass
    return consts


def _function_node(fn: Any) -> ast.FunctionDef | None:
    try:
        tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    except (OSError, TypeError, SyntaxError, IndentationError):
        return None
    return next((n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef))), None)


def _without_docstring(body: list[ast.stmt]) -> list[ast.stmt]:
    if body and isinstance(body[0], ast.Expr) and isinstance(body[0].value, ast.Constant) \
            and isinstance(body[0].value.value, str):
        return body[1:]
    return body


class _IndexEvaluator:
    """Evaluates integer index expressions of one function body to affine forms."""

    def __init__(self, group: str, consts: dict[str, Any], depth: int = 0) -> None:
        self.group, self.consts, self.depth = group, consts, depth
        self.env: dict[str, Any] = {}  # name -> Affine | tuple of Affine

    def eval(self, node: ast.AST | None) -> Any:
        if isinstance(node, ast.Constant):
            value = node.value
            return _affine_const(value) if isinstance(value, int) and not isinstance(value, bool) else None
        if isinstance(node, ast.Name):
            if node.id in self.env:
                return self.env[node.id]
            value = self.consts.get(node.id)
            if isinstance(value, (int, np.integer)) and not isinstance(value, bool):
                return _affine_const(int(value))
            return None
        if isinstance(node, ast.Tuple):
            parts = tuple(self.eval(elt) for elt in node.elts)
            return None if any(part is None or isinstance(part, tuple) for part in parts) else parts
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)):
            inner = self.eval(node.operand)
            if not isinstance(inner, dict):
                return None
            return _affine_add({}, inner, -1) if isinstance(node.op, ast.USub) else inner
        if isinstance(node, ast.BinOp):
            left, right = self.eval(node.left), self.eval(node.right)
            if not isinstance(left, dict) or not isinstance(right, dict):
                return None
            if isinstance(node.op, ast.Add):
                return _affine_add(left, right)
            if isinstance(node.op, ast.Sub):
                return _affine_add(left, right, -1)
            if isinstance(node.op, ast.Mult):
                return _affine_mul(left, right)
            return None
        if isinstance(node, ast.Subscript):
            index = node.slice
            if not (isinstance(index, ast.Constant) and isinstance(index.value, int)):
                return None
            base = node.value
            if (isinstance(base, ast.Attribute) and base.attr == "group_id" and isinstance(base.value, ast.Name)
                    and base.value.id == self.group and self.group and index.value in (0, 1)):
                return {(_GID0, _GID1)[index.value]: 1}
            whole = self.eval(base)
            if isinstance(whole, tuple) and 0 <= index.value < len(whole):
                return whole[index.value]
            return None
        if isinstance(node, ast.Call):
            return self._inline(node)
        return None

    def _inline(self, node: ast.Call) -> Any:
        """A call of a plain Python helper whose body is one `return <index expression>`."""
        if node.keywords or not isinstance(node.func, ast.Name) or self.depth >= 4:
            return None
        fn = self.consts.get(node.func.id)
        if not isinstance(fn, FunctionType):
            return None
        args = [self.eval(arg) for arg in node.args]
        if any(not isinstance(arg, dict) for arg in args):
            return None
        fn_node = _function_node(fn)
        if fn_node is None:
            return None
        spec = fn_node.args
        if spec.vararg or spec.kwarg or spec.kwonlyargs or spec.defaults or len(spec.args) != len(args):
            return None
        body = _without_docstring(list(fn_node.body))
        if len(body) != 1 or not isinstance(body[0], ast.Return):
            return None
        inner = _IndexEvaluator("", _function_consts(fn), self.depth + 1)
        inner.env = {param.arg: arg for param, arg in zip(spec.args, args)}
        return inner.eval(body[0].value)

    def assign(self, stmt: ast.Assign) -> bool:
        """Binds the targets of an index assignment; False if it is not one."""
        if len(stmt.targets) != 1:
            return False
        target, value = stmt.targets[0], self.eval(stmt.value)
        if isinstance(target, ast.Name) and isinstance(value, dict):
            self.env[target.id] = value
            return True
        if (isinstance(target, ast.Tuple) and isinstance(value, tuple) and len(target.elts) == len(value)
                and all(isinstance(elt, ast.Name) for elt in target.elts)):
            for elt, part in zip(target.elts, value):
                self.env[elt.id] = part
            return True
        return False


_FORBIDDEN_IN_HELPERS = (ast.If, ast.While, ast.For, ast.Try, ast.With, ast.IfExp, ast.Lambda, ast.Global,
                         ast.Nonlocal, ast.Match, ast.ListComp, ast.SetComp, ast.DictComp, ast.GeneratorExp)


def _helper_is_straight_line(fn: Any) -> str | None:
    """The workgroup helpers are validated by running them on probe workgroups (`hc._tile_probe`);
    that only means something for code without branches or loops of its own."""
    fn_node = _function_node(fn)
    if fn_node is None:
        return f"source of helper `{getattr(fn, '__name__', fn)}` is unavailable"
    for node in ast.walk(fn_node):
        if isinstance(node, _FORBIDDEN_IN_HELPERS):
            return (f"helper `{fn.__name__}` contains a `{type(node).__name__}` statement or expression; helpers "
                    f"around the intrinsic must be straight-line code")
    return None


def _check_body(kernel_fn: Any, params: list[str], a: str, b: str, c: str, tile: tuple[int, int, int],
                k_dim: Any, b_transposed: bool = False, bias: str | None = None,
                facts: dict[str, Any] | None = None, output_dtype: str = "float32") -> list[str]:
    """Checks that the kernel body is, statement for statement, the tiled matmul of
    examples/amdgpu_gfx11_wmma_matmul.py:312-326 (or a member of its family):

        row0, col0 = <index expressions equal to group.group_id[0] * tm, group.group_id[1] * tn>
        acc = <init helper>(group[, c, row0, col0])
        for k0 in range(0, K, tk):
            a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + tk], shape=(tm, tk))
            b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))   # or b[cols, ks]
            acc = <step helper>(group, a_tile, b_tile, acc)
        acc = <element-wise statement>            # zero or more
        <store helper>(group, c, row0, col0, acc)

    and nothing else. Returns problems (empty when the body has that form).

    `facts` receives "accumulate", "epilogue" and "calls": the helper calls with their arguments
    classified, for the probe that validates what the helpers do (`hc._tile_probe`)."""
    fn_node = _function_node(kernel_fn)
    if fn_node is None:
        return ["kernel source is unavailable, so its body cannot be checked"]
    consts = _function_consts(kernel_fn)
    group = params[0]
    tm, tn, tk = tile

    def const_value(node: ast.AST | None) -> Any:
        if isinstance(node, ast.Constant):
            return node.value
        if isinstance(node, ast.Name):
            return consts.get(node.id)
        return None

    body = _without_docstring(list(fn_node.body))
    loops = [stmt for stmt in body if isinstance(stmt, ast.For)]
    nested = [n for stmt in body for n in ast.walk(stmt) if isinstance(n, (ast.For, ast.While)) and n not in loops]
    if len(loops) != 1 or nested:
        return [f"expected exactly one k-loop in the kernel body, found {len(loops) + len(nested)}"
                if len(loops) + len(nested) != 1 else "the k-loop must be a top-level statement of the kernel body"]
    loop = loops[0]
    at = body.index(loop)
    problems: list[str] = []

    # -- the loop header ---------------------------------------------------------------------
    it = loop.iter
    ok_range = (isinstance(it, ast.Call) and isinstance(it.func, ast.Name) and it.func.id == "range"
                and not it.keywords and len(it.args) == 3 and const_value(it.args[0]) == 0
                and const_value(it.args[2]) == tk and isinstance(loop.target, ast.Name) and not loop.orelse)
    if not ok_range:
        return [f"k-loop must be `for k0 in range(0, K, {tk})`"]
    stop = it.args[1]
    # K may be spelled `a.shape[1]`, `b.shape[0]` or as the K symbol / literal itself.
    spelled = ast.unparse(stop).replace(" ", "")
    k_names = {f"{a}.shape[1]", f"{b}.shape[1]" if b_transposed else f"{b}.shape[0]"}
    if isinstance(k_dim, str):
        k_names.add(k_dim)
    if spelled not in k_names and const_value(stop) != k_dim:
        problems.append(f"k-loop bound `{ast.unparse(stop)}` is not the shared extent of {a} and {b}")
    k_var = loop.target.id

    # -- the accumulator variable: `acc = f(..., acc)` closes the loop body --------------------
    def plain_call(node: ast.AST | None) -> ast.Call | None:
        ok = (isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and not node.keywords
              and not any(isinstance(arg, ast.Starred) for arg in node.args))
        return node if ok else None

    def single_name_target(stmt: ast.stmt) -> str | None:
        if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name):
            return stmt.targets[0].id
        return None

    acc = None
    for stmt in loop.body:
        name = single_name_target(stmt)
        call = plain_call(stmt.value) if name else None
        if call is not None and any(isinstance(arg, ast.Name) and arg.id == name for arg in call.args):
            acc = name
    if acc is None:
        return problems + ["the k-loop must update the accumulators as `acc = f(group, a_tile, b_tile, acc)`"]

    # -- before the loop: tile origins, then the accumulator initialiser -----------------------
    index = _IndexEvaluator(group, consts)
    row_origin, col_origin = {_GID0: tm}, {_GID1: tn}
    calls: dict[str, Any] = {}

    def classify(call: ast.Call, what: str, tiles: dict[str, str]) -> tuple[tuple, ...] | None:
        """The arguments of a helper call as the probe takes them, or None (problem recorded)."""
        kinds: list[tuple] = []
        for arg in call.args:
            if isinstance(arg, ast.Name) and arg.id == group:
                kinds.append(("group",))
            elif isinstance(arg, ast.Name) and arg.id == c:
                kinds.append(("c",))
            elif isinstance(arg, ast.Name) and arg.id == acc:
                kinds.append(("acc",))
            elif isinstance(arg, ast.Name) and bias is not None and arg.id == bias:
                kinds.append(("bias",))
            elif isinstance(arg, ast.Name) and arg.id in tiles:
                kinds.append((tiles[arg.id],))
            else:
                value = index.eval(arg)
                if value == row_origin:
                    kinds.append(("origin", lambda g0, g1: g0 * tm))
                elif value == col_origin:
                    kinds.append(("origin", lambda g0, g1: g1 * tn))
                else:
                    found = _affine_text(value) if isinstance(value, dict) else "not an index expression"
                    problems.append(
                        f"argument `{ast.unparse(arg)}` of the {what} `{ast.unparse(call)}` must be the group, a "
                        f"buffer, the accumulators, or the tile's row origin ({_affine_text(row_origin)}) or "
                        f"column origin ({_affine_text(col_origin)}); it is {found}")
                    return None
        return tuple(kinds)

    def helper_of(call: ast.Call, what: str) -> Any:
        fn = consts.get(call.func.id)
        if not isinstance(fn, FunctionType):
            problems.append(f"the {what} `{ast.unparse(call)}` must call a helper function defined in Python")
            return None
        why = _helper_is_straight_line(fn)
        if why:
            problems.append(why)
            return None
        return fn

    def helper_call(call: ast.Call, what: str, tiles: dict[str, str] | None = None) -> Any:
        from ._tile_probe import HelperCall

        fn = helper_of(call, what)
        kinds = classify(call, what, tiles or {}) if fn is not None else None
        return None if fn is None or kinds is None else HelperCall(fn, kinds, ast.unparse(call))

    accumulate = False
    initialised = False
    for stmt in body[:at]:
        text = ast.unparse(stmt)
        if single_name_target(stmt) == acc:
            call = plain_call(stmt.value)
            if call is None or initialised:
                problems.append(f"`{text}`: the accumulators must be initialised once, by a call such as "
                                f"`{acc} = zero_accumulators({group})` or `{acc} = load_accumulators({group}, {c}, "
                                f"row0, col0)`")
                continue
            initialised = True
            calls["init"] = helper_call(call, "accumulator initialiser")
            kinds = calls["init"].args if calls["init"] is not None else ()
            accumulate = ("c",) in kinds
            if ("acc",) in kinds or ("bias",) in kinds:
                problems.append(f"`{text}`: the accumulator initialiser may only receive the group, `{c}` and "
                                f"the tile origin")
        elif initialised or not (isinstance(stmt, ast.Assign) and index.assign(stmt)):
            problems.append(f"`{text}` before the k-loop is neither a tile-origin assignment (an integer "
                            f"expression over {group}.group_id) nor the accumulator initialiser")
    if not initialised:
        problems.append(f"`{acc}` must be initialised before the k-loop")
    if accumulate and output_dtype != "float32":
        problems.append(f"a kernel that loads its accumulators from `{c}` needs a float32 `{c}` (got {output_dtype})")

    # -- the loop body: one window of a, one of b, one step -----------------------------------
    index.env[k_var] = {_KVAR: 1}
    tiles: dict[str, str] = {}
    b_axes = (1, 0) if b_transposed else (0, 1)  # (k axis, n axis) of b as stored
    wanted = {
        a: ("a_tile", ((row_origin, tm, "rows", f"{group}.group_id[0] * {tm}"), ({_KVAR: 1}, tk, "columns", k_var))),
        b: ("b_tile", tuple(
            ({_KVAR: 1}, tk, "rows" if axis == 0 else "columns", k_var) if axis == b_axes[0]
            else (col_origin, tn, "rows" if axis == 0 else "columns", f"{group}.group_id[1] * {tn}")
            for axis in (0, 1))),
    }
    step_stmt = None
    for stmt in loop.body:
        text = ast.unparse(stmt)
        name = single_name_target(stmt)
        if name == acc and step_stmt is None and plain_call(stmt.value) is not None:
            step_stmt = stmt
            continue
        load = stmt.value if name and isinstance(stmt.value, ast.Call) else None
        func = load.func if load is not None else None
        is_load = (isinstance(func, ast.Attribute) and func.attr == "load" and isinstance(func.value, ast.Name)
                   and func.value.id == group and len(load.args) == 1
                   and isinstance(load.args[0], ast.Subscript) and isinstance(load.args[0].value, ast.Name)
                   and load.args[0].value.id in wanted)
        if not is_load or step_stmt is not None:
            problems.append(f"`{text}` in the k-loop is not one of: a `{group}.load` of a window of `{a}`, one of "
                            f"`{b}`, then `{acc} = f({group}, a_tile, b_tile, {acc})`")
            continue
        source = load.args[0]
        buffer = source.value.id
        role, axes = wanted[buffer]
        if role in tiles.values():
            problems.append(f"expected one group.load of a window of `{buffer}` per k-step, found another: `{text}`")
            continue
        tiles[name] = role
        parts = list(source.slice.elts) if isinstance(source.slice, ast.Tuple) else [source.slice]
        if len(parts) != 2 or not all(isinstance(p, ast.Slice) and p.step is None for p in parts):
            problems.append(f"the load of `{buffer}` must slice both axes as `lo:hi`")
            continue
        extents = []
        for axis, (part, (origin, extent, axis_name, origin_text)) in enumerate(zip(parts, axes)):
            lo, hi = index.eval(part.lower), index.eval(part.upper)
            extents.append(extent)
            if lo != origin or not isinstance(hi, dict) or _affine_add(hi, origin, -1) != _affine_const(extent):
                k_axis = origin == {_KVAR: 1}
                found = ast.unparse(part)
                problems.append(
                    f"axis {axis} of the `{buffer}` window must "
                    + (f"advance with the k-loop variable as `{k_var} : {k_var} + {extent}`" if k_axis
                       else f"be the tile's {axis_name} `o : o + {extent}` with o = {origin_text}")
                    + f" (found `{found}`)")
        keywords = {kw.arg: kw.value for kw in load.keywords}
        shape_node = keywords.get("shape")
        shape_ok = (set(keywords) == {"shape"} and isinstance(shape_node, ast.Tuple)
                    and [const_value(elt) for elt in shape_node.elts] == extents)
        if not shape_ok:
            problems.append(f"the load of `{buffer}` must be `{group}.load(<window>, shape={tuple(extents)})` with "
                            f"no other keyword")
    for buffer, (role, _) in wanted.items():
        if role not in tiles.values():
            problems.append(f"expected one group.load of a window of `{buffer}` per k-step, found 0")
    if step_stmt is None:
        problems.append(f"the k-loop must end with `{acc} = f({group}, a_tile, b_tile, {acc})`")
    elif not problems or all(role in tiles.values() for role in ("a_tile", "b_tile")):
        call = plain_call(step_stmt.value)
        calls["step"] = helper_call(call, "multiply-accumulate step", tiles)
        kinds = calls["step"].args if calls["step"] is not None else None
        if kinds is not None and (sorted(k[0] for k in kinds if k[0] != "group") != ["a_tile", "acc", "b_tile"]):
            problems.append(f"`{ast.unparse(step_stmt)}` must receive the two tiles loaded in this k-step and "
                            f"`{acc}`, each once, and nothing else but the group")

    # -- after the loop: element-wise statements, then the store -------------------------------
    ops: list[tuple] = []
    stored = False
    narrowed = False  # the accumulators have been converted to the 16-bit type of `c`
    for stmt in body[at + 1:]:
        text = ast.unparse(stmt)
        if stored:
            problems.append(f"`{text}` follows the store" + (f" and uses `{acc}` after the store"
                                                             if acc in _names_in(stmt) else ""))
            continue
        call = plain_call(stmt.value) if isinstance(stmt, ast.Expr) else None
        if call is not None and any(isinstance(arg, ast.Name) and arg.id == c for arg in call.args):
            stored = True
            calls["store"] = helper_call(call, "store")
            kinds = calls["store"].args if calls["store"] is not None else None
            if kinds is not None and (kinds.count(("c",)) != 1 or kinds.count(("acc",)) != 1 or ("bias",) in kinds):
                problems.append(f"the store `{text}` must receive `{c}` and `{acc}`, each once")
            continue
        ok_target = single_name_target(stmt) == acc
        op = _elementwise_op(stmt.value, acc, bias, const_value) if ok_target else None
        if op is not None and op and op[0] == "astype":
            target = _dtype_name_of(op[1], consts)
            if target == "float32" and not narrowed:
                continue
            if target == output_dtype and target != "float32" and not narrowed:
                narrowed = True
                continue
            op = None
        elif op and narrowed:
            problems.append(f"`{text}` runs on the 16-bit values: element-wise statements must come before "
                            f"`{acc}.astype({output_dtype})`")
            continue
        if op is None:
            problems.append(
                f"`{text}` is not an element-wise statement this target folds into the store "
                f"(`{acc} = {acc} * x`, `+ x`, `- x`, `np.maximum({acc}, x)`, `np.minimum({acc}, x)` with a "
                f"numeric constant x, `{acc} = f(..., bias, ..., {acc})`, `{acc}.astype(<float32 or the dtype of {c}>)`)")
            continue
        if op[0] == "bias":
            if "bias" in calls:
                problems.append(f"`{bias}` must be added to `{acc}` exactly once between the k-loop and the store")
                continue
            calls["bias"] = helper_call(plain_call(stmt.value), "bias addition") if plain_call(stmt.value) else None
            if plain_call(stmt.value) is None:
                problems.append(f"`{text}` must be a plain call `{acc} = f({group}, {bias}, col0, {acc})`")
        ops.append(op)
    if not stored:
        problems.append(f"`{c}` must be passed to a store after the k-loop")
    if len(ops) > _MAX_EPILOGUE_OPS:
        problems.append(f"at most {_MAX_EPILOGUE_OPS} element-wise statements can be folded into the store, "
                        f"found {len(ops)}")
    bias_ops = sum(1 for op in ops if op[0] == "bias")
    if bias is not None and bias_ops != 1 and not any("exactly once" in p for p in problems):
        problems.append(f"`{bias}` must be added to `{acc}` exactly once between the k-loop and the store")
    if facts is not None:
        facts.update({"accumulate": accumulate, "epilogue": tuple(ops), "calls": calls})
    return problems


def _number(node: ast.AST | None, const_value: Any) -> float | None:
    """A numeric constant as the kernel spells it: a literal, a module-level or closure name,
    `np.float32(<that>)`, or a negation of one. The statement runs in fp32, so the value is
    rounded to fp32."""
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)):
        inner = _number(node.operand, const_value)
        if inner is None:
            return None
        return -inner if isinstance(node.op, ast.USub) else inner
    if isinstance(node, ast.Call) and len(node.args) == 1 and not node.keywords:
        func = node.func
        name = func.attr if isinstance(func, ast.Attribute) else (func.id if isinstance(func, ast.Name) else None)
        if name in ("float32", "float64", "float16", "float"):
            return _number(node.args[0], const_value)
        return None
    value = const_value(node)
    if isinstance(value, bool) or not isinstance(value, (int, float, np.integer, np.floating)):
        return None
    value = float(np.float32(value))
    return value if np.isfinite(value) else None


def _dtype_name_of(node: ast.AST, consts: dict[str, Any]) -> str | None:
    """The NumPy dtype name an expression such as `np.float16`, `ml_dtypes.bfloat16` or a closure
    variable holding a scalar type denotes, or None."""
    try:
        if isinstance(node, ast.Name):
            value = consts[node.id]
        elif isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name):
            value = getattr(consts[node.value.id], node.attr)
        elif isinstance(node, ast.Constant) and isinstance(node.value, str):
            value = node.value
        else:
            return None
        return np.dtype(value).name
    except (KeyError, AttributeError, TypeError):
        return None


def _elementwise_op(value: ast.AST, acc: str, bias: str | None, const_value: Any) -> tuple | None:
    """One statement `acc = <value>` as a fused operation; () for a no-op; None if unsupported."""
    def is_acc(node: ast.AST) -> bool:
        return isinstance(node, ast.Name) and node.id == acc

    if isinstance(value, ast.BinOp):
        left, right = value.left, value.right
        if isinstance(value.op, (ast.Mult, ast.Add)) and (is_acc(left) or is_acc(right)):
            x = _number(right if is_acc(left) else left, const_value)
            if x is not None:
                return ("scale" if isinstance(value.op, ast.Mult) else "add", x)
        if isinstance(value.op, ast.Sub) and is_acc(left):
            x = _number(right, const_value)
            if x is not None:
                return ("add", -x)
        return None
    if isinstance(value, ast.Call):
        func = value.func
        name = func.attr if isinstance(func, ast.Attribute) else (func.id if isinstance(func, ast.Name) else None)
        if name in ("maximum", "minimum") and len(value.args) == 2 and not value.keywords:
            first, second = value.args
            if is_acc(first) or is_acc(second):
                x = _number(second if is_acc(first) else first, const_value)
                if x is not None:
                    return ("max" if name == "maximum" else "min", x)
            return None
        if name == "astype" and isinstance(func, ast.Attribute) and is_acc(func.value) and len(value.args) == 1:
            return ("astype", value.args[0])  # resolved by the caller against the dtype of c
        names = {arg.id for arg in value.args if isinstance(arg, ast.Name)}
        if bias is not None and bias in names and acc in names:
            return ("bias",)
    return None


@dataclass(frozen=True)
class LoweringContext:
    """What an intrinsic's `.lower(target="nvidia-sm100a")` hook receives as its first argument.

    In the reference a lowering hook gets a builder context and returns IR values
    (examples/amdgpu_gfx11_wmma_matmul.py:200-228; nothing ever calls those hooks). This target
    does not build IR: the whole k-loop of WMMA steps becomes tcgen05.mma instructions, so the
    hook's role is to describe or steer that mapping. It may return a mapping with any of
        "variant": "auto" | "dense" | "skinny"   which kernel family launches use
    plus free-form descriptive entries, which are kept on the plan.
    """

    target: str
    tile: tuple[int, int, int]
    wave_size: int
    input_dtype: str
    cta_tiles: tuple[tuple[int, int, int], ...] = ((256, 256, 128), (128, 256, 64))
    instruction: str = "tcgen05.mma.kind::f16 (fp32 accumulate in tensor memory)"


_VARIANTS = ("auto", "dense", "skinny")


def _run_lowering_hook(intrinsic: Any, tile: tuple[int, int, int], wave: int, dtype: str) -> tuple[Any, list[str]]:
    hook = (getattr(intrinsic, "__hc_lowerings__", {}) or {}).get(NVIDIA_SM100A)
    if hook is None:
        return None, []
    try:
        result = hook(LoweringContext(NVIDIA_SM100A, tile, wave, dtype))
    except Exception as exc:  # a user's hook must not break compilation
        return None, [f"lowering hook of {intrinsic.__name__} raised {type(exc).__name__}: {exc}"]
    if result is None:
        return None, []
    if not isinstance(result, dict):
        return None, [f"lowering hook of {intrinsic.__name__} must return a mapping or None"]
    variant = result.get("variant", "auto")
    if variant not in _VARIANTS:
        return None, [f"lowering hook of {intrinsic.__name__}: variant must be one of {list(_VARIANTS)}"]
    return dict(result), []


def _probe_helpers(facts: dict[str, Any], tile: tuple[int, int, int], wave: int, acc_len: int,
                   input_dtype: str, b_transposed: bool) -> list[str]:
    """Runs the helper calls `_check_body` classified on probe workgroups (`hc._tile_probe`): the
    initialiser, the step with its intrinsic, the bias addition and the store must together leave
    `(c +) a @ b (+ bias)` in exactly the workgroup's tile of `c`, at interior, edge and corner tiles."""
    from ._tile_probe import probe_helper_chain

    calls = facts.get("calls", {})
    if any(calls.get(key) is None for key in ("init", "step", "store")):
        return ["the kernel's helper calls could not be resolved"]
    if input_dtype == "float16":
        element_type: Any = np.float16
    else:
        import ml_dtypes

        element_type = getattr(ml_dtypes, input_dtype)
    return probe_helper_chain(init=calls["init"], step=calls["step"], store=calls["store"],
                              bias=calls.get("bias"), tile=tile, wave=wave, acc_len=acc_len,
                              input_dtype=element_type, accumulate=bool(facts.get("accumulate")),
                              b_transposed=b_transposed)


# ------------------------------------------------------------------ recogniser ----------


def recognise_tiled_matmul(kernel_fn: Any) -> tuple[GemmContract | None, list[str]]:
    """Decides whether `kernel_fn` is a tiled WMMA matmul the sm_100a kernels implement.

    Returns (contract, diagnostics). `contract` is None when the kernel does not match; the
    diagnostics then say what is missing.
    """
    name = getattr(kernel_fn, "__name__", "<kernel>")
    meta = getattr(kernel_fn, "__hc_kernel__", None)
    if meta is None:
        return None, [f"{name}: not a @kernel function"]
    problems: list[str] = []

    try:
        params = list(inspect.signature(kernel_fn).parameters)
    except (TypeError, ValueError):
        return None, [f"{name}: signature is not inspectable"]
    if len(params) not in (4, 5):
        return None, [f"{name}: expected (group, a, b, c) or (group, a, b, c, bias) parameters, "
                      f"found {len(params)} parameters"]
    annotations = resolved_annotations(kernel_fn)
    specs = []
    vectors = []
    for param in params[1:]:
        spec = annotations.get(param)
        rank = len(getattr(spec, "dimensions", ()))
        if type(spec).__name__ != "BufferSpec" or rank not in (1, 2):
            return None, [f"{name}: parameter `{param}` must be annotated as a rank-2 Buffer"
                          + (" (or the rank-1 bias)" if len(params) == 5 else "")]
        keys = tuple(_dim_key(d) for d in spec.dimensions)
        if None in keys:
            return None, [f"{name}: extents of `{param}` must be symbols or integers"]
        (specs if rank == 2 else vectors).append((param, keys, spec.dtype))
    if len(specs) != 3 or len(vectors) != len(params) - 4:
        return None, [f"{name}: expected three rank-2 buffers (a, b, c)"
                      + (" and one rank-1 bias" if len(params) == 5 else "")
                      + f", found {len(specs)} rank-2 and {len(vectors)} rank-1"]

    # Operand roles from how the extents chain: a[M,K] b[K,N] c[M,N] in any parameter order.
    roles = None
    b_transposed = False
    for ia, ib, ic in ((0, 1, 2), (0, 2, 1), (1, 0, 2), (1, 2, 0), (2, 0, 1), (2, 1, 0)):
        (pa, (am, ak), da), (pb, b_dims, db), (pc, (cm, cn), dc) = specs[ia], specs[ib], specs[ic]
        if not (am == cm and dc in _SUPPORTED_OUTPUT_DTYPES and da == db and da in _SUPPORTED_INPUT_DTYPES):
            continue
        for transposed in (False, True):
            bk, bn = (b_dims[1], b_dims[0]) if transposed else b_dims
            # With m == n == k as fixed equal extents the untransposed reading wins.
            if ak == bk and bn == cn and roles is None:
                roles = (pa, pb, pc, am, bn, ak, da, dc)
                b_transposed = transposed
        if roles is not None and (ia, ib, ic) == (0, 1, 2):
            break
    if roles is None:
        described = ", ".join(f"{p}: Buffer{list(k)} {d}" for p, k, d in specs)
        return None, [
            f"{name}: buffers ({described}) are not a[M,K], b[K,N] (or b[N,K]) of one of "
            f"{list(_SUPPORTED_INPUT_DTYPES)} and c[M,N] of one of {list(_SUPPORTED_OUTPUT_DTYPES)}"
        ]
    a, b, c, m_dim, n_dim, k_dim, input_dtype, output_dtype = roles
    bias = None
    if vectors:
        bias, (bias_dim,), bias_dtype = vectors[0]
        if bias_dim != n_dim or bias_dtype != "float32":
            return None, [f"{name}: `{bias}` must be Buffer[{n_dim}, float32], one value per column of `{c}`"]

    intrinsics = [fn for fn in _reachable_callables(kernel_fn) if hasattr(fn, "__hc_intrinsic__")]
    matches = []
    for fn in intrinsics:
        outcome = _match_mma_contract(fn, input_dtype, b_transposed)
        if isinstance(outcome, str):
            problems.append(f"intrinsic {fn.__name__}: {outcome}")
        else:
            matches.append((fn, outcome))
    if len(matches) != 1:
        if not intrinsics:
            problems.append("no @kernel.intrinsic is reachable from the kernel body")
        elif len(matches) > 1:
            problems.append("more than one matrix-multiply intrinsic is reachable from the kernel body")
        return None, [f"{name}: {p}" for p in problems]
    intrinsic, (tile, acc_len) = matches[0]
    problems = []  # contract mismatches of other intrinsics no longer matter

    wave, geometry_problems = _check_geometry(meta, {"m": m_dim, "n": n_dim, "k": k_dim}, tile, acc_len)
    problems.extend(geometry_problems)
    facts: dict[str, Any] = {}
    problems.extend(_check_body(kernel_fn, params, a, b, c, tile, k_dim, b_transposed, bias, facts, output_dtype))
    if problems:
        return None, [f"{name}: {p}" for p in problems]
    problems.extend(_probe_helpers(facts, tile, wave, acc_len, input_dtype, b_transposed))
    if problems:
        return None, [f"{name}: {p}" for p in problems]

    lowerings = getattr(intrinsic, "__hc_lowerings__", {}) or {}
    lowering, hook_problems = _run_lowering_hook(intrinsic, tile, wave, input_dtype)
    if hook_problems:
        return None, [f"{name}: {p}" for p in hook_problems]
    contract = GemmContract(
        kernel_name=name, a_param=a, b_param=b, c_param=c, m_dim=m_dim, n_dim=n_dim, k_dim=k_dim,
        input_dtype=input_dtype, output_dtype=output_dtype, tile=tile, wave_size=wave,
        accumulators_per_lane=acc_len, intrinsic_name=intrinsic.__name__,
        intrinsic_const_attrs=tuple(sorted(intrinsic.__hc_intrinsic__.const_attrs)),
        has_target_lowering=NVIDIA_SM100A in lowerings,
        lowering=lowering,
        b_transposed=b_transposed,
        accumulate=bool(facts.get("accumulate", False)),
        epilogue=tuple(facts.get("epilogue", ())),
        bias_param=bias,
    )
    return contract, []
