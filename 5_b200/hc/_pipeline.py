"""Compilation targets of `hc.compile`, and the NVIDIA sm_100a target's kernel recogniser.

In the reference, `hc/_pipeline.py` drives an MLIR transform schedule that lowers the
frontend IR to the `hc` dialect and stops there (run_front_to_hc, hc/_pipeline.py:62-113);
no target can execute anything. Here the module keeps that role -- "turn a decorated kernel
into something a handle can carry" -- for targets that need no MLIR. One target exists:

    "nvidia-sm100a"   maps the tiled WMMA matmul kernel family onto the hand-written B200
                      kernels behind include/hc-c/Cuda.h.

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
_SUPPORTED_INPUT_DTYPES = ("float16", "bfloat16")
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
    plan: GemmContract | None
    diagnostics: tuple[str, ...]


def known_targets() -> tuple[str, ...]:
    return (NVIDIA_SM100A,)


def lower_for_target(kernel_fn: Any, target: str) -> TargetResult:
    if target != NVIDIA_SM100A:
        raise ValueError(f"unknown hc.compile target {target!r}; known targets: {list(known_targets())}")
    plan, diagnostics = recognise_tiled_matmul(kernel_fn)
    return TargetResult(target, plan, tuple(diagnostics))


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


class _BodyShape(ast.NodeVisitor):
    """Collects the facts of the kernel body the recogniser relies on."""

    def __init__(self, group: str, a: str, b: str, c: str) -> None:
        self.group, self.a, self.b, self.c = group, a, b, c
        self.k_loops: list[ast.For] = []
        self.loads_in_loop: dict[str, list[ast.Subscript]] = {a: [], b: []}
        self.c_uses_after_loop = 0
        self._loop_depth = 0
        self._after_loop = False

    def visit_For(self, node: ast.For) -> None:
        self.k_loops.append(node)
        self._loop_depth += 1
        for stmt in node.body:
            self.visit(stmt)
        self._loop_depth -= 1
        self._after_loop = True

    def visit_Call(self, node: ast.Call) -> None:
        func = node.func
        is_group_load = (isinstance(func, ast.Attribute) and func.attr == "load"
                         and isinstance(func.value, ast.Name) and func.value.id == self.group)
        if is_group_load and self._loop_depth == 1 and node.args:
            src = node.args[0]
            if isinstance(src, ast.Subscript) and isinstance(src.value, ast.Name) and src.value.id in self.loads_in_loop:
                self.loads_in_loop[src.value.id].append(src)
        if self._after_loop and any(isinstance(arg, ast.Name) and arg.id == self.c for arg in node.args):
            self.c_uses_after_loop += 1
        self.generic_visit(node)


def _names_in(node: ast.AST | None) -> set[str]:
    return {n.id for n in ast.walk(node) if isinstance(n, ast.Name)} if node is not None else set()


_MAX_EPILOGUE_OPS = 4


def _check_body(kernel_fn: Any, params: list[str], a: str, b: str, c: str, tile: tuple[int, int, int],
                k_dim: Any, b_transposed: bool = False, bias: str | None = None,
                facts: dict[str, Any] | None = None, output_dtype: str = "float32") -> list[str]:
    """Structural check of the k-loop: `for k0 in range(0, K, tk)` with one masked load of an
    A window `a[rows, k0:k0+tk]` and one of a B window `b[k0:k0+tk, cols]`, then a store
    that receives `c`. Returns problems (empty when the body has the expected shape).

    `facts`, when given, receives what surrounds the loop: "accumulate" (the accumulators come
    from a call that is given `c` before the loop) and "epilogue" (the element-wise statements on
    the accumulators between the loop and the store)."""
    try:
        tree = ast.parse(textwrap.dedent(inspect.getsource(kernel_fn)))
    except (OSError, TypeError, SyntaxError):
        return ["kernel source is unavailable, so its k-loop cannot be checked"]
    fn_node = next((n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef))), None)
    if fn_node is None:
        return ["kernel source does not define a function"]
    consts = dict(getattr(kernel_fn, "__globals__", {}))
    try:
        consts.update(inspect.getclosurevars(kernel_fn).nonlocals)
    except (TypeError, ValueError):
        pass

    def const_value(node: ast.AST | None) -> Any:
        if isinstance(node, ast.Constant):
            return node.value
        if isinstance(node, ast.Name):
            return consts.get(node.id)
        return None

    shape = _BodyShape(params[0], a, b, c)
    for stmt in fn_node.body:
        shape.visit(stmt)
    problems: list[str] = []
    if len(shape.k_loops) != 1:
        return [f"expected exactly one k-loop in the kernel body, found {len(shape.k_loops)}"]
    loop = shape.k_loops[0]
    tk = tile[2]
    it = loop.iter
    ok_range = (isinstance(it, ast.Call) and isinstance(it.func, ast.Name) and it.func.id == "range"
                and len(it.args) == 3 and const_value(it.args[0]) == 0 and const_value(it.args[2]) == tk)
    if ok_range:
        stop = it.args[1]
        # K may be spelled `a.shape[1]`, `b.shape[0]` or as the K symbol / literal itself.
        spelled = ast.unparse(stop).replace(" ", "")
        k_names = {f"{a}.shape[1]", f"{b}.shape[1]" if b_transposed else f"{b}.shape[0]"}
        if isinstance(k_dim, str):
            k_names.add(k_dim)
        if spelled not in k_names and const_value(stop) != k_dim:
            problems.append(f"k-loop bound `{ast.unparse(stop)}` is not the shared extent of {a} and {b}")
    else:
        problems.append(f"k-loop must be `for k0 in range(0, K, {tk})`")
    k_var = loop.target.id if isinstance(loop.target, ast.Name) else None
    for name, axis in ((a, 1), (b, 1 if b_transposed else 0)):
        loads = shape.loads_in_loop[name]
        if len(loads) != 1:
            problems.append(f"expected one group.load of a window of `{name}` per k-step, found {len(loads)}")
            continue
        index = loads[0].slice
        parts = list(index.elts) if isinstance(index, ast.Tuple) else [index]
        if len(parts) != 2 or not all(isinstance(p, ast.Slice) for p in parts):
            problems.append(f"the load of `{name}` must slice both axes")
            continue
        k_slice, other = parts[axis], parts[1 - axis]
        if k_var is None or k_var not in _names_in(k_slice.lower) or k_var not in _names_in(k_slice.upper):
            problems.append(f"axis {axis} of the `{name}` window must advance with the k-loop variable")
        if k_var is not None and k_var in (_names_in(other.lower) | _names_in(other.upper)):
            problems.append(f"axis {1 - axis} of the `{name}` window must not depend on the k-loop variable")
    if shape.c_uses_after_loop < 1:
        problems.append(f"`{c}` must be passed to a store after the k-loop")
    surroundings = _loop_surroundings(fn_node, loop, c, bias, const_value, problems, output_dtype, consts)
    if facts is not None:
        facts.update(surroundings)
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


def _loop_surroundings(fn_node: ast.AST, loop: ast.For, c: str, bias: str | None, const_value: Any,
                       problems: list[str], output_dtype: str = "float32",
                       consts: dict[str, Any] | None = None) -> dict[str, Any]:
    """Reads the top-level statements before and after the k-loop (see `_check_body`)."""
    body = list(fn_node.body)
    if loop not in body:
        problems.append("the k-loop must be a top-level statement of the kernel body")
        return {"accumulate": False, "epilogue": ()}
    at = body.index(loop)

    def call_names(node: ast.AST) -> set[str]:
        return {arg.id for arg in getattr(node, "args", ()) if isinstance(arg, ast.Name)}

    # The accumulator variable: assigned in the loop from a call that also receives it.
    acc = None
    for stmt in loop.body:
        if (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name)
                and isinstance(stmt.value, ast.Call) and stmt.targets[0].id in call_names(stmt.value)):
            acc = stmt.targets[0].id
    if acc is None:
        problems.append("the k-loop must update the accumulators as `acc = f(..., acc)`")
        return {"accumulate": False, "epilogue": ()}

    accumulate = False
    initialised = False
    for stmt in body[:at]:
        if (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name)
                and stmt.targets[0].id == acc):
            initialised = True
            accumulate = isinstance(stmt.value, ast.Call) and c in call_names(stmt.value)
        elif c in _names_in(stmt):
            problems.append(f"`{c}` may only be read before the k-loop to initialise `{acc}`")
    if not initialised:
        problems.append(f"`{acc}` must be initialised before the k-loop")

    if accumulate and output_dtype != "float32":
        problems.append(f"a kernel that loads its accumulators from `{c}` needs a float32 `{c}` (got {output_dtype})")
    ops: list[tuple] = []
    stored = False
    narrowed = False  # the accumulators have been converted to the 16-bit type of `c`
    for stmt in body[at + 1:]:
        text = ast.unparse(stmt)
        if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Call) and c in call_names(stmt.value):
            if acc not in call_names(stmt.value):
                problems.append(f"the store `{text}` must receive `{acc}`")
            stored = True
            continue
        if acc not in _names_in(stmt):
            continue
        if stored:
            problems.append(f"`{text}` uses `{acc}` after the store")
            continue
        ok_target = (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1
                     and isinstance(stmt.targets[0], ast.Name) and stmt.targets[0].id == acc)
        op = _elementwise_op(stmt.value, acc, bias, const_value) if ok_target else None
        if op is not None and op and op[0] == "astype":
            target = _dtype_name_of(op[1], consts or {})
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
        elif op:
            ops.append(op)
    if len(ops) > _MAX_EPILOGUE_OPS:
        problems.append(f"at most {_MAX_EPILOGUE_OPS} element-wise statements can be folded into the store, "
                        f"found {len(ops)}")
    bias_ops = sum(1 for op in ops if op[0] == "bias")
    if bias is not None and bias_ops != 1:
        problems.append(f"`{bias}` must be added to `{acc}` exactly once between the k-loop and the store")
    return {"accumulate": accumulate, "epilogue": tuple(ops)}


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
