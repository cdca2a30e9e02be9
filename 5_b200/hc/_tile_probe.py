"""Compile-time probe of a tiled-matmul kernel's helper chain.

The NVIDIA target replaces a whole hc kernel by a hand-written GEMM, so it must know that the
kernel *is* that GEMM. The statements of the kernel body itself (tile origins, the k-loop and
its windows, the element-wise statements, the store call) are checked syntactically by
`hc._pipeline`. What the body calls -- the accumulator initialiser, the multiply-accumulate
helper with its `@kernel.intrinsic`, the bias helper, the store helper -- is lane arithmetic
that can be spelled in many ways (the reference's example and this repository's spell the
same distribution differently: examples/amdgpu_gfx11_wmma_matmul.py:77-106, 262-298), so it
is not matched against a pattern. It is *run*: this module executes those helpers, as the
Python functions they are, for single workgroups of a small ragged problem, on a minimal host
model of the workgroup surface they use, and compares what they leave in `c` with the
product they must compute. Integer-valued probe data make the comparison exact.

The model follows the reference simulator for exactly the calls such helpers make:
`group.load` copies the overlap of a (NumPy-clipped) window into a tile whose remaining
elements are inactive (hc/simulator.py:1338-1357); `group.store` writes the active overlap
(hc/simulator.py:1441-1458); `@group.workitems` runs the function once per lane and stacks
the per-lane vectors along trailing (wave, 1) axes (hc/simulator.py:292-300, 1090-1095);
values carry an activity mask, `with_inactive` fills it, reading an inactive scalar is an
error here (a poison value there, hc/_sim_types.py:285-305, 353-357). Barriers, subgroups,
reductions and layouts are not modelled: a helper that needs them fails the probe and the
kernel is refused, which is the safe direction.

Nothing here runs at launch time and nothing here produces a result a caller sees: the probe
only decides whether `hc.compile(..., target="nvidia-sm100a")` accepts a kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence

import numpy as np

__all__ = ["ProbeError", "ProbeValue", "ProbeGroup", "HelperCall", "probe_helper_chain"]


class ProbeError(Exception):
    """A helper did something the probe model does not cover, or computed something else."""


def _as_index(index: Any) -> Any:
    if isinstance(index, tuple):
        return tuple(_as_index(part) for part in index)
    if isinstance(index, (int, np.integer, slice)) or index is Ellipsis:
        return index
    raise ProbeError(f"unsupported index {index!r} on a tile value")


class ProbeValue:
    """A tile or vector value: dense payload plus activity mask (the simulator's masked value)."""

    __array_priority__ = 1000

    def __init__(self, data: Any, mask: Any = None) -> None:
        self._data = np.asarray(data)
        self._mask = np.ones(self._data.shape, bool) if mask is None else np.asarray(mask, bool)
        if self._mask.shape != self._data.shape:
            raise ProbeError("payload and mask shapes differ")

    shape = property(lambda self: tuple(int(d) for d in self._data.shape))
    dtype = property(lambda self: self._data.dtype)
    ndim = property(lambda self: int(self._data.ndim))

    def __array__(self, *args: Any, **kwargs: Any) -> np.ndarray:
        raise TypeError("tile values do not implicitly convert to numpy arrays")

    def __bool__(self) -> bool:
        raise TypeError("tile values do not define truthiness")

    def __len__(self) -> int:
        return self.shape[0]

    def __getitem__(self, index: Any) -> Any:
        index = _as_index(index)
        data, mask = self._data[index], self._mask[index]
        if np.isscalar(mask) or getattr(mask, "ndim", 1) == 0:
            if not bool(mask):
                raise ProbeError("a helper reads an element that is inactive (outside its buffer) without "
                                 "`with_inactive(value=...)`")
            return data
        return ProbeValue(data, mask)

    def vec(self, shape: Sequence[int] | None = None) -> "ProbeValue":
        if shape is not None and tuple(shape) != self.shape:
            return ProbeValue(self._data.reshape(tuple(shape)), self._mask.reshape(tuple(shape)))
        return ProbeValue(self._data, self._mask)

    def with_inactive(self, *, value: Any) -> "ProbeValue":
        return ProbeValue(np.where(self._mask, self._data, np.asarray(value, dtype=self.dtype)))

    def astype(self, dtype: Any) -> "ProbeValue":
        return ProbeValue(self._data.astype(dtype), self._mask.copy())

    def _binary(self, other: Any, op: Callable[[Any, Any], Any], reverse: bool = False) -> "ProbeValue":
        if isinstance(other, ProbeValue):
            other_data, other_mask = other._data, other._mask
        elif isinstance(other, (int, float, np.number)):
            other_data, other_mask = other, True
        else:
            raise ProbeError(f"unsupported operand {type(other).__name__} in tile arithmetic")
        data = op(other_data, self._data) if reverse else op(self._data, other_data)
        return ProbeValue(data, np.logical_and(self._mask, other_mask))

    def __add__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.add)

    def __radd__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.add, True)

    def __sub__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.subtract)

    def __rsub__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.subtract, True)

    def __mul__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.multiply)

    def __rmul__(self, other: Any) -> "ProbeValue":
        return self._binary(other, np.multiply, True)


class _ProbeWorkItem:
    def __init__(self, lane: int, group_id: tuple[int, int], wave: int) -> None:
        self._local = (lane, 0)
        self._global = (group_id[0] * wave + lane, group_id[1])

    def local_id(self) -> tuple[int, int]:
        return self._local

    def global_id(self) -> tuple[int, int]:
        return self._global


class ProbeGroup:
    """One workgroup: (wave, 1) workitems, the calls matmul helpers make on `group`."""

    def __init__(self, group_id: tuple[int, int], wave: int, work_shape: tuple[int, int]) -> None:
        self.group_id = group_id
        self.shape = (wave, 1)
        self.size = wave
        self.work_shape = work_shape
        self.work_offset = (group_id[0] * wave, group_id[1])
        self._wave = wave
        self._in_workitems = False

    # -- collective regions -------------------------------------------------------------
    def workitems(self, fn: Callable[[Any], Any]) -> Callable[[], Any]:
        def run() -> Any:
            if self._in_workitems:
                raise ProbeError("nested @group.workitems regions")
            self._in_workitems = True
            try:
                results = [fn(_ProbeWorkItem(lane, self.group_id, self._wave)) for lane in range(self._wave)]
            finally:
                self._in_workitems = False
            if all(result is None for result in results):
                return None
            if not all(isinstance(result, ProbeValue) for result in results):
                raise ProbeError("every workitem must return a vector value (or all of them nothing)")
            shapes = {result.shape for result in results}
            if len(shapes) != 1:
                raise ProbeError(f"workitems returned vectors of different shapes {sorted(shapes)}")
            data = np.stack([result._data for result in results], axis=-1)[..., None]
            mask = np.stack([result._mask for result in results], axis=-1)[..., None]
            return ProbeValue(data, mask)

        return run

    def subgroups(self, fn: Any) -> Any:
        raise ProbeError("@group.subgroups is not covered by the probe model")

    def barrier(self) -> None:
        raise ProbeError("group.barrier() is not covered by the probe model")

    # -- loads, stores, allocation ------------------------------------------------------
    @staticmethod
    def _source(source: Any) -> tuple[np.ndarray, np.ndarray]:
        if isinstance(source, ProbeValue):
            return source._data, source._mask
        if isinstance(source, np.ndarray):
            return source, np.ones(source.shape, bool)
        raise ProbeError("load source must be a buffer window or a tile value")

    def _load(self, source: Any, shape: Any, mask: Any, layout: Any) -> ProbeValue:
        if mask is not None or layout is not None or shape is None:
            raise ProbeError("the probe model covers `load(window, shape=...)` only")
        shape = tuple(int(extent) for extent in shape)
        data, active = self._source(source)
        if data.ndim != len(shape):
            raise ProbeError("load rank does not match the requested shape")
        out = np.zeros(shape, data.dtype)
        out_mask = np.zeros(shape, bool)
        overlap = tuple(slice(0, min(shape[i], data.shape[i])) for i in range(len(shape)))
        out[overlap] = data[overlap]
        out_mask[overlap] = active[overlap]
        return ProbeValue(out, out_mask)

    def load(self, source: Any, *, shape: Any = None, mask: Any = None, layout: Any = None) -> ProbeValue:
        if self._in_workitems:
            raise ProbeError("group.load() inside @group.workitems")
        return self._load(source, shape, mask, layout)

    def vload(self, source: Any, *, shape: Any = None, mask: Any = None, layout: Any = None) -> ProbeValue:
        return self._load(source, shape, mask, layout)

    def store(self, target: Any, value: Any) -> None:
        if not isinstance(target, np.ndarray):
            raise ProbeError("store target must be a window of a buffer")
        if not isinstance(value, ProbeValue):
            raise ProbeError("store source must be a tile or vector value")
        if target.ndim != value.ndim:
            raise ProbeError("store source and target ranks must match")
        overlap = tuple(slice(0, min(target.shape[i], value.shape[i])) for i in range(target.ndim))
        region = target[overlap]
        active = value._mask[overlap]
        region[active] = value._data[overlap][active]

    def _filled(self, shape: Any, dtype: Any, fill: Any, layout: Any, active: bool = True) -> ProbeValue:
        if layout is not None:
            raise ProbeError("layouts are not covered by the probe model")
        shape = tuple(int(extent) for extent in shape)
        return ProbeValue(np.full(shape, fill, np.dtype(dtype)), np.full(shape, active, bool))

    def zeros(self, *, shape: Any, dtype: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, 0, layout)

    def vzeros(self, *, shape: Any, dtype: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, 0, layout)

    def ones(self, *, shape: Any, dtype: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, 1, layout)

    def vones(self, *, shape: Any, dtype: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, 1, layout)

    def full(self, *, shape: Any, dtype: Any, fill_value: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, fill_value, layout)

    def vfull(self, *, shape: Any, dtype: Any, fill_value: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, fill_value, layout)

    def empty(self, *, shape: Any, dtype: Any, layout: Any = None) -> ProbeValue:
        return self._filled(shape, dtype, 0, layout, active=False)


@dataclass(frozen=True)
class HelperCall:
    """One call the kernel body makes: the helper and, per positional argument, what it is.

    An argument is ("group",), ("a_tile",), ("b_tile",), ("acc",), ("c",), ("bias",), or
    ("origin", f) with f(gid0, gid1) -> int, the value of an index expression the recogniser has
    already shown to be the tile's row or column origin.
    """

    fn: Callable[..., Any]
    args: tuple[tuple, ...]
    text: str  # the call as written, for diagnostics


def _call(call: HelperCall, values: dict[str, Any], gid: tuple[int, int]) -> Any:
    args = []
    for arg in call.args:
        if arg[0] == "origin":
            args.append(int(arg[1](gid[0], gid[1])))
        else:
            args.append(values[arg[0]])
    return call.fn(*args)


def _probe_matrix(rng: np.random.Generator, shape: tuple[int, ...], dtype: Any, lo: int, hi: int) -> np.ndarray:
    return rng.integers(lo, hi + 1, size=shape).astype(dtype)


def probe_helper_chain(*, init: HelperCall, step: HelperCall, store: HelperCall, bias: HelperCall | None,
                       tile: tuple[int, int, int], wave: int, acc_len: int, input_dtype: Any,
                       accumulate: bool, b_transposed: bool) -> list[str]:
    """Runs init -> two k-steps -> (bias) -> store for several workgroups of a ragged problem and
    checks `c` against the product. Returns the problems found (empty: the chain is a matmul tile).

    The problem has 2 full tiles plus a partial one along m and n and one full plus one partial
    k-step, so interior, edge and corner workgroups (masked loads, clipped stores) are all
    exercised. Values are small integers: every product and sum is exact in float16/bfloat16
    inputs and float32 accumulation, so `c` must match exactly.
    """
    tm, tn, tk = tile
    m, n, k = 2 * tm + max(1, tm // 3), 2 * tn + max(1, tn // 2), tk + max(1, tk // 2)
    rng = np.random.default_rng(20240229)
    a = _probe_matrix(rng, (m, k), input_dtype, -3, 3)
    b_kn = _probe_matrix(rng, (k, n), input_dtype, -3, 3)
    b = np.ascontiguousarray(b_kn.T) if b_transposed else b_kn
    c_before = _probe_matrix(rng, (m, n), np.float32, -64, 64)
    bias_vec = _probe_matrix(rng, (n,), np.float32, -32, 32)
    product = a.astype(np.float32) @ b_kn.astype(np.float32)
    expect = product + (c_before if accumulate else 0)
    work_shape = (-(-m // tm) * wave, -(-n // tn))
    problems: list[str] = []

    def run(gid: tuple[int, int], with_bias: bool) -> np.ndarray:
        c = c_before.copy()
        group = ProbeGroup(gid, wave, work_shape)
        values: dict[str, Any] = {"group": group, "c": c, "bias": bias_vec}
        acc = _call(init, values, gid)
        if not isinstance(acc, ProbeValue) or acc.shape != (acc_len, wave, 1) or acc.dtype != np.float32:
            got = f"{type(acc).__name__} {getattr(acc, 'shape', '')} {getattr(acc, 'dtype', '')}".strip()
            raise ProbeError(f"`{init.text}` must give {acc_len} float32 accumulators per lane "
                             f"(shape ({acc_len}, {wave}, 1)), got {got}")
        if not accumulate and (np.any(acc._data != 0) or not np.all(acc._mask)):
            raise ProbeError(f"`{init.text}` does not start the accumulators at zero")
        values["acc"] = acc
        r0, c0 = gid[0] * tm, gid[1] * tn
        for k0 in range(0, k, tk):
            values["a_tile"] = group.load(a[r0:r0 + tm, k0:k0 + tk], shape=(tm, tk))
            values["b_tile"] = (group.load(b[c0:c0 + tn, k0:k0 + tk], shape=(tn, tk)) if b_transposed
                                else group.load(b[k0:k0 + tk, c0:c0 + tn], shape=(tk, tn)))
            acc = _call(step, values, gid)
            if not isinstance(acc, ProbeValue) or acc.shape != (acc_len, wave, 1):
                raise ProbeError(f"`{step.text}` must return the updated accumulators")
            values["acc"] = acc
        if with_bias and bias is not None:
            acc = _call(bias, values, gid)
            if not isinstance(acc, ProbeValue) or acc.shape != (acc_len, wave, 1):
                raise ProbeError(f"`{bias.text}` must return the updated accumulators")
            values["acc"] = acc
        _call(store, values, gid)
        return c

    tiles_m, tiles_n = -(-m // tm), -(-n // tn)
    for gid in ((0, 0), (1, 0), (0, 1), (tiles_m - 1, 1), (1, tiles_n - 1), (tiles_m - 1, tiles_n - 1)):
        for with_bias in ((False, True) if bias is not None else (False,)):
            try:
                c = run(gid, with_bias)
            except ProbeError as exc:
                return [str(exc)]
            except Exception as exc:  # a user's helper may fail in any way on the probe model
                return [f"running the kernel's helpers for workgroup {gid} on probe tiles raised "
                        f"{type(exc).__name__}: {exc}"]
            want = c_before.copy()
            rows = slice(gid[0] * tm, min(m, gid[0] * tm + tm))
            cols = slice(gid[1] * tn, min(n, gid[1] * tn + tn))
            want[rows, cols] = expect[rows, cols] + (bias_vec[None, cols] if with_bias else 0)
            if not np.array_equal(c, want):
                outside = want.copy()
                outside[rows, cols] = c[rows, cols]
                where = ("writes outside its tile of `c`" if not np.array_equal(outside, c)
                         else "leaves values in its tile of `c` that are not" +
                              (" c +" if accumulate else "") + " a @ b" + (" + bias" if with_bias else ""))
                problems.append(
                    f"the helper chain `{init.text}` / `{step.text}` / "
                    + (f"`{bias.text}` / " if with_bias and bias is not None else "")
                    + f"`{store.text}` {where} (probe workgroup {gid} of a {m}x{n}x{k} problem)")
                return problems
    return problems
