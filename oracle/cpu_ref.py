"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only `tests/`, `__graft_entry__.smoke()` and the CPU-baseline / reference legs of
`bench.py` may import this module; the product (`5_b200/`) never does and fails loudly
when its CUDA library is missing instead of falling back to anything here.

What is restated: the arithmetic of the reference example kernel as its simulator executes
it (examples/amdgpu_gfx11_wmma_matmul.py:178-190 per-lane multiply-accumulate, :315-326
k-loop and store; hc/simulator.py:1338-1357 masked loads, :1441-1458 clipped stores):

    C[i, j] = sum over k ascending of fp32(A[i, k]) * fp32(B[k, j]),  fp32 at every step.

Pinning: `tests/test_oracle.py` checks every function here bit-for-bit against fixtures that
`tests/golden/make_golden.py` produced by running the unmodified reference simulator
(shapes of the reference's own tests/test_examples.py:22-33 and example main(), config 1 of
the benchmark, and a bfloat16 twin).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libhc_oracle.so"
_LIB: ctypes.CDLL | None = None

F16 = 0
BF16 = 1


def build(force: bool = False) -> Path:
    """Compiles hc_matmul_oracle.c with the Makefile beside it (gcc, seconds)."""
    if force or not _LIB_PATH.exists() or (
        _LIB_PATH.stat().st_mtime < (_HERE / "hc_matmul_oracle.c").stat().st_mtime
    ):
        env = dict(os.environ)
        env.setdefault("CC", "gcc")
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True, env=env)
    return _LIB_PATH


def load() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(str(build()))  # rebuilt when the source is newer than the library
        if not hasattr(lib, "hc_oracle_matmul_fused") or not hasattr(lib, "hc_oracle_supports_f8"):  # a stale library with a fresh timestamp
            lib = ctypes.CDLL(str(build(force=True)))
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        lib.hc_oracle_matmul.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64, ci, ci]
        lib.hc_oracle_matmul.restype = ci
        lib.hc_oracle_matmul_rows.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64, ci, i64, i64, ci]
        lib.hc_oracle_matmul_rows.restype = ci
        lib.hc_oracle_matmul_fused.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64, ci, ci, ci, vp, vp, vp, ci]
        lib.hc_oracle_matmul_fused.restype = ci
        lib.hc_oracle_matmul_tiled.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64, ci]
        lib.hc_oracle_matmul_tiled.restype = ci
        lib.hc_oracle_max_threads.restype = ci
        _LIB = lib
    return _LIB


def max_threads() -> int:
    return int(load().hc_oracle_max_threads())


F8E4M3FN = 2
F8E5M2 = 3
_DTYPE_CODES = {"float16": F16, "bfloat16": BF16, "float8_e4m3fn": F8E4M3FN, "float8_e5m2": F8E5M2}


def dtype_code(dtype: np.dtype) -> int:
    name = np.dtype(dtype).name
    if name not in _DTYPE_CODES:
        raise ValueError(f"the oracle handles {sorted(_DTYPE_CODES)} inputs, got {name}")
    return _DTYPE_CODES[name]


def _as_bits(x: np.ndarray) -> np.ndarray:
    if x.ndim != 2:
        raise ValueError("the oracle expects rank-2 matrices")
    return np.ascontiguousarray(x).view(np.uint8 if x.dtype.itemsize == 1 else np.uint16)


def _check(a: np.ndarray, b: np.ndarray) -> tuple[int, int, int, int]:
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"shape mismatch: A {a.shape}, B {b.shape}")
    if a.dtype != b.dtype:
        raise ValueError("A and B must have the same dtype")
    return a.shape[0], b.shape[1], a.shape[1], dtype_code(a.dtype)


def matmul_k_ascending(a: np.ndarray, b: np.ndarray, *, threads: int = 0,
                       rows: tuple[int, int] | None = None) -> np.ndarray:
    """k-ascending fp32 product via the C restatement (fast form).

    With `rows=(r0, r1)` only those rows of C are computed (the others are left 0), which
    bounds the CPU time on large problems.
    """
    m, n, k, code = _check(a, b)
    abits, bbits = _as_bits(a), _as_bits(b)
    c = np.zeros((m, n), np.float32)
    r0, r1 = (0, m) if rows is None else rows
    rc = load().hc_oracle_matmul_rows(abits.ctypes.data, max(k, 1), bbits.ctypes.data, max(n, 1),
                                      c.ctypes.data, max(n, 1), m, n, k, code, r0, r1, threads)
    if rc != 0:
        raise MemoryError("the oracle could not allocate its widened copy of B")
    return c


EPILOGUE_KINDS = {"scale": 1, "add": 2, "max": 3, "min": 4, "bias": 5}


def matmul_fused(a: np.ndarray, b: np.ndarray, *, c0: np.ndarray | None = None, epilogue=(),
                 bias: np.ndarray | None = None, threads: int = 0, out_dtype=None) -> np.ndarray:
    """Members of the kernel family around the example: accumulators that start from `c0`
    (C += A.B) and element-wise statements after the k-loop, e.g.
    `(("scale", 0.5), ("bias",), ("max", 0.0))`, in the reference simulator's fp32 order. With
    `out_dtype` (float16 / bfloat16, a kernel whose `c` is a 16-bit buffer) the fp32 values are
    rounded to nearest even at the end, as the simulator's `astype` / store does."""
    m, n, k, code = _check(a, b)
    abits, bbits = _as_bits(a), _as_bits(b)
    c = np.zeros((m, n), np.float32) if c0 is None else np.array(c0, dtype=np.float32, order="C", copy=True)
    kinds = np.array([EPILOGUE_KINDS[op[0]] for op in epilogue], dtype=np.int32)
    values = np.array([float(op[1]) if len(op) > 1 else 0.0 for op in epilogue], dtype=np.float32)
    bias32 = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    rc = load().hc_oracle_matmul_fused(abits.ctypes.data, max(k, 1), bbits.ctypes.data, max(n, 1),
                                       c.ctypes.data, max(n, 1), m, n, k, code, 0 if c0 is None else 1,
                                       len(kinds), kinds.ctypes.data, values.ctypes.data,
                                       None if bias32 is None else bias32.ctypes.data, threads)
    if rc != 0:
        raise MemoryError("the oracle could not allocate its widened copy of B")
    return c if out_dtype is None else c.astype(out_dtype)


def matmul_tiled(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Literal workgroup / k-step / lane restatement (slow; small shapes)."""
    m, n, k, code = _check(a, b)
    abits, bbits = _as_bits(a), _as_bits(b)
    c = np.zeros((m, n), np.float32)
    load().hc_oracle_matmul_tiled(abits.ctypes.data, max(k, 1), bbits.ctypes.data, max(n, 1),
                                  c.ctypes.data, max(n, 1), m, n, k, code)
    return c


def matmul_numpy(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The same arithmetic in NumPy: one fp32 rank-1 update per k, k ascending."""
    m, n, k, _ = _check(a, b)
    a32 = a.astype(np.float32)
    b32 = b.astype(np.float32)
    c = np.zeros((m, n), np.float32)
    for kk in range(k):
        c += a32[:, kk : kk + 1] * b32[kk : kk + 1, :]
    return c


def map_elementwise(x: np.ndarray, ops, other: np.ndarray | None = None) -> np.ndarray:
    """The masked element-wise kernel class as the reference simulator executes it
    (tests/test_simulator.py:210-224; loads hc/simulator.py:1338-1357, stores :1441-1458; value
    arithmetic hc/_sim_types.py:373-420, which applies the NumPy ufunc to the payload): every
    element below the buffers' extent goes through the statements once, each statement one
    float32 NumPy operation. `ops` as the recogniser lists them: ("scale", c), ("add", c),
    ("max", c), ("min", c), ("rsub", c), ("add_other",), ("sub_other",), ("rsub_other",),
    ("mul_other",), ("max_other",), ("min_other",), and "rmax" / "rmin" (with a constant or
    "_other") for maximum / minimum with the chain as the second operand."""
    v = np.array(x, dtype=np.float32, copy=True)
    w = None if other is None else np.asarray(other, dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        for op in ops:
            kind = op[0]
            operand = w if kind.endswith("_other") else np.float32(op[1])
            base = kind[: -len("_other")] if kind.endswith("_other") else kind
            if base in ("scale", "mul"):
                v = v * operand
            elif base == "add":
                v = v + operand
            elif base == "sub":
                v = v - operand
            elif base == "rsub":
                v = operand - v
            elif base == "max":
                v = np.maximum(v, operand)
            elif base == "min":
                v = np.minimum(v, operand)
            elif base == "rmax":  # operand order matters when neither is greater (signed zeros)
                v = np.maximum(operand, v)
            elif base == "rmin":
                v = np.minimum(operand, v)
            else:
                raise ValueError(f"unknown operation {kind!r}")
    return v.astype(np.float32, copy=False)


def pairwise_distance(x1: np.ndarray, x2: np.ndarray, *, take_sqrt: bool = True, rows_per_block: int = 64) -> np.ndarray:
    """The pairwise kernel class as the reference simulator executes it (tests/test_simulator.py:142-167):
    out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h]) ** 2) in float32, one NumPy operation per step -- the
    difference, the power (np.power with exponent 2, hc/_sim_types.py:403-404), the sum. The simulator
    reduces every (i, j) with `np.sum(payload[active])` over a contiguous float32 vector of h values
    (hc/_sim_types.py:1050-1066, 1100-1102), NumPy's pairwise summation; reducing the last axis of a
    contiguous block is the same inner loop, so the rows are evaluated a block at a time here
    (`pairwise_sum_in_numpy_order` restates that order explicitly and the tests hold both against
    np.sum)."""
    x1 = np.ascontiguousarray(x1, dtype=np.float32)
    x2 = np.ascontiguousarray(x2, dtype=np.float32)
    w1, w2 = x1.shape[0], x2.shape[0]
    out = np.empty((w1, w2), np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        for r0 in range(0, w1, rows_per_block):
            block = np.power(x1[r0 : r0 + rows_per_block, None, :] - x2[None, :, :], 2)
            total = np.ascontiguousarray(block).sum(axis=2)
            out[r0 : r0 + rows_per_block] = np.sqrt(total) if take_sqrt else total
    return out


def row_sums(x: np.ndarray, *, square: bool = False, take_sqrt: bool = False, restated: bool = False) -> np.ndarray:
    """The row-sum kernel class as the reference simulator executes it: out[i] = np.sum of row i in
    float32 (`_reduce_active` hands the active values of a row, a contiguous vector, to np.sum,
    hc/_sim_types.py:1050-1066, 1100-1102), with every value multiplied by itself first (`square`:
    `rows * rows` and `rows ** 2` are the same float32 product) and np.sqrt of the sum (`take_sqrt`) if
    asked. Reducing the last axis of a contiguous matrix runs the same inner loop per row, so the
    fast form is one NumPy call; `restated` computes every row with `pairwise_sum_in_numpy_order`
    plus the reduction's initial value +0 instead (the tests hold the two against each other).
    A matrix without columns gives no output at all in the simulator (a reduction over no active
    value is inactive and is not stored); callers handle that case, this function returns zeros."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        values = x * x if square else x
        if restated:
            total = np.array([np.float32(np.float32(0.0) + pairwise_sum_in_numpy_order(row)) for row in values],
                             np.float32).reshape(x.shape[0])
        else:
            total = np.ascontiguousarray(values).sum(axis=1, dtype=np.float32)
        return np.sqrt(total) if take_sqrt else total


def pairwise_sum_in_numpy_order(values: np.ndarray) -> np.float32:
    """NumPy's float32 sum of a contiguous vector, written out: fewer than 8 values are added in
    order; up to 128 go into eight interleaved accumulators r[i % 8] that are combined as
    ((r0 + r1) + (r2 + r3)) + ((r4 + r5) + (r6 + r7)) before the n % 8 tail is added in order; longer
    vectors are split at n / 2 rounded down to a multiple of 8 and the two sums are added. This is
    the order the CUDA pairwise kernel follows."""
    a = np.asarray(values, dtype=np.float32)
    n = a.shape[0]
    f = np.float32
    with np.errstate(invalid="ignore", over="ignore"):
        if n < 8:
            total = f(0.0)
            for v in a:
                total = f(total + v)
            return total
        if n <= 128:
            r = [f(v) for v in a[:8]]
            i = 8
            while i < n - n % 8:
                for j in range(8):
                    r[j] = f(r[j] + a[i + j])
                i += 8
            total = f(f(f(r[0] + r[1]) + f(r[2] + r[3])) + f(f(r[4] + r[5]) + f(r[6] + r[7])))
            while i < n:
                total = f(total + a[i])
                i += 1
            return total
        left = n // 2
        left -= left % 8
        return f(pairwise_sum_in_numpy_order(a[:left]) + pairwise_sum_in_numpy_order(a[left:]))
