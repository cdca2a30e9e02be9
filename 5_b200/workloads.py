"""The five benchmark configurations: seeded synthetic inputs, work counts, and the
tolerance check against a float64 product.

The shapes, seeds and distributions are the benchmark's own definition of the workload (no
external dataset stands behind them):

  1  "sim_64"       M=N=K=64, float16, A then B ~ N(0,1) from default_rng(0)
  2  "gemm_8192"    M=N=K=8192, float16, N(0,1)/sqrt(K), default_rng(1)
  3  "ragged"       M=4095, N=3073, K=1031, bfloat16, U(-1,1), default_rng(2)
  4  "skinny"       M=8, N=16384, K=8192, float16, A ~ N(0,1), B ~ N(0,0.02), default_rng(3)
  5  "sharded"      M=16384, N=32768, K=16384, float16, N(0,1)/sqrt(K), default_rng(4);
                    B is generated per 2048-column block from default_rng([4, block]) so that a
                    rank can produce its own column slab without materialising all of B

Algorithmic work per product: flops = 2*M*N*K; bytes = 2*M*K + 2*K*N + 4*M*N (each operand
read once, C written once).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

__all__ = ["CONFIGS", "Workload", "register_custom", "check_against_float64", "flops", "algorithmic_bytes", "make_inputs",
           "make_sharded_inputs", "SHARDED_BLOCK_COLUMNS"]

SHARDED_BLOCK_COLUMNS = 2048


@dataclass(frozen=True)
class Workload:
    name: str
    m: int
    n: int
    k: int
    dtype: str
    seed: int


CONFIGS = {
    "sim_64": Workload("sim_64", 64, 64, 64, "float16", 0),
    "gemm_8192": Workload("gemm_8192", 8192, 8192, 8192, "float16", 1),
    "ragged": Workload("ragged", 4095, 3073, 1031, "bfloat16", 2),
    "skinny": Workload("skinny", 8, 16384, 8192, "float16", 3),
    "sharded": Workload("sharded", 16384, 32768, 16384, "float16", 4),
    # Not one of the five benchmark configurations: a product with few tiles and a long k-loop (eight
    # 128x256 tiles), the shape class whose tiles are shared among thread-block clusters.
    "long_k": Workload("long_k", 512, 512, 16384, "float16", 6),
}


def register_custom(m: int, n: int, k: int, dtype: str = "float16") -> str:
    """Adds workload "custom": an arbitrary shape with the distribution of configuration 2
    (N(0,1)/sqrt(K), default_rng(5)), for profiling other members of the kernel family."""
    CONFIGS["custom"] = Workload("custom", int(m), int(n), int(k), dtype, 5)
    return "custom"


def with_input_dtype(name: str, dtype: str) -> str:
    """Registers workload `name` again with another element type of A and B (same shape, seed and
    distribution, values rounded to `dtype`), e.g. "float8_e4m3fn"; returns the new workload's name."""
    w = CONFIGS[name]
    if dtype == w.dtype:
        return name
    alias = f"{name}:{dtype}"
    CONFIGS[alias] = Workload(alias, w.m, w.n, w.k, dtype, w.seed)
    return alias


def flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def algorithmic_bytes(m: int, n: int, k: int) -> float:
    return 2.0 * m * k + 2.0 * k * n + 4.0 * m * n


def _np_dtype(name: str):
    if name in ("bfloat16", "float8_e4m3fn", "float8_e5m2"):
        import ml_dtypes

        return getattr(ml_dtypes, name)
    return np.dtype(name).type


def _normal(rng: np.random.Generator, shape: tuple[int, int], scale: float, dtype) -> np.ndarray:
    out = rng.standard_normal(shape, dtype=np.float32)
    if scale != 1.0:
        out *= np.float32(scale)
    return out.astype(dtype)


def make_inputs(name: str) -> tuple[np.ndarray, np.ndarray]:
    """A and B of configurations 1-4 (and of 5, in full; prefer make_sharded_inputs there)."""
    w = CONFIGS[name]
    dtype = _np_dtype(w.dtype)
    name = name.split(":", 1)[0]  # "<workload>:<dtype>" (with_input_dtype) draws like <workload>
    if name == "sharded":
        a, b = make_sharded_inputs(0, w.n)
        return a, b
    rng = np.random.default_rng(w.seed)
    if name == "sim_64":
        a = rng.standard_normal((w.m, w.k)).astype(dtype)
        b = rng.standard_normal((w.k, w.n)).astype(dtype)
    elif name in ("gemm_8192", "custom", "long_k"):
        scale = 1.0 / np.sqrt(w.k)
        a = _normal(rng, (w.m, w.k), scale, dtype)
        b = _normal(rng, (w.k, w.n), scale, dtype)
    elif name == "ragged":
        a = rng.uniform(-1.0, 1.0, size=(w.m, w.k)).astype(dtype)
        b = rng.uniform(-1.0, 1.0, size=(w.k, w.n)).astype(dtype)
    elif name == "skinny":
        a = _normal(rng, (w.m, w.k), 1.0, dtype)
        b = _normal(rng, (w.k, w.n), 0.02, dtype)
    else:  # pragma: no cover
        raise KeyError(name)
    return a, b


def make_sharded_inputs(col_begin: int, col_end: int, *, m: int | None = None, k: int | None = None,
                        with_a: bool = True) -> tuple[np.ndarray | None, np.ndarray]:
    """Configuration 5: A (replicated) and columns [col_begin, col_end) of B.

    Column boundaries must be multiples of SHARDED_BLOCK_COLUMNS. `m` / `k` shrink the
    problem for tests while keeping the generator's structure.
    """
    w = CONFIGS["sharded"]
    m = w.m if m is None else m
    k = w.k if k is None else k
    if col_begin % SHARDED_BLOCK_COLUMNS or col_end % SHARDED_BLOCK_COLUMNS:
        raise ValueError(f"slab boundaries must be multiples of {SHARDED_BLOCK_COLUMNS}")
    scale = 1.0 / np.sqrt(w.k)
    a = None
    if with_a:
        a = _normal(np.random.default_rng([w.seed, 1 << 20]), (m, k), scale, np.float16)
    b = np.empty((k, col_end - col_begin), np.float16)
    for block in range(col_begin // SHARDED_BLOCK_COLUMNS, col_end // SHARDED_BLOCK_COLUMNS):
        rng = np.random.default_rng([w.seed, block])
        lo = block * SHARDED_BLOCK_COLUMNS - col_begin
        b[:, lo : lo + SHARDED_BLOCK_COLUMNS] = _normal(rng, (k, SHARDED_BLOCK_COLUMNS), scale, np.float16)
    return a, b


def check_against_float64(c: np.ndarray, a: np.ndarray, b: np.ndarray, *,
                          rows: np.ndarray | None = None, c0: np.ndarray | None = None,
                          epilogue: tuple = (), bias: np.ndarray | None = None) -> dict[str, float | bool]:
    """The benchmark's parity rule, versus a float64 product of the same low-precision inputs:
    relative Frobenius error <= 1e-3 and, element-wise, |C - ref| <= 1e-2 * (|A| |B|).

    `rows` restricts the check to a sample of rows (the reference product of a large problem
    is computed on the CPU, so the sample bounds host time); the result says how many rows
    were checked.

    For the other members of the kernel family the reference value is ops(C0 + A.B): `c0` is C
    before the launch (accumulating member), `epilogue` the element-wise operations in order
    (("scale", x), ("add", x), ("max", x), ("min", x), ("bias",)) and `bias` the per-column
    vector. The element bound is carried through them (|C0| and the added constants join it,
    a scale multiplies it, max/min leave it).
    """
    if rows is not None:
        a = a[rows]
        c = c[rows]
        c0 = None if c0 is None else c0[rows]
    a64 = a.astype(np.float64)
    b64 = b.astype(np.float64)
    ref = a64 @ b64
    bound = np.abs(a64) @ np.abs(b64)
    if c0 is not None:
        ref = ref + c0
        bound = bound + np.abs(c0)
    for op in epilogue:
        x = float(np.float32(op[1])) if len(op) > 1 else 0.0
        if op[0] == "scale":
            ref, bound = ref * x, bound * abs(x)
        elif op[0] == "add":
            ref, bound = ref + x, bound + abs(x)
        elif op[0] == "bias":
            ref, bound = ref + bias[None, :], bound + np.abs(bias)[None, :]
        elif op[0] == "max":
            ref = np.maximum(ref, x)
        elif op[0] == "min":
            ref = np.minimum(ref, x)
        else:
            raise ValueError(f"unknown operation {op[0]!r}")
    diff = np.abs(c.astype(np.float64) - ref)
    rel_fro = float(np.linalg.norm(diff) / max(np.linalg.norm(ref), 1e-300))
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(bound > 0, diff / bound, np.where(diff > 0, np.inf, 0.0))
    max_ratio = float(ratio.max()) if ratio.size else 0.0
    finite = bool(np.isfinite(c).all())
    return {
        "rel_frobenius": rel_fro,
        "max_element_ratio": max_ratio,
        "finite": finite,
        "rows_checked": int(c.shape[0]),
        "ok": bool(finite and rel_fro <= 1e-3 and max_ratio <= 1e-2),
    }
