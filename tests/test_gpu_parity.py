"""Parity of the CUDA path with the oracle, on a B200. Everything goes through the public
surface (`hc.compile(..., target="nvidia-sm100a")` handle or `hc.cuda`), i.e. the C ABI.

Tolerance (tensor cores add in a different order than the oracle's k-ascending fp32 chain, so
bit equality is not expected): versus a float64 product of the same low-precision inputs,
relative Frobenius error <= 1e-3 and |C - ref| <= 1e-2 * (|A| |B|) element-wise. Versus the
oracle / the reference simulator's stored output the same bound is applied with the oracle in
place of the float64 product.
"""

from __future__ import annotations

import numpy as np
import pytest

import hc
import workloads
from conftest import GOLDEN_NAMES, load_golden, np_dtype
from examples.b200_wmma_matmul import compiled_for, gpu_wmma_matmul
from hc import cuda
from hc.errors import DeviceError
from oracle import cpu_ref

pytestmark = pytest.mark.gpu

REL_FROBENIUS = 1e-3
ELEMENT_RATIO = 1e-2


def assert_close_to_oracle(c: np.ndarray, a: np.ndarray, b: np.ndarray, expect: np.ndarray | None = None) -> None:
    expect = cpu_ref.matmul_k_ascending(a, b) if expect is None else expect
    assert c.shape == expect.shape and c.dtype == np.float32
    assert np.isfinite(c).all()
    bound = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
    diff = np.abs(c.astype(np.float64) - expect.astype(np.float64))
    assert (diff <= ELEMENT_RATIO * bound + 1e-30).all(), float((diff / np.maximum(bound, 1e-30)).max())
    norm = np.linalg.norm(expect.astype(np.float64))
    assert np.linalg.norm(diff) <= REL_FROBENIUS * max(norm, 1e-30)
    assert workloads.check_against_float64(c, a, b)["ok"]


def random_inputs(m: int, n: int, k: int, dtype: str, seed: int = 0, scale: float = 1.0):
    rng = np.random.default_rng([seed, m, n, k])
    a = (rng.standard_normal((m, k)) * scale).astype(np_dtype(dtype))
    b = (rng.standard_normal((k, n)) * scale).astype(np_dtype(dtype))
    return a, b


# ---------------------------------------------------------------- golden vectors --------


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_handle_matches_reference_simulator_output(name: str) -> None:
    a, b, c_sim = load_golden(name)
    c = np.full(c_sim.shape, np.nan, np.float32)
    handle = compiled_for(a.dtype.name)
    assert handle(a, b, c) is None
    assert_close_to_oracle(c, a, b, expect=c_sim)


def test_simulator_launch_entry_point(gpu_ctx) -> None:
    """`hc.simulator.launch(kernel, a, b, c)`, the call the reference's example makes, on the GPU."""
    import hc.simulator as sim
    from examples.b200_wmma_matmul import tiled_wmma_matmul_for

    a, b, c_sim = load_golden("sim_f16_m17_n19_k18_seed7")
    c = np.full(c_sim.shape, np.nan, np.float32)
    assert sim.launch(tiled_wmma_matmul_for("float16"), a, b, c) is None
    assert_close_to_oracle(c, a, b, expect=c_sim)


def test_reference_tests_own_tolerance_on_its_shapes() -> None:
    # tests/test_examples.py:22-33 of the reference uses atol=2e-6 against its blocked product;
    # the tensor-core result stays inside 1e-5 of it at these sizes (K <= 32, |values| <= 1).
    with np.load(load_golden.__globals__["GOLDEN"] / "blocked_reference.npz") as blocked:
        for name in blocked.files:
            a, b, _ = load_golden(name)
            np.testing.assert_allclose(gpu_wmma_matmul(a, b), blocked[name], rtol=0.0, atol=1e-5)


# ---------------------------------------------------------------- shape ladder ----------

DENSE_SHAPES = [
    (65, 1, 1), (65, 17, 3), (128, 256, 64), (128, 256, 16), (129, 257, 65), (127, 255, 63),
    (200, 200, 8), (256, 512, 200), (300, 520, 1000), (1024, 96, 130), (65, 3000, 100), (2048, 2048, 512),
]


@pytest.mark.parametrize("shape", DENSE_SHAPES)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_dense_ladder(shape: tuple[int, int, int], dtype: str) -> None:
    m, n, k = shape
    a, b = random_inputs(m, n, k, dtype)
    assert cuda.plan_gemm(m, n, k, dtype).variant == "dense"
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b)


SKINNY_SHAPES = [
    (1, 1, 1), (1, 128, 64), (8, 128, 64), (8, 129, 65), (7, 1000, 777), (16, 640, 4096), (17, 640, 1024),
    (32, 255, 300), (33, 512, 2048), (64, 3000, 520), (8, 4096, 8192), (3, 100, 16384),
]


@pytest.mark.parametrize("shape", SKINNY_SHAPES)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_skinny_ladder(shape: tuple[int, int, int], dtype: str) -> None:
    m, n, k = shape
    a, b = random_inputs(m, n, k, dtype, scale=0.25)
    # (NumPy buffers take the skinny kernel for every m <= 64; on device buffers 8 < m <= 64 with few
    # column blocks may go to the dense tiles shared among clusters instead.)
    assert cuda.plan_gemm(m, n, k, dtype, variant=cuda.VARIANT_SKINNY).variant == "skinny"
    assert cuda.plan_gemm(m, n, k, dtype).variant in ("skinny", "dense", "tiny")
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b)


TRANSPOSED_SHAPES = [
    (17, 19, 18), (128, 256, 64), (129, 257, 65), (300, 520, 1000), (1024, 96, 130), (513, 1000, 264),
    (2048, 2048, 512), (8, 129, 65), (7, 1000, 777), (33, 512, 2048), (64, 3000, 520), (8, 4096, 8192),
]


@pytest.mark.parametrize("shape", TRANSPOSED_SHAPES)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_b_stored_transposed(shape: tuple[int, int, int], dtype: str) -> None:
    """The Buffer[N, K] member of the kernel family (B handed over as stored, [n, k]): dense
    single-CTA, CTA-pair and skinny shapes, aligned and odd pitches."""
    m, n, k = shape
    a, b = random_inputs(m, n, k, dtype, scale=0.25)
    bt = np.ascontiguousarray(b.T)
    c = gpu_wmma_matmul(a, bt, b_transposed=True)
    assert_close_to_oracle(c, a, b)


WIDE_SHAPES = [(512, 256, 64), (513, 257, 130), (1100, 700, 300), (1024, 1024, 2048), (2500, 3000, 520), (300, 5000, 1000)]


@pytest.mark.parametrize("shape", WIDE_SHAPES)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float8_e4m3fn"])
def test_dense_wide_tiles(shape, dtype: str, gpu_ctx, monkeypatch) -> None:
    """The 512x256-tile kernel, forced onto shapes far smaller than it is chosen for so that edge
    tiles on every axis, a second accumulator half that lies wholly outside C, both layouts of B,
    fused operations, a 16-bit C and accumulation by TMA additions all run through it."""
    monkeypatch.setenv("HC_CUDA_DENSE_WIDE", "1")
    m, n, k = shape
    assert gpu_ctx.plan(m, n, k, dtype).tiles_m == -(-m // 512)
    a, b = float8_inputs(m, n, k, dtype) if dtype.startswith("float8") else random_inputs(m, n, k, dtype, scale=0.25)
    expect = cpu_ref.matmul_k_ascending(a, b)
    da, db, dbt = gpu_ctx.to_device(a), gpu_ctx.to_device(b), gpu_ctx.to_device(np.ascontiguousarray(b.T))
    guard = 3
    raw = cuda.DeviceBuffer(gpu_ctx, (m + 2 * guard, n + 8), np.float32)
    raw.fill_bytes(0xFF)
    dc = raw.window(guard, guard + m, 4, 4 + n)  # 16-byte aligned rows: the TMA-store path
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    whole = raw.to_numpy()
    c = np.ascontiguousarray(whole[guard : guard + m, 4 : 4 + n])
    assert_close_to_oracle(c, a, b, expect=expect)
    whole[guard : guard + m, 4 : 4 + n] = np.nan
    assert np.isnan(whole).all()  # nothing written outside C
    dct = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, dbt, dct, b_transposed=True)
    gpu_ctx.synchronize()
    assert np.array_equal(dct.to_numpy(), c)
    odd = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + 1)  # ordinary stores
    gpu_ctx.gemm(da, db, odd)
    gpu_ctx.synchronize()
    assert np.array_equal(odd.to_numpy(), c)
    bias = np.random.default_rng(4).standard_normal(n).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", 0.0))
    gpu_ctx.gemm(da, db, dct, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    assert_fused_close(dct.to_numpy(), a, b, epilogue=ops, bias=bias)
    c0 = np.random.default_rng(5).standard_normal((m, n)).astype(np.float32)
    dct.copy_from_host(c0)
    gpu_ctx.gemm(da, db, dct, accumulate=True)  # performed by the TMA stores
    gpu_ctx.synchronize()
    assert_fused_close(dct.to_numpy(), a, b, c0=c0)
    half = gpu_ctx.empty((m, n), np.float16)
    gpu_ctx.gemm(da, db, half)
    gpu_ctx.synchronize()
    assert np.array_equal(half.to_numpy(), c.astype(np.float16))
    monkeypatch.setenv("HC_CUDA_DENSE_WIDE", "0")
    gpu_ctx.gemm(da, db, dct)
    gpu_ctx.synchronize()
    assert_close_to_oracle(dct.to_numpy(), a, b, expect=expect)  # the 256x256 tiles, for comparison
    for buf in (da, db, dbt, raw, dct, odd, dbias, half):
        buf.free()


NARROW_SHAPES = [
    # one tile; ragged on every axis; more tiles than SMs (several rounds through both accumulators);
    # k below, at and across a ring stage; n below one tile
    (100, 300, 64), (128, 128, 128), (129, 130, 70), (1000, 1100, 520), (1536, 1536, 1536), (2100, 2300, 200), (333, 40, 500),
]


@pytest.mark.parametrize("shape", NARROW_SHAPES)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float8_e4m3fn"])
def test_dense_narrow_tiles(shape, dtype: str, gpu_ctx, monkeypatch) -> None:
    """The 128x128 tiles of the single-CTA dense kernel, forced onto every shape so that edge tiles on
    every axis, several rounds of tiles, both layouts of B, ordinary stores, fused operations, both
    kinds of accumulation and a 16-bit C run through them; same bits as the 256-wide tiles."""
    monkeypatch.setenv("HC_CUDA_DENSE_NARROW", "1")
    m, n, k = shape
    plan = gpu_ctx.plan(m, n, k, dtype, variant=cuda.VARIANT_DENSE)
    assert (plan.tile_n, plan.tiles_m, plan.tiles_n, plan.splits) == (128, -(-m // 128), -(-n // 128), 1)
    a, b = float8_inputs(m, n, k, dtype) if dtype.startswith("float8") else random_inputs(m, n, k, dtype, scale=0.25)
    expect = cpu_ref.matmul_k_ascending(a, b)
    da, db, dbt = gpu_ctx.to_device(a), gpu_ctx.to_device(b), gpu_ctx.to_device(np.ascontiguousarray(b.T))
    guard = 3
    raw = cuda.DeviceBuffer(gpu_ctx, (m + 2 * guard, n + 8), np.float32)
    raw.fill_bytes(0xFF)
    dc = raw.window(guard, guard + m, 4, 4 + n)  # 16-byte aligned rows: the TMA-store path
    gpu_ctx.gemm(da, db, dc, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    whole = raw.to_numpy()
    c = np.ascontiguousarray(whole[guard : guard + m, 4 : 4 + n])
    assert_close_to_oracle(c, a, b, expect=expect)
    whole[guard : guard + m, 4 : 4 + n] = np.nan
    assert np.isnan(whole).all()  # nothing written outside C
    dct = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, dbt, dct, b_transposed=True, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    assert np.array_equal(dct.to_numpy(), c)
    odd = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + 1)  # ordinary stores
    gpu_ctx.gemm(da, db, odd, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    assert np.array_equal(odd.to_numpy(), c)
    bias = np.random.default_rng(4).standard_normal(n).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", 0.0))
    gpu_ctx.gemm(da, db, dct, epilogue=ops, bias=dbias, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    assert_fused_close(dct.to_numpy(), a, b, epilogue=ops, bias=bias)
    c0 = np.random.default_rng(5).standard_normal((m, n)).astype(np.float32)
    dct.copy_from_host(c0)
    gpu_ctx.gemm(da, db, dct, accumulate=True, variant=cuda.VARIANT_DENSE)  # performed by the TMA stores
    gpu_ctx.synchronize()
    assert_fused_close(dct.to_numpy(), a, b, c0=c0)
    odd.copy_from_host(c0)
    gpu_ctx.gemm(da, db, odd, accumulate=True, epilogue=(("scale", 2.0),), variant=cuda.VARIANT_DENSE)  # reads C
    gpu_ctx.synchronize()
    assert_fused_close(odd.to_numpy(), a, b, c0=c0, epilogue=(("scale", 2.0),))
    half = gpu_ctx.empty((m, n), np.float16)
    gpu_ctx.gemm(da, db, half, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    assert np.array_equal(half.to_numpy(), c.astype(np.float16))
    monkeypatch.setenv("HC_CUDA_DENSE_NARROW", "0")
    assert gpu_ctx.plan(m, n, k, dtype, variant=cuda.VARIANT_DENSE).tile_n == 256
    gpu_ctx.gemm(da, db, dct, variant=cuda.VARIANT_DENSE)
    gpu_ctx.synchronize()
    if gpu_ctx.plan(m, n, k, dtype, variant=cuda.VARIANT_DENSE).splits == 1:
        assert np.array_equal(dct.to_numpy(), c)  # the 256-wide tiles: the same sums in the same order
    else:
        assert_close_to_oracle(dct.to_numpy(), a, b, expect=expect)
    for buf in (da, db, dbt, raw, dct, odd, dbias, half):
        buf.free()


FLOAT8_SHAPES = [
    # dense on single CTAs and CTA pairs, skinny with and without split-k; k below, at and across the
    # 128-element stage of the 8-bit kernels; odd pitches (repack) and aligned ones
    (17, 19, 18), (128, 256, 128), (129, 257, 130), (300, 520, 1000), (1024, 96, 257), (513, 1000, 264),
    (2048, 2048, 512), (8, 129, 65), (7, 1000, 777), (33, 512, 2048), (64, 3000, 520), (8, 4096, 8192),
]


def float8_inputs(m: int, n: int, k: int, dtype: str):
    """Values spread over the format's range, subnormals included (products stay exact in fp32)."""
    rng = np.random.default_rng([8, m, n, k])
    scales = [0.01, 0.25, 2.0] if dtype == "float8_e4m3fn" else [1e-4, 0.25, 16.0]
    a = (rng.standard_normal((m, k)) * rng.choice(scales, size=(m, k))).astype(np_dtype(dtype))
    b = (rng.standard_normal((k, n)) * rng.choice(scales, size=(k, n))).astype(np_dtype(dtype))
    return a, b


@pytest.mark.parametrize("shape", FLOAT8_SHAPES)
@pytest.mark.parametrize("dtype", ["float8_e4m3fn", "float8_e5m2"])
def test_float8_members(shape: tuple[int, int, int], dtype: str) -> None:
    """The float8 members of the kernel family, B stored [K, N] (transposed on the device before the
    product) and [N, K] (read where it stands): same tolerance rule as the 16-bit members."""
    m, n, k = shape
    a, b = float8_inputs(m, n, k, dtype)
    expect = cpu_ref.matmul_k_ascending(a, b)
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b, expect=expect)
    c_t = gpu_wmma_matmul(a, np.ascontiguousarray(b.T), b_transposed=True)
    assert_close_to_oracle(c_t, a, b, expect=expect)


def test_float8_fixtures_and_device_buffers(gpu_ctx) -> None:
    a, b, c_sim = load_golden("simf8_e4m3fn_m33_n17_k40_seed16")
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b, expect=c_sim)
    a, bt, c_sim = load_golden("simf8_e5m2_bt_m17_n19_k18_seed17")
    assert_close_to_oracle(gpu_wmma_matmul(a, bt, b_transposed=True), a, np.ascontiguousarray(bt.T), expect=c_sim)
    # Device buffers: both layouts of B give the same bits (same tiles, same k order), and a launch
    # with fused operations and a 16-bit C goes through the same epilogues as the 16-bit inputs.
    a, b = float8_inputs(384, 1100, 520, "float8_e4m3fn")
    da, db, dbt = gpu_ctx.to_device(a), gpu_ctx.to_device(b), gpu_ctx.to_device(np.ascontiguousarray(b.T))
    dc, dct = gpu_ctx.empty((384, 1100), np.float32), gpu_ctx.empty((384, 1100), np.float32)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.gemm(da, dbt, dct, b_transposed=True)
    gpu_ctx.synchronize()
    assert_close_to_oracle(dc.to_numpy(), a, b)
    assert np.array_equal(dc.to_numpy(), dct.to_numpy())
    bias = np.random.default_rng(3).standard_normal(1100).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", 0.0))
    gpu_ctx.gemm(da, db, dc, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    assert_fused_close(dc.to_numpy(), a, b, epilogue=ops, bias=bias)
    half = gpu_ctx.empty((384, 1100), np.float16)
    gpu_ctx.gemm(da, dbt, half, b_transposed=True)
    gpu_ctx.synchronize()
    assert np.array_equal(half.to_numpy(), dct.to_numpy().astype(np.float16))
    for buf in (da, db, dbt, dc, dct, dbias, half):
        buf.free()


def test_transposed_b_fixture_and_device_buffers(gpu_ctx) -> None:
    a, bt, c_sim = load_golden("simbt_f16_m17_n19_k18_seed9")
    assert_close_to_oracle(gpu_wmma_matmul(a, bt, b_transposed=True), a, np.ascontiguousarray(bt.T), expect=c_sim)
    a, b = random_inputs(384, 1100, 520, "float16")
    bt = np.ascontiguousarray(b.T)
    da, dbt = gpu_ctx.to_device(a), gpu_ctx.to_device(bt)
    dc = gpu_ctx.empty((384, 1100), np.float32)
    compiled_for("float16", None, True)(da, dbt, dc)
    expect = gpu_wmma_matmul(a, b)
    assert_close_to_oracle(dc.to_numpy(), a, b)
    # Same tiles and k order as the [K, N] kernel: the tensor cores see the same operands.
    assert np.array_equal(dc.to_numpy(), expect)


# ---------------------------------------------------------------- around the k-loop -----


def assert_fused_close(out, a, b, *, c0=None, epilogue=(), bias=None, use_oracle=True) -> None:
    """`out` against ops(C0 + A.B) in float64, with the benchmark's element bound carried through
    the element-wise operations (each is 1-Lipschitz up to its scale factor), and against the
    oracle's fp32 restatement under the same bound."""
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    ref = a64 @ b64
    bound = np.abs(a64) @ np.abs(b64)
    if c0 is not None:
        ref = ref + c0
        bound = bound + np.abs(c0)
    for op in epilogue:
        if op[0] == "scale":
            ref, bound = ref * np.float32(op[1]), bound * abs(op[1])
        elif op[0] == "add":
            ref, bound = ref + np.float32(op[1]), bound + abs(op[1])
        elif op[0] == "bias":
            ref, bound = ref + bias[None, :], bound + np.abs(bias)[None, :]
        elif op[0] == "max":
            ref = np.maximum(ref, np.float32(op[1]))
        else:
            ref = np.minimum(ref, np.float32(op[1]))
    assert out.shape == ref.shape and out.dtype == np.float32 and np.isfinite(out).all()
    diff = np.abs(out - ref)
    assert (diff <= ELEMENT_RATIO * bound + 1e-30).all(), float((diff / np.maximum(bound, 1e-30)).max())
    assert np.linalg.norm(diff) <= REL_FROBENIUS * max(np.linalg.norm(ref), 1e-30)
    if use_oracle:
        expect = cpu_ref.matmul_fused(a, b, c0=c0, epilogue=epilogue, bias=bias)
        assert (np.abs(out.astype(np.float64) - expect) <= ELEMENT_RATIO * bound + 1e-30).all()


def test_accumulating_and_fused_fixtures() -> None:
    """The members the reference simulator executed (host arrays through the compiled handles)."""
    golden = load_golden.__globals__["GOLDEN"]
    a, b, c_sim = load_golden("simacc_f16_m17_n19_k18_seed11")
    with np.load(golden / "simacc_f16_m17_n19_k18_seed11.npz") as data:
        c0 = data["c0"]
    c = c0.copy()
    compiled_for("float16", None, False, "accumulate")(a, b, c)
    assert_fused_close(c, a, b, c0=c0)
    np.testing.assert_allclose(c, c_sim, rtol=0, atol=2e-6)  # the reference test's own tolerance
    strided = np.zeros((17, 40), np.float32)[:, ::2][:, :19]  # not row-major: staged through a copy
    strided[...] = c0
    compiled_for("float16", None, False, "accumulate")(a, b, strided)
    assert np.array_equal(strided, c)

    a, b, c_sim = load_golden("simfused_bf16_m33_n17_k40_seed12")
    with np.load(golden / "simfused_bf16_m33_n17_k40_seed12.npz") as data:
        bias = data["bias"]
    c = np.full((33, 17), np.float32(-7.0))
    compiled_for("bfloat16", None, False, "fused")(a, b, c, bias)
    assert_fused_close(c, a, b, epilogue=(("scale", 0.125), ("bias",), ("max", 0.0)), bias=bias)
    np.testing.assert_allclose(c, c_sim, rtol=0, atol=2e-6)
    assert np.array_equal(c == 0, c_sim == 0)  # clipped in the same places


def test_fused_fixture_with_infinities_and_nan(gpu_ctx) -> None:
    """NaN and infinities go through the fused maximum / minimum as in NumPy (and so in the
    reference simulator): NaN stays NaN, -inf is clipped, +inf stays. Host arrays through the
    handle (dense kernel) and device buffers through the skinny and dense kernels."""
    golden = load_golden.__globals__["GOLDEN"]
    a, b, c_sim = load_golden("simfusednan_bf16_m33_n17_k40_seed14")
    with np.load(golden / "simfusednan_bf16_m33_n17_k40_seed14.npz") as data:
        bias = data["bias"]
    ops = (("scale", 0.125), ("bias",), ("max", 0.0))

    def check(c: np.ndarray) -> None:
        assert np.array_equal(np.isnan(c), np.isnan(c_sim))
        assert np.array_equal(np.isposinf(c), np.isposinf(c_sim)) and not np.isneginf(c).any()
        finite = np.isfinite(c_sim)
        np.testing.assert_allclose(c[finite], c_sim[finite], rtol=0, atol=2e-6)
        assert np.array_equal(c[finite] == 0, c_sim[finite] == 0)

    c = np.full((33, 17), np.float32(-7.0))
    compiled_for("bfloat16", None, False, "fused")(a, b, c, bias)
    check(c)
    da, db, dbias = gpu_ctx.to_device(a), gpu_ctx.to_device(b), gpu_ctx.to_device(bias)
    for variant in (cuda.VARIANT_SKINNY, cuda.VARIANT_DENSE):
        dc = gpu_ctx.empty((33, 17), np.float32)
        gpu_ctx.gemm(da, db, dc, variant=variant, epilogue=ops, bias=dbias)
        check(dc.to_numpy())
        gpu_ctx.gemm(da, db, dc, variant=variant, epilogue=(("min", 1.0),))
        assert np.array_equal(np.isnan(dc.to_numpy()), np.isnan(c_sim))
        dc.free()
    for buf in (da, db, dbias):
        buf.free()


FUSED_SHAPES = [
    # dense on single CTAs / CTA pairs, aligned and odd pitches; skinny with and without split-k
    (128, 256, 64, 0), (300, 520, 136, 0), (513, 1001, 264, 3), (1024, 1024, 256, 0), (2050, 2051, 130, 1),
    (8, 4096, 512, 0), (8, 129, 2048, 0), (33, 515, 1024, 5), (64, 16384, 256, 0),
]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", FUSED_SHAPES)
def test_accumulate_and_fused_operations_on_device_buffers(shape, dtype: str, gpu_ctx) -> None:
    m, n, k, pad = shape
    a, b = random_inputs(m, n, k, dtype, scale=0.25)
    rng = np.random.default_rng([m, n, k, 77])
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dbias = gpu_ctx.to_device(bias)
    dc = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + pad)
    cases = [
        dict(accumulate=True),
        dict(epilogue=(("scale", 0.5), ("bias",), ("max", 0.0))),
        dict(accumulate=True, epilogue=(("bias",), ("scale", -2.0), ("min", 1.0), ("add", 0.25))),
    ]
    for case in cases:
        dc.copy_from_host(c0)
        gpu_ctx.gemm(da, db, dc, bias=dbias if any(op[0] == "bias" for op in case.get("epilogue", ())) else None,
                     **case)
        gpu_ctx.synchronize()
        assert_fused_close(dc.to_numpy(), a, b, c0=c0 if case.get("accumulate") else None,
                           epilogue=case.get("epilogue", ()), bias=bias, use_oracle=m * n * k <= 1 << 28)
    # Two accumulating launches in a row add the product twice.
    dc.copy_from_host(c0)
    gpu_ctx.gemm(da, db, dc, accumulate=True)
    gpu_ctx.gemm(da, db, dc, accumulate=True)
    gpu_ctx.synchronize()
    twice = dc.to_numpy()
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    product = dc.to_numpy()
    np.testing.assert_allclose(twice, c0 + 2 * product, rtol=1e-5, atol=1e-5)
    for buf in (da, db, dc, dbias):
        buf.free()


def test_fused_operations_on_host_arrays(gpu_ctx) -> None:
    """Host buffers: C and the bias travel to the device first; the large case takes the
    pipelined row-panel path, where each panel's rows of C arrive before its product."""
    for m, n, k in ((200, 300, 264), (2048, 2304, 2048), (16, 5000, 1024)):
        a, b = random_inputs(m, n, k, "float16", scale=0.25)
        rng = np.random.default_rng([m, n, k, 78])
        c0 = rng.standard_normal((m, n)).astype(np.float32)
        bias = rng.standard_normal((n,)).astype(np.float32)
        ops = (("scale", 0.5), ("bias",), ("max", -0.25))
        c = c0.copy()
        gpu_ctx.gemm_host(a, b, c, accumulate=True, epilogue=ops, bias=bias)
        assert_fused_close(c, a, b, c0=c0, epilogue=ops, bias=bias, use_oracle=m * n * k <= 1 << 28)


def test_fused_operations_with_k_zero(gpu_ctx) -> None:
    """No product: the launch whose k-loop runs zero times still applies what surrounds it."""
    rng = np.random.default_rng(5)
    m, n = 37, 129
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    a = np.zeros((m, 0), np.float16)
    b = np.zeros((0, n), np.float16)
    c = c0.copy()
    gpu_ctx.gemm_host(a, b, c, accumulate=True)
    assert np.array_equal(c, c0)
    gpu_ctx.gemm_host(a, b, c, accumulate=True, epilogue=(("scale", 2.0), ("bias",)), bias=bias)
    assert np.array_equal(c, c0 * np.float32(2.0) + bias[None, :])
    gpu_ctx.gemm_host(a, b, c, epilogue=(("add", 3.0), ("min", 1.0)))
    assert np.array_equal(c, np.full((m, n), np.float32(1.0)))
    dc = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + 3)
    dc.copy_from_host(c0)
    da, db = cuda.DeviceBuffer(gpu_ctx, (m, 0), np.float16, ld=8), cuda.DeviceBuffer(gpu_ctx, (0, n), np.float16, ld=n)
    gpu_ctx.gemm(da, db, dc, accumulate=True, epilogue=(("max", 0.0),))
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), np.maximum(c0, np.float32(0)))
    assert compiled_for("float16", None, False, "fused")(a, b, c, bias) is None
    assert np.array_equal(c, np.maximum(np.zeros((m, n), np.float32) * np.float32(0.125) + bias[None, :], 0))


DENSE_SPLIT_SHAPES = [
    # few tiles, long k: the plan splits k over the idle CTAs (single CTAs, CTA pairs, odd pitches)
    (128, 2048, 4096, 0), (96, 1000, 8192, 3), (256, 1024, 8192, 0), (300, 700, 6000, 1), (512, 512, 16384, 0),
    (256, 256, 32768, 0), (1024, 1024, 4096, 0), (130, 258, 2050, 5),
]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", DENSE_SPLIT_SHAPES)
def test_dense_split_k(shape, dtype: str, gpu_ctx) -> None:
    """Dense shapes with few tiles: partial tiles per k range, added in split order by whichever
    unit finishes last. Checked against the oracle, for determinism, and with the fused members."""
    m, n, k, pad = shape
    plan = gpu_ctx.plan(m, n, k, dtype, ldc=n + pad)
    assert plan.variant == "dense" and plan.splits > 1, plan
    a, b = random_inputs(m, n, k, dtype, scale=0.25)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + pad)
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    first = dc.to_numpy()
    assert_close_to_oracle(first, a, b)
    for _ in range(3):  # the counters are back at zero and the order of arrival does not matter
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(da, db, dc)
        gpu_ctx.synchronize()
        assert np.array_equal(dc.to_numpy(), first)
    rng = np.random.default_rng([m, n, k, 5])
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", -0.5))
    dc.copy_from_host(c0)
    gpu_ctx.gemm(da, db, dc, accumulate=True, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    assert_fused_close(dc.to_numpy(), a, b, c0=c0, epilogue=ops, bias=bias, use_oracle=m * n * k <= 1 << 28)
    bt = gpu_ctx.to_device(np.ascontiguousarray(b.T))
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, bt, dc, b_transposed=True)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), first)
    for buf in (da, db, dc, dbias, bt):
        buf.free()


CLUSTER_CASES = [
    # (m, n, k, cluster size, clusters per tile)
    (256, 256, 32768, 8, 7), (256, 256, 32768, 16, 3), (512, 512, 16384, 4, 4), (300, 500, 4100, 16, 1),
    (300, 500, 4100, 2, 6), (128, 256, 1024, 2, 1), (130, 264, 2048, 8, 2), (384, 768, 12288, 4, 3),
    (129, 520, 704, 4, 2),  # eleven k-blocks over eight CTAs: ranges of one and two blocks
]


@pytest.mark.parametrize("case", CLUSTER_CASES)
def test_dense_cluster_form(case, gpu_ctx, monkeypatch) -> None:
    """Few tiles, long k, a float32 C that TMA can address: the CTAs that share a tile are one or several
    thread-block clusters and add their partial tiles through distributed shared memory (and, between
    clusters, through partial sums in global memory). Every cluster size and number of clusters per tile
    gives the oracle's product, bit-identical from launch to launch, with the fused members and float8."""
    m, n, k, size, groups = case
    monkeypatch.setenv("HC_CUDA_DENSE_CLUSTER", str(size))
    monkeypatch.setenv("HC_CUDA_DENSE_CLUSTER_GROUPS", str(groups))
    plan = gpu_ctx.plan(m, n, k, "float16")
    assert (plan.variant, plan.cluster_size, plan.splits) == ("dense", size, size * groups), plan
    assert plan.grid == plan.tiles_m * plan.tiles_n * size * groups and plan.tiles_m == -(-m // 128)
    a, b = random_inputs(m, n, k, "float16", scale=0.25)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((m, n), np.float32)
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    first = dc.to_numpy()
    assert_close_to_oracle(first, a, b)
    for _ in range(3):  # the order of arrival does not matter and the counters are back at zero
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(da, db, dc)
        gpu_ctx.synchronize()
        assert np.array_equal(dc.to_numpy(), first)
    rng = np.random.default_rng([m, n, k, 9])
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", -0.5), ("min", 2.0))
    for accumulate, epilogue in ((True, ()), (True, ops), (False, ops)):
        dc.copy_from_host(c0)
        gpu_ctx.gemm(da, db, dc, accumulate=accumulate, epilogue=epilogue, bias=dbias if epilogue else None)
        gpu_ctx.synchronize()
        assert_fused_close(dc.to_numpy(), a, b, c0=c0 if accumulate else None, epilogue=epilogue, bias=bias,
                           use_oracle=m * n * k <= 1 << 28)
    bt = gpu_ctx.to_device(np.ascontiguousarray(b.T))
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, bt, dc, b_transposed=True)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), first)
    # The same product without clusters: equal up to the order of the partial sums.
    monkeypatch.setenv("HC_CUDA_DENSE_CLUSTER", "0")
    assert gpu_ctx.plan(m, n, k, "float16").cluster_size == 0
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    np.testing.assert_allclose(dc.to_numpy(), first, rtol=0, atol=2e-3)
    # float8 operands (twice the k per stage) and bfloat16.
    monkeypatch.setenv("HC_CUDA_DENSE_CLUSTER", str(size))
    for dtype in ("float8_e4m3fn", "bfloat16"):
        if dtype.startswith("float8"):
            a8, b8 = float8_inputs(m, n, k, dtype)
            b8 = np.ascontiguousarray(b8.T)  # [N, K]: no transposition launch
        else:
            a8, b8 = random_inputs(m, n, k, dtype, scale=0.25)
        if gpu_ctx.plan(m, n, k, dtype, b_transposed=dtype.startswith("float8")).cluster_size != size:
            continue  # too few k-blocks of 128 for this many CTAs
        d8a, d8b = gpu_ctx.to_device(a8), gpu_ctx.to_device(b8)
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(d8a, d8b, dc, b_transposed=dtype.startswith("float8"))
        gpu_ctx.synchronize()
        assert_close_to_oracle(dc.to_numpy(), a8, b8.T if dtype.startswith("float8") else b8)
        d8a.free(), d8b.free()
    for buf in (da, db, dc, dbias, bt):
        buf.free()


def test_dense_cluster_form_is_not_chosen_where_it_cannot_store(gpu_ctx) -> None:
    """A 16-bit C, a pitch that TMA cannot address and push targets keep the counter-based split."""
    assert gpu_ctx.plan(256, 256, 32768, "float16").cluster_size > 0
    assert gpu_ctx.plan(256, 256, 32768, "float16", ldc=259).cluster_size == 0
    assert gpu_ctx.plan(256, 256, 32768, "float16", c_dtype="bfloat16").cluster_size == 0


def test_dense_split_k_forced(gpu_ctx, monkeypatch) -> None:
    """Split counts the plan would not choose, on a shape with many tiles per CTA (units of one tile
    land on different CTAs in different rounds)."""
    m, n, k = 1100, 2300, 1536
    a, b = random_inputs(m, n, k, "float16", scale=0.25)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    unsplit = dc.to_numpy()
    for mode in ("single", "pair"):
        monkeypatch.setenv("HC_CUDA_DENSE_MODE", mode)
        for splits in (2, 3, 5):
            monkeypatch.setenv("HC_CUDA_DENSE_SPLITS", str(splits))
            assert gpu_ctx.plan(m, n, k, "float16").splits == splits
            dc.fill_bytes(0xFF)
            gpu_ctx.gemm(da, db, dc)
            gpu_ctx.synchronize()
            out = dc.to_numpy()
            assert_close_to_oracle(out, a, b)
            np.testing.assert_allclose(out, unsplit, rtol=0, atol=1e-4)


@pytest.mark.parametrize("shape", [(4864, 1024, 8192), (2432, 2048, 8200), (9600, 512, 8192)])
def test_dense_split_of_the_last_round(shape, gpu_ctx, monkeypatch) -> None:
    """More tiles than CTAs with a small remainder: the tiles of the last, partly filled round
    are split over k, the earlier ones are not."""
    m, n, k = shape
    plan = gpu_ctx.plan(m, n, k, "float16")
    tiles = plan.tiles_m * plan.tiles_n
    assert plan.splits > 1 and 0 < plan.first_split_tile < tiles, plan
    a, b = random_inputs(m, n, k, "float16", scale=0.25)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((m, n), np.float32)
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    out = dc.to_numpy()
    rows = _sample_rows(m)
    assert workloads.check_against_float64(out, a, b, rows=rows)["ok"]
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), out)
    monkeypatch.setenv("HC_CUDA_DENSE_SPLITS", "1")
    assert gpu_ctx.plan(m, n, k, "float16").splits == 1
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    whole = dc.to_numpy()
    np.testing.assert_allclose(out, whole, rtol=0, atol=2e-3)  # fp32 reassociation over k = 8192
    assert (out != whole).any()  # the split tiles were added in a different order
    for buf in (da, db, dc):
        buf.free()


def assert_narrow_close(out, a, b, *, epilogue=(), bias=None) -> None:
    """A 16-bit C against the float64 reference: the benchmark's element bound plus half a unit in
    the last place of the output type."""
    eps = 2.0 ** -11 if out.dtype == np.float16 else 2.0 ** -8
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    ref = a64 @ b64
    bound = np.abs(a64) @ np.abs(b64)
    for op in epilogue:
        if op[0] == "scale":
            ref, bound = ref * np.float32(op[1]), bound * abs(op[1])
        elif op[0] == "add":
            ref, bound = ref + np.float32(op[1]), bound + abs(op[1])
        elif op[0] == "bias":
            ref, bound = ref + bias[None, :], bound + np.abs(bias)[None, :]
        elif op[0] == "max":
            ref = np.maximum(ref, np.float32(op[1]))
        else:
            ref = np.minimum(ref, np.float32(op[1]))
    got = out.astype(np.float64)
    assert np.isfinite(got).all()
    diff = np.abs(got - ref)
    assert (diff <= ELEMENT_RATIO * bound + eps * np.abs(ref) + 1e-30).all(), float(diff.max())


NARROW_SHAPES = [
    # TMA path (pitch a multiple of 8 elements), plain path (odd pitch), skinny, split-k, edges
    (128, 256, 64, 0), (300, 520, 136, 0), (513, 1001, 264, 3), (1024, 1024, 256, 0), (2050, 2051, 130, 1),
    (8, 4096, 512, 0), (33, 515, 1024, 5), (64, 16384, 256, 0), (128, 2048, 4096, 0), (300, 700, 6000, 1),
]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", NARROW_SHAPES)
def test_16_bit_c(shape, dtype: str, gpu_ctx) -> None:
    m, n, k, pad = shape
    a, b = random_inputs(m, n, k, dtype, scale=0.25)
    out_type = np_dtype(dtype)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = cuda.DeviceBuffer(gpu_ctx, (m, n), out_type, ld=n + pad)
    d32 = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, db, d32)
    dc.fill_bytes(0x7F)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    out = dc.to_numpy()
    assert out.dtype == np.dtype(out_type)
    assert_narrow_close(out, a, b)
    # Exactly the float32 result rounded to nearest even where both take the same plan (so the same
    # float32 bits); a split float32 product may instead share its tiles among clusters, which adds
    # the partial sums in another order.
    same_plan = gpu_ctx.plan(m, n, k, dtype).cluster_size == gpu_ctx.plan(m, n, k, dtype, ldc=n + pad, c_dtype=dtype).cluster_size
    if same_plan:
        assert np.array_equal(out.view(np.uint16), d32.to_numpy().astype(out_type).view(np.uint16))
    else:
        np.testing.assert_allclose(out.astype(np.float32), d32.to_numpy(), rtol=2.0 ** -7, atol=1e-3)
    bias = np.linspace(-1, 1, n).astype(np.float32)
    dbias = gpu_ctx.to_device(bias)
    ops = (("scale", 0.5), ("bias",), ("max", 0.0))
    gpu_ctx.gemm(da, db, dc, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    assert_narrow_close(dc.to_numpy(), a, b, epilogue=ops, bias=bias)
    with pytest.raises(DeviceError, match="accumulate needs a float32 C"):
        gpu_ctx.gemm(da, db, dc, accumulate=True)
    for buf in (da, db, dc, d32, dbias):
        buf.free()


def test_narrow_member_fixture_and_host_arrays(gpu_ctx) -> None:
    import ml_dtypes

    a, b, c_sim32 = load_golden("simnarrow_bf16_m33_n17_k40_seed13")
    c = np.full((33, 17), 7.0).astype(ml_dtypes.bfloat16)
    compiled_for("bfloat16", None, False, "narrow")(a, b, c)
    assert_narrow_close(c, a, b)
    # One unit in the last place of bfloat16 at most, where the float32 sums straddle a rounding point.
    assert np.abs(c.astype(np.float32) - c_sim32).max() <= 2.0 ** -7 * np.abs(c_sim32).max()
    assert (c.astype(np.float32) == c_sim32).mean() > 0.98
    # The type of C is independent of the operands' type.
    a, b = random_inputs(200, 264, 136, "bfloat16", scale=0.25)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((200, 264), np.float16)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert_narrow_close(dc.to_numpy(), a, b)
    # k == 0 and the large host paths (pageable: row panels; pinned: alternating panels).
    z = np.full((5, 9), 3.0).astype(np.float16)
    gpu_ctx.gemm_host(np.zeros((5, 0), np.float16), np.zeros((0, 9), np.float16), z, epilogue=(("add", 1.5),))
    assert np.array_equal(z, np.full((5, 9), 1.5, np.float16))
    m, n, k = 3000, 4100, 1100
    a, b = random_inputs(m, n, k, "float16", scale=0.25)
    c_store = np.full((m + 2, n + 4), np.float16(9.0))
    gpu_ctx.gemm_host(a, b, c_store[1:-1, 2:-2])
    pa, pb = cuda.pinned_empty(a.shape, a.dtype), cuda.pinned_empty(b.shape, b.dtype)
    pc = cuda.pinned_empty((m, n), np.float16)
    pa[...], pb[...] = a, b
    gpu_ctx.gemm_host(pa, pb, pc)
    assert np.array_equal(pc, c_store[1:-1, 2:-2])
    assert (c_store[0] == 9).all() and (c_store[-1] == 9).all() and (c_store[:, :2] == 9).all() and (c_store[:, -2:] == 9).all()
    assert_narrow_close(np.ascontiguousarray(pc[:64]), a[:64], b)


def test_concurrent_calls_from_threads(gpu_ctx) -> None:
    """Launches from several host threads at once, as the reference tests its simulator
    (tests/test_simulator.py:1113-1125): calls on one context are serialised inside the library,
    contexts of their own run side by side; every thread gets its own product."""
    import threading

    handle = compiled_for("float16")
    shapes = [(200 + 37 * i, 300 + 11 * i, 136 + 64 * i) for i in range(6)]
    problems = [random_inputs(m, n, k, "float16", seed=i, scale=0.25) for i, (m, n, k) in enumerate(shapes)]
    results: list = [None] * len(shapes)
    errors: list = []

    def through_the_handle(i: int) -> None:
        try:
            a, b = problems[i]
            for _ in range(5):
                c = np.full((a.shape[0], b.shape[1]), np.nan, np.float32)
                handle(a, b, c)
                results[i] = c
        except Exception as exc:  # noqa: BLE001 - reported below
            errors.append((i, exc))

    def through_an_own_context(i: int) -> None:
        try:
            ctx = cuda.Context(0)
            a, b = problems[i]
            da, db = ctx.to_device(a), ctx.to_device(b)
            dc = ctx.empty((a.shape[0], b.shape[1]), np.float32)
            for _ in range(5):
                ctx.gemm(da, db, dc)
                ctx.synchronize()
            results[i] = dc.to_numpy()
            ctx.close()
        except Exception as exc:  # noqa: BLE001
            errors.append((i, exc))

    threads = [threading.Thread(target=through_the_handle if i % 2 == 0 else through_an_own_context, args=(i,))
               for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    for (a, b), c in zip(problems, results):
        assert c is not None
        assert_close_to_oracle(c, a, b)


def test_bound_gemm_launches_like_gemm(gpu_ctx) -> None:
    a, b = random_inputs(300, 520, 136, "float16", scale=0.25)
    bias = np.linspace(-1, 1, 520).astype(np.float32)
    da, db, dbias = gpu_ctx.to_device(a), gpu_ctx.to_device(b), gpu_ctx.to_device(bias)
    dc, dd = gpu_ctx.empty((300, 520), np.float32), gpu_ctx.empty((300, 520), np.float32)
    ops = (("bias",), ("max", 0.0))
    gpu_ctx.gemm(da, db, dc, epilogue=ops, bias=dbias)
    bound = gpu_ctx.bind_gemm(da, db, dd, epilogue=ops, bias=dbias)
    for _ in range(3):
        dd.fill_bytes(0xFF)
        bound.launch()
        gpu_ctx.synchronize()
        assert np.array_equal(dd.to_numpy(), dc.to_numpy())
    with pytest.raises(ValueError, match="bias must be a float32 buffer of n values"):
        gpu_ctx.bind_gemm(da, db, dd, epilogue=ops, bias=da)


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes(seed: int, gpu_ctx) -> None:
    """Seeded random shapes, small and awkward ones included, in both element types and both B
    layouts, on device buffers with random extra pitch: every result against float64 and the
    oracle's bound. Catches tile-scheduling and edge-predication corner cases the fixed ladders
    do not name."""
    rng = np.random.default_rng(1000 + seed)
    for _ in range(12):
        kind = rng.integers(0, 4)
        if kind == 0:
            m, n, k = (int(rng.integers(1, 65)), int(rng.integers(1, 2000)), int(rng.integers(1, 3000)))
        elif kind == 1:
            m, n, k = (int(rng.integers(65, 700)), int(rng.integers(1, 1500)), int(rng.integers(1, 600)))
        elif kind == 2:
            m, n, k = (int(rng.integers(1, 300)), int(rng.integers(1, 300)), int(rng.integers(1, 300)))
        else:
            m, n, k = (int(rng.integers(700, 2600)), int(rng.integers(1500, 4200)), int(rng.integers(16, 200)))
        dtype = "bfloat16" if rng.integers(0, 2) else "float16"
        transposed = bool(rng.integers(0, 2))
        a = (rng.standard_normal((m, k)) * 0.5).astype(np_dtype(dtype))
        b = (rng.standard_normal((k, n)) * 0.5).astype(np_dtype(dtype))
        b_stored = np.ascontiguousarray(b.T) if transposed else b
        pads = [int(x) for x in rng.choice([0, 0, 1, 3, 8, 64], size=3)]
        da = cuda.DeviceBuffer(gpu_ctx, a.shape, a.dtype, ld=a.shape[1] + pads[0])
        db = cuda.DeviceBuffer(gpu_ctx, b_stored.shape, b.dtype, ld=b_stored.shape[1] + pads[1])
        dc = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + pads[2])
        da.copy_from_host(a)
        db.copy_from_host(b_stored)
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(da, db, dc, b_transposed=transposed)
        gpu_ctx.synchronize()
        c = dc.to_numpy()
        report = workloads.check_against_float64(c, a, b)
        assert report["ok"], (m, n, k, dtype, transposed, pads, report)
        for buf in (da, db, dc):
            buf.free()


def test_skinny_split_k_is_deterministic(gpu_ctx) -> None:
    a, b = random_inputs(8, 2048, 8192, "float16", scale=0.1)
    assert gpu_ctx.plan(8, 2048, 8192, "float16").splits > 1
    first = gpu_wmma_matmul(a, b)
    for _ in range(5):
        assert np.array_equal(first, gpu_wmma_matmul(a, b))


def test_forced_variants_agree(gpu_ctx) -> None:
    a, b = random_inputs(48, 700, 900, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    outs = []
    for variant in (cuda.VARIANT_DENSE, cuda.VARIANT_SKINNY):
        dc = gpu_ctx.empty((48, 700), np.float32)
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(da, db, dc, variant=variant)
        gpu_ctx.synchronize()
        outs.append(dc.to_numpy())
        assert_close_to_oracle(outs[-1], a, b)
    assert np.allclose(outs[0], outs[1], rtol=0, atol=1e-3)


def test_lowering_hook_chooses_the_kernel_family() -> None:
    """A kernel whose intrinsic registers `.lower(target="nvidia-sm100a")` returning
    {"variant": "dense"} runs the dense kernels even for a shape that would go to the skinny one."""
    from examples.b200_wmma_matmul import build_tiled_wmma_matmul
    from hc._pipeline import NVIDIA_SM100A, _reachable_callables

    kern = build_tiled_wmma_matmul(np.float16)
    mma = next(fn for fn in _reachable_callables(kern) if hasattr(fn, "__hc_intrinsic__"))
    mma.lower(target=NVIDIA_SM100A)(lambda ctx, *args, **kwargs: {"variant": "dense"})
    handle = hc.compile(kern, target=NVIDIA_SM100A)
    assert handle.plan.lowering == {"variant": "dense"}
    a, b = random_inputs(40, 520, 300, "float16")
    c = np.zeros((40, 520), np.float32)
    handle(a, b, c)
    assert_close_to_oracle(c, a, b)
    # The skinny kernel (default for m <= 64) sums in a different order: close, not identical.
    assert np.allclose(c, gpu_wmma_matmul(a, b), rtol=0, atol=1e-3)


# ---------------------------------------------------------------- edges ------------------


def test_zero_k_writes_zeros_and_empty_shapes_write_nothing() -> None:
    handle = compiled_for("float16")
    c = np.full((5, 7), 3.0, np.float32)
    handle(np.zeros((5, 0), np.float16), np.zeros((0, 7), np.float16), c)
    assert not c.any()
    c = np.full((0, 7), 3.0, np.float32)
    handle(np.zeros((0, 4), np.float16), np.zeros((4, 7), np.float16), c)
    c = np.full((5, 0), 3.0, np.float32)
    handle(np.zeros((5, 4), np.float16), np.zeros((4, 0), np.float16), c)


@pytest.mark.parametrize("frame", [(12, 4), (13, 3), (1, 1), (35, 0)])
@pytest.mark.parametrize("shape", [(130, 300, 70), (9, 300, 130), (515, 770, 96)])
def test_nothing_outside_c_is_written(gpu_ctx, shape, frame) -> None:
    """C sits inside a wider device matrix filled with a sentinel; after the launch only the
    M x N window may differ, and A and B must be unchanged. The frames cover a 16-byte-aligned
    window as well as odd pitches and bases (rows that start on arbitrary 4-byte boundaries)."""
    m, n, k = shape
    pad, col_off = frame
    a, b = random_inputs(m, n, k, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    frame_buf = cuda.DeviceBuffer(gpu_ctx, (m + 2, n + pad), np.float32)
    frame_buf.fill_bytes(0x7F)
    window = frame_buf.window(1, m + 1, col_off, n + col_off)  # one row down, col_off columns in
    gpu_ctx.gemm(da, db, window)
    gpu_ctx.synchronize()
    whole = frame_buf.to_numpy()
    sentinel = np.frombuffer(b"\x7f\x7f\x7f\x7f", np.float32)[0]
    inside = whole[1 : m + 1, col_off : n + col_off]
    assert_close_to_oracle(np.ascontiguousarray(inside), a, b)
    mask = np.ones_like(whole, bool)
    mask[1 : m + 1, col_off : n + col_off] = False
    assert (whole[mask].view(np.uint32) == sentinel.view(np.uint32)).all()
    assert np.array_equal(da.to_numpy().view(np.uint16), a.view(np.uint16))
    assert np.array_equal(db.to_numpy().view(np.uint16), b.view(np.uint16))


def test_unaligned_pitches_and_bases_on_device(gpu_ctx) -> None:
    """Odd pitches (K=1031-like) and a base that is only 2-byte aligned take the repack path (one copy launch for both operands, then the GEMM)."""
    m, n, k = 150, 333, 77
    a, b = random_inputs(m, n, k, "bfloat16")
    plan = gpu_ctx.plan(m, n, k, "bfloat16")
    assert plan.repack_a and plan.repack_b and plan.kernel_launches == 2
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert_close_to_oracle(dc.to_numpy(), a, b)


def test_numpy_views_and_strides() -> None:
    rng = np.random.default_rng(3)
    big_a = rng.standard_normal((100, 200)).astype(np.float16)
    big_b = rng.standard_normal((200, 300)).astype(np.float16)
    a = big_a[10:75, 8:136]            # row-major view with a pitch
    b = big_b[8:136, 20:290]
    c_store = np.full((65, 400), np.nan, np.float32)
    c = c_store[:, 100:370]
    compiled_for("float16")(a, b, c)
    assert_close_to_oracle(np.ascontiguousarray(c), np.ascontiguousarray(a), np.ascontiguousarray(b))
    assert np.isnan(c_store[:, :100]).all() and np.isnan(c_store[:, 370:]).all()
    at = np.ascontiguousarray(a).T.copy().T  # column-major A: staged through a contiguous copy
    assert not at.flags.c_contiguous
    c2 = np.zeros((65, 270), np.float32)
    compiled_for("float16")(at, b, c2)
    assert np.array_equal(c2, np.ascontiguousarray(c))
    c3 = np.zeros((270, 65), np.float32).T  # column-major C: written through a staged copy
    compiled_for("float16")(a, b, c3)
    assert np.array_equal(c3, c2)


@pytest.mark.parametrize("b_transposed", [False, True])
def test_large_product_on_pinned_buffers_in_alternating_panels(gpu_ctx, b_transposed: bool) -> None:
    """Pinned host arrays: A and B travel in alternating panels and C returns block by block. The
    result must equal the device-buffer path bit for bit, with and without fused operations, and
    leave the surroundings of a strided C alone."""
    m, n, k = 3000, 4100, 1100
    a, b = random_inputs(m, n, k, "float16", scale=0.25)
    b_host = np.ascontiguousarray(b.T) if b_transposed else b
    pa, pb = cuda.pinned_empty(a.shape, a.dtype), cuda.pinned_empty(b_host.shape, b_host.dtype)
    pc_store = cuda.pinned_empty((m + 2, n + 6), np.float32)
    pa[...] = a
    pb[...] = b_host
    pc_store[...] = np.nan
    pc = pc_store[1:-1, 3:-3]
    gpu_ctx.gemm_host(pa, pb, pc, b_transposed=b_transposed)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b_host)
    dc = gpu_ctx.empty((m, n), np.float32)
    gpu_ctx.gemm(da, db, dc, b_transposed=b_transposed)
    gpu_ctx.synchronize()
    assert np.array_equal(np.ascontiguousarray(pc), dc.to_numpy())
    assert np.isnan(pc_store[0]).all() and np.isnan(pc_store[-1]).all()
    assert np.isnan(pc_store[:, :3]).all() and np.isnan(pc_store[:, -3:]).all()
    assert workloads.check_against_float64(np.ascontiguousarray(pc), a, b, rows=_sample_rows(m))["ok"]
    bias = np.linspace(-2, 2, n).astype(np.float32)
    ops = (("scale", 0.5), ("bias",), ("max", 0.0))
    gpu_ctx.gemm_host(pa, pb, pc, b_transposed=b_transposed, epilogue=ops, bias=bias)
    dbias = gpu_ctx.to_device(bias)
    gpu_ctx.gemm(da, db, dc, b_transposed=b_transposed, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    assert np.array_equal(np.ascontiguousarray(pc), dc.to_numpy())
    # Accumulation needs C on the device first: the row-panel schedule, same bits as one launch.
    c0 = np.random.default_rng(3).standard_normal((m, n)).astype(np.float32)
    pc[...] = c0
    gpu_ctx.gemm_host(pa, pb, pc, b_transposed=b_transposed, accumulate=True)
    dc.copy_from_host(c0)
    gpu_ctx.gemm(da, db, dc, b_transposed=b_transposed, accumulate=True)
    gpu_ctx.synchronize()
    assert np.array_equal(np.ascontiguousarray(pc), dc.to_numpy())
    for buf in (da, db, dc, dbias):
        buf.free()


def test_large_ragged_product_on_pageable_numpy_buffers(gpu_ctx) -> None:
    """Config 3 through the handle on ordinary (pageable) NumPy arrays: large enough for the
    host call to pipeline its copies in row panels. The result must equal the device-buffer
    path bit for bit and leave the arrays' surroundings alone."""
    a, b = workloads.make_inputs("ragged")
    c_store = np.full((4095 + 2, 3073 + 5), np.nan, np.float32)
    c = c_store[1:-1, 2:-3]
    compiled_for("bfloat16")(a, b, c)
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((4095, 3073), np.float32)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(np.ascontiguousarray(c), dc.to_numpy())
    assert np.isnan(c_store[0]).all() and np.isnan(c_store[-1]).all()
    assert np.isnan(c_store[:, :2]).all() and np.isnan(c_store[:, -3:]).all()
    rows = _sample_rows(4095)
    assert workloads.check_against_float64(np.ascontiguousarray(c), a, b, rows=rows)["ok"]


def test_device_buffers_through_the_handle(gpu_ctx) -> None:
    a, b = random_inputs(200, 264, 96, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((200, 264), np.float32)
    handle = compiled_for("float16")
    assert handle(da, db, dc) is None  # synchronous, like the simulator
    assert_close_to_oracle(dc.to_numpy(), a, b)
    with pytest.raises(hc.LaunchError, match="all numpy.ndarray or all DeviceBuffer"):
        handle(a, db, dc)
    with pytest.raises(hc.LaunchError, match="conflicting binding for N"):
        handle(da, db, gpu_ctx.empty((200, 265), np.float32))


def test_device_call_rejects_bad_arguments(gpu_ctx) -> None:
    a, b = random_inputs(128, 256, 64, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    with pytest.raises(hc.DeviceError, match="must not overlap"):
        gpu_ctx.gemm(da, db, cuda.DeviceBuffer.wrap(gpu_ctx, db.ptr, (128, 256), np.float32))
    dc = gpu_ctx.empty((128, 256), np.float32)
    with pytest.raises(hc.DeviceError, match="skinny variant needs m <= 64"):
        gpu_ctx.gemm(da, db, dc, variant=cuda.VARIANT_SKINNY)
    gpu_ctx.gemm(da, db, dc)  # the context is still usable
    gpu_ctx.synchronize()
    assert_close_to_oracle(dc.to_numpy(), a, b)


@pytest.mark.parametrize("shape", [(300, 520, 200), (100, 300, 96), (1024, 2048, 512)])
def test_push_targets_receive_every_tile(gpu_ctx, shape) -> None:
    """hcCudaGemmPush on one device: two extra buffers (here local ones; across GPUs they are
    peers' memory) must end up identical to C, windows and edges included."""
    m, n, k = shape
    a, b = random_inputs(m, n, k, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    frames = [gpu_ctx.empty((m + 1, n + 8), np.float32) for _ in range(3)]
    for frame in frames:
        frame.fill_bytes(0x7F)
    views = [frame.window(1, m + 1, 4, n + 4) for frame in frames]
    gpu_ctx.gemm(da, db, views[0], push=views[1:])
    gpu_ctx.synchronize()
    results = [frame.to_numpy() for frame in frames]
    assert_close_to_oracle(np.ascontiguousarray(results[0][1:, 4 : n + 4]), a, b)
    assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])
    sentinel = np.frombuffer(b"\x7f\x7f\x7f\x7f", np.uint32)[0]
    assert (results[0][0].view(np.uint32) == sentinel).all()
    assert (results[0][:, :4].view(np.uint32) == sentinel).all() and (results[0][:, n + 4 :].view(np.uint32) == sentinel).all()
    with pytest.raises(hc.DeviceError, match="overlaps c"):
        gpu_ctx.gemm(da, db, views[0], push=[views[0]])
    odd = gpu_ctx.empty((m, n + 1), np.float32)
    with pytest.raises(hc.DeviceError, match="multiple of 4"):
        gpu_ctx.gemm(da, db, odd.window(0, m, 0, n), push=[odd.window(0, m, 0, n)])


def test_a_wait_that_runs_out_is_reported_and_survivable(gpu_ctx) -> None:
    """The give-up path of the kernels' bounded waits, made to happen on purpose: a one-thread
    kernel waits about a millisecond on a barrier nobody signals, then reports it. Nothing
    faults; the context reports the timeout once and keeps working."""
    gpu_ctx.synchronize()
    gpu_ctx.selftest_device_timeout(2_000_000)
    with pytest.raises(hc.DeviceError, match="HC_CUDA_ERR_DEVICE_TIMEOUT") as info:
        gpu_ctx.synchronize()
    assert info.value.status == 5
    gpu_ctx.synchronize()  # the status was cleared
    a, b = random_inputs(8, 2048, 8192, "float16", scale=0.1)  # split-k: uses the counters that were reset
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b)
    a, b = random_inputs(300, 300, 300, "float16")
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((300, 300), np.float32)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert_close_to_oracle(dc.to_numpy(), a, b)


def test_pinned_arrays_round_trip(gpu_ctx) -> None:
    a_src, b_src = random_inputs(70, 80, 90, "float16")
    a = cuda.pinned_empty(a_src.shape, a_src.dtype)
    b = cuda.pinned_empty(b_src.shape, b_src.dtype)
    c = cuda.pinned_empty((70, 80), np.float32)
    a[...] = a_src
    b[...] = b_src
    compiled_for("float16")(a, b, c)
    assert_close_to_oracle(np.array(c), a_src, b_src)


# ---------------------------------------------------------------- properties at full size


def _sample_rows(m: int, count: int = 24) -> np.ndarray:
    rows = np.unique(np.concatenate([np.arange(0, m, max(1, m // count)), [m - 1]]))
    return rows.astype(np.int64)


@pytest.mark.parametrize("name", ["gemm_8192", "ragged", "skinny"])
def test_full_size_configs(name: str, gpu_ctx) -> None:
    """Configs 2-4 at full size: sampled rows against float64 and against the oracle, plus
    properties that need no reference: the result is reproducible, scaling A by 2 scales C by
    exactly 2 (a power of two commutes with every rounding), and a row permutation of A
    permutes the rows of C."""
    a, b = workloads.make_inputs(name)
    w = workloads.CONFIGS[name]
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((w.m, w.n), np.float32)
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    c = dc.to_numpy()
    assert np.isfinite(c).all()
    rows = _sample_rows(w.m)
    report = workloads.check_against_float64(c, a, b, rows=rows)
    assert report["ok"], report
    sample = np.ascontiguousarray(a[rows])
    expect = cpu_ref.matmul_k_ascending(sample, b)
    assert_close_to_oracle(np.ascontiguousarray(c[rows]), sample, b, expect=expect)

    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), c)

    doubled = gpu_ctx.to_device((a.astype(np.float32) * 2).astype(a.dtype))
    gpu_ctx.gemm(doubled, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), c * np.float32(2))
    doubled.free()

    if w.m >= 128:
        perm = np.random.default_rng(0).permutation(w.m)
        permuted = gpu_ctx.to_device(np.ascontiguousarray(a[perm]))
        gpu_ctx.gemm(permuted, db, dc)
        gpu_ctx.synchronize()
        assert np.array_equal(dc.to_numpy(), c[perm])
        permuted.free()
    for buf in (da, db, dc):
        buf.free()


def test_config5_slab_at_full_size(gpu_ctx, monkeypatch) -> None:
    """Config 5's per-rank problem at 8 GPUs, at full size on one GPU (16384 x 4096 x 16384, the last
    rank's column slab, on the 512x256 tiles): sampled rows against float64 and the oracle, run-to-run
    reproducibility, and the same bits from the 256x256 tiles."""
    w = workloads.CONFIGS["sharded"]
    lo, hi = w.n - w.n // 8, w.n
    a, b = workloads.make_sharded_inputs(lo, hi)
    assert gpu_ctx.plan(w.m, hi - lo, w.k, "float16").tiles_m == w.m // 512
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    dc = gpu_ctx.empty((w.m, hi - lo), np.float32)
    dc.fill_bytes(0xFF)
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    c = dc.to_numpy()
    assert np.isfinite(c).all()
    rows = _sample_rows(w.m)
    assert workloads.check_against_float64(c, a, b, rows=rows)["ok"]
    sample = np.ascontiguousarray(a[rows])
    assert_close_to_oracle(np.ascontiguousarray(c[rows]), sample, b, expect=cpu_ref.matmul_k_ascending(sample, b))
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), c)
    monkeypatch.setenv("HC_CUDA_DENSE_WIDE", "0")
    assert gpu_ctx.plan(w.m, hi - lo, w.k, "float16").tiles_m == w.m // 256
    gpu_ctx.gemm(da, db, dc)
    gpu_ctx.synchronize()
    assert np.array_equal(dc.to_numpy(), c)
    for buf in (da, db, dc):
        buf.free()


def test_config1_through_the_example_entry_point() -> None:
    a, b = workloads.make_inputs("sim_64")
    golden_a, golden_b, c_sim = load_golden("sim_f16_m64_n64_k64_normal_seed0")
    assert np.array_equal(a.view(np.uint16), golden_a.view(np.uint16))
    assert np.array_equal(b.view(np.uint16), golden_b.view(np.uint16))
    assert_close_to_oracle(gpu_wmma_matmul(a, b), a, b, expect=c_sim)


def test_sharded_config_scaled_down_on_one_gpu(gpu_ctx) -> None:
    """Config 5's structure on one device: two column slabs computed separately and
    assembled equal the unsharded product bit for bit (slabs are tile-aligned)."""
    from hc.distributed import ShardedMatmul, assemble_row_major

    m, k, n = 384, 640, 4096
    a, b = workloads.make_sharded_inputs(0, n, m=m, k=k)
    handle = compiled_for("float16")
    slabs = []
    for rank in range(2):
        sharded = ShardedMatmul(handle, gpu_ctx, n, 2, rank, align=256)
        da, db, dc = sharded.upload(a, b)
        sharded.run(da, db, dc)
        gpu_ctx.synchronize()
        slabs.append(dc.to_numpy())
    whole = gpu_wmma_matmul(a, b)
    assert np.array_equal(assemble_row_major(np.stack(slabs)), whole)
    assert_close_to_oracle(whole, a, b)
