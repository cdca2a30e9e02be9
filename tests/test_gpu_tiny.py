"""The tiny variant on a B200: products and sums rounded one by one with k ascending on the float32
pipes, so the output is bit-identical to the reference simulator's stored outputs and to the oracle
(the tensor-core kernels agree with them to rounding). AUTO takes it for one 64x64 tile with a short
k -- benchmark configuration 1 and every matmul fixture -- and it can be forced for any shape."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import GOLDEN, GOLDEN_NAMES, load_golden, np_dtype
from examples.b200_wmma_matmul import compiled_for
from hc import cuda
from oracle import cpu_ref

pytestmark = pytest.mark.gpu


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    if got.shape != want.shape or got.dtype != want.dtype:
        return False
    bits = np.uint32 if got.dtype == np.float32 else np.uint16
    nan = np.isnan(want.astype(np.float32))
    return bool(np.array_equal(np.isnan(got.astype(np.float32)), nan)
                and np.array_equal(got.view(bits)[~nan], want.view(bits)[~nan]))


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_matmul_fixtures_are_reproduced_bit_for_bit(name: str, gpu_ctx) -> None:
    a, b, c_sim = load_golden(name)
    m, k = a.shape
    n = b.shape[1]
    assert gpu_ctx.plan(m, n, k, a.dtype.name).variant == "tiny"  # what AUTO does with these shapes
    c = np.full(c_sim.shape, np.nan, np.float32)
    assert compiled_for(a.dtype.name)(a, b, c) is None
    assert same_bits(c, c_sim)
    # The tensor-core kernels on the same inputs: the same numbers to rounding.
    da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
    for variant in (cuda.VARIANT_SKINNY, cuda.VARIANT_DENSE):
        dc = gpu_ctx.empty((m, n), np.float32)
        gpu_ctx.gemm(da, db, dc, variant=variant)
        gpu_ctx.synchronize()
        np.testing.assert_allclose(dc.to_numpy(), c_sim, rtol=0, atol=1e-5 * max(1.0, float(np.abs(c_sim).max())))
        dc.free()
    da.free(), db.free()


def test_every_member_of_the_family_is_bit_identical_to_the_simulator() -> None:
    a, b, c_sim = load_golden("simbt_f16_m17_n19_k18_seed9")  # b stored [N, K]
    c = np.zeros(c_sim.shape, np.float32)
    compiled_for("float16", None, True)(a, b, c)
    assert same_bits(c, c_sim)

    a, b, c_sim = load_golden("simacc_f16_m17_n19_k18_seed11")
    with np.load(GOLDEN / "simacc_f16_m17_n19_k18_seed11.npz") as data:
        c = data["c0"].copy()
    compiled_for("float16", None, False, "accumulate")(a, b, c)
    assert same_bits(c, c_sim)

    for name in ("simfused_bf16_m33_n17_k40_seed12", "simfusednan_bf16_m33_n17_k40_seed14"):
        a, b, c_sim = load_golden(name)
        with np.load(GOLDEN / f"{name}.npz") as data:
            bias = data["bias"]
        c = np.full(c_sim.shape, np.float32(-7.0))
        compiled_for("bfloat16", None, False, "fused")(a, b, c, bias)
        assert same_bits(c, c_sim), name

    with np.load(GOLDEN / "simnarrow_bf16_m33_n17_k40_seed13.npz") as data:
        a = data["a_bits"].view(np_dtype("bfloat16"))
        b = data["b_bits"].view(np_dtype("bfloat16"))
        c_sim = data["c_bits"].view(np_dtype("bfloat16"))
    c = np.zeros(c_sim.shape, np_dtype("bfloat16"))
    compiled_for("bfloat16", None, False, "narrow")(a, b, c)
    assert same_bits(c, c_sim)


@pytest.mark.parametrize("shape", [(1, 1, 1), (64, 64, 128), (63, 65, 129), (130, 300, 70), (200, 100, 500),
                                   (17, 700, 33), (257, 129, 64)])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_forced_on_any_shape_it_equals_the_oracle(shape, dtype: str, gpu_ctx) -> None:
    m, n, k = shape
    rng = np.random.default_rng([m, n, k, 31])
    a = (rng.standard_normal((m, k)) * rng.choice([1e-3, 1.0, 30.0], size=(m, k))).astype(np_dtype(dtype))
    b = (rng.standard_normal((k, n)) * rng.choice([1e-3, 1.0, 30.0], size=(k, n))).astype(np_dtype(dtype))
    want = cpu_ref.matmul_k_ascending(a, b)
    for pads in ((0, 0, 0), (1, 3, 5)):
        da = cuda.DeviceBuffer(gpu_ctx, (m, k), a.dtype, ld=k + pads[0])
        db = cuda.DeviceBuffer(gpu_ctx, (k, n), b.dtype, ld=n + pads[1])
        dc = cuda.DeviceBuffer(gpu_ctx, (m, n), np.float32, ld=n + pads[2])
        da.copy_from_host(a), db.copy_from_host(b)
        dc.fill_bytes(0xFF)
        gpu_ctx.gemm(da, db, dc, variant=cuda.VARIANT_TINY)
        gpu_ctx.synchronize()
        assert same_bits(dc.to_numpy(), want), (shape, pads)
        plan = gpu_ctx.plan(m, n, k, dtype, variant=cuda.VARIANT_TINY, lda=k + pads[0], ldb=n + pads[1], ldc=n + pads[2])
        assert (plan.variant, plan.kernel_launches, plan.repack_a, plan.scratch_bytes) == ("tiny", 1, False, 0)
        for buf in (da, db, dc):
            buf.free()
    # The fused and accumulating members, B stored [N, K], against the oracle's restatement.
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    ops = (("scale", 0.5), ("bias",), ("max", -0.25), ("min", 3.0))
    da, dbt = gpu_ctx.to_device(a), gpu_ctx.to_device(np.ascontiguousarray(b.T))
    dc, dbias = gpu_ctx.to_device(c0), gpu_ctx.to_device(bias)
    gpu_ctx.gemm(da, dbt, dc, variant=cuda.VARIANT_TINY, b_transposed=True, accumulate=True, epilogue=ops, bias=dbias)
    gpu_ctx.synchronize()
    want = cpu_ref.matmul_fused(a, b, c0=c0, epilogue=ops, bias=bias)
    assert same_bits(dc.to_numpy(), want.astype(np.float32))
    for buf in (da, dbt, dc, dbias):
        buf.free()


def test_push_targets_and_float8_stay_with_the_tensor_core_kernels(gpu_ctx) -> None:
    assert gpu_ctx.plan(64, 64, 64, "float8_e4m3fn", b_transposed=True).variant == "skinny"
    with pytest.raises(cuda.DeviceError, match="16-bit operands"):
        gpu_ctx.plan(64, 64, 64, "float8_e4m3fn", b_transposed=True, variant=cuda.VARIANT_TINY)
    assert gpu_ctx.plan(64, 65, 64, "float16").variant == "skinny"   # two tiles
    assert gpu_ctx.plan(64, 64, 129, "float16").variant == "skinny"  # a longer k
