"""The CPU oracle is pinned against outputs of the reference simulator itself."""

from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import GOLDEN, GOLDEN_NAMES, REFERENCE, REPO, load_golden, np_dtype
from oracle import cpu_ref


def test_fixtures_are_present() -> None:
    assert len(GOLDEN_NAMES) == 6
    assert (GOLDEN / "simbt_f16_m17_n19_k18_seed9.npz").exists()
    assert (GOLDEN / "simacc_f16_m17_n19_k18_seed11.npz").exists()
    assert (GOLDEN / "simfused_bf16_m33_n17_k40_seed12.npz").exists()
    assert (GOLDEN / "simfusednan_bf16_m33_n17_k40_seed14.npz").exists()
    assert (GOLDEN / "simnarrow_bf16_m33_n17_k40_seed13.npz").exists()
    assert (GOLDEN / "blocked_reference.npz").exists()


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_is_bit_identical_to_the_reference_simulator(name: str) -> None:
    a, b, c_sim = load_golden(name)
    for fn in (cpu_ref.matmul_k_ascending, cpu_ref.matmul_tiled, cpu_ref.matmul_numpy):
        out = fn(a, b)
        assert out.dtype == np.float32
        assert np.array_equal(out.view(np.uint32), c_sim.view(np.uint32)), fn.__name__


def test_transposed_b_kernel_fixture() -> None:
    """The Buffer[N, K] member of the kernel family, as the reference simulator executed it:
    the oracle on the un-transposed B reproduces its output bit for bit."""
    a, bt, c_sim = load_golden("simbt_f16_m17_n19_k18_seed9")
    assert bt.shape == (19, 18)
    out = cpu_ref.matmul_k_ascending(a, np.ascontiguousarray(bt.T))
    assert np.array_equal(out.view(np.uint32), c_sim.view(np.uint32))


def test_accumulating_and_fused_kernel_fixtures() -> None:
    """The C += A.B member and the member with element-wise statements after the k-loop, as the
    reference simulator executed them: the oracle's restatement is bit-identical."""
    a, b, c_sim = load_golden("simacc_f16_m17_n19_k18_seed11")
    with np.load(GOLDEN / "simacc_f16_m17_n19_k18_seed11.npz") as data:
        c0 = data["c0"]
    out = cpu_ref.matmul_fused(a, b, c0=c0)
    assert np.array_equal(out.view(np.uint32), c_sim.view(np.uint32))
    assert not np.array_equal(out, cpu_ref.matmul_k_ascending(a, b))  # C's old contents matter
    # Starting from C is not the same rounding as adding C at the end.
    late = cpu_ref.matmul_k_ascending(a, b) + c0
    assert np.abs(late - c_sim).max() < 1e-5

    a, b, c_sim = load_golden("simfused_bf16_m33_n17_k40_seed12")
    with np.load(GOLDEN / "simfused_bf16_m33_n17_k40_seed12.npz") as data:
        bias = data["bias"]
    ops = (("scale", 0.125), ("bias",), ("max", 0.0))
    out = cpu_ref.matmul_fused(a, b, epilogue=ops, bias=bias)
    assert np.array_equal(out.view(np.uint32), c_sim.view(np.uint32))
    assert (c_sim == 0).any() and (c_sim > 0).any()  # the maximum clips some elements, not all
    by_hand = np.maximum(cpu_ref.matmul_numpy(a, b) * np.float32(0.125) + bias[None, :], np.float32(0))
    assert np.array_equal(by_hand.view(np.uint32), c_sim.view(np.uint32))
    # Order matters: the statements are applied as written.
    swapped = cpu_ref.matmul_fused(a, b, epilogue=(("bias",), ("scale", 0.125), ("max", 0.0)), bias=bias)
    assert not np.array_equal(swapped, c_sim)
    for op, fn in ((("add", 1.5), lambda x: x + np.float32(1.5)), (("min", 0.25), lambda x: np.minimum(x, np.float32(0.25)))):
        assert np.array_equal(cpu_ref.matmul_fused(a, b, epilogue=(op,)), fn(cpu_ref.matmul_numpy(a, b)))


def test_fused_kernel_fixture_with_infinities_and_nan() -> None:
    """np.maximum keeps a NaN (inf * 0 or inf - inf inside the k-sum); -inf is clipped to 0, +inf
    stays. The reference simulator's output on such inputs is reproduced bit for bit, NaN
    positions included."""
    a, b, c_sim = load_golden("simfusednan_bf16_m33_n17_k40_seed14")
    with np.load(GOLDEN / "simfusednan_bf16_m33_n17_k40_seed14.npz") as data:
        bias = data["bias"]
    assert np.isnan(c_sim).any() and np.isposinf(c_sim).any() and not np.isneginf(c_sim).any()
    assert np.isnan(c_sim[7]).all() and np.isnan(c_sim[3, 2]) and np.isnan(c_sim[11]).all()
    assert (c_sim[20] == 0).any()  # -inf * positive b, clipped by the maximum
    out = cpu_ref.matmul_fused(a, b, epilogue=(("scale", 0.125), ("bias",), ("max", 0.0)), bias=bias)
    assert np.array_equal(np.isnan(out), np.isnan(c_sim))
    finite = ~np.isnan(c_sim)
    assert np.array_equal(out[finite].view(np.uint32), c_sim[finite].view(np.uint32))
    low = cpu_ref.matmul_fused(a, b, epilogue=(("min", 1.0),))
    assert np.array_equal(np.isnan(low), np.isnan(c_sim))


def test_narrow_kernel_fixture() -> None:
    """The member whose c is a bfloat16 buffer, as the reference simulator executed it: fp32
    accumulation, rounded to nearest even on the way out."""
    import ml_dtypes

    a, b, c_sim32 = load_golden("simnarrow_bf16_m33_n17_k40_seed13")
    with np.load(GOLDEN / "simnarrow_bf16_m33_n17_k40_seed13.npz") as data:
        c_bits = data["c_bits"]
    out = cpu_ref.matmul_fused(a, b, out_dtype=ml_dtypes.bfloat16)
    assert out.dtype == ml_dtypes.bfloat16 and np.array_equal(out.view(np.uint16), c_bits)
    assert np.array_equal(out.astype(np.float32), c_sim32)
    assert not np.array_equal(cpu_ref.matmul_k_ascending(a, b), c_sim32)  # the rounding is visible


def test_oracle_meets_the_reference_tests_own_tolerance() -> None:
    # tests/test_examples.py:22-33 of the reference: atol 2e-6 against its blocked product.
    with np.load(GOLDEN / "blocked_reference.npz") as blocked:
        for name in blocked.files:
            a, b, _ = load_golden(name)
            np.testing.assert_allclose(cpu_ref.matmul_k_ascending(a, b), blocked[name], rtol=0.0, atol=2e-6)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (16, 16, 16), (17, 19, 18), (3, 130, 77), (40, 5, 129), (8, 256, 96)])
def test_tiled_and_flat_restatements_agree(dtype: str, shape: tuple[int, int, int]) -> None:
    m, n, k = shape
    rng = np.random.default_rng(hash((dtype, shape)) % 2**32)
    a = rng.standard_normal((m, k)).astype(np_dtype(dtype))
    b = rng.standard_normal((k, n)).astype(np_dtype(dtype))
    flat = cpu_ref.matmul_k_ascending(a, b)
    assert np.array_equal(flat, cpu_ref.matmul_tiled(a, b))
    assert np.array_equal(flat, cpu_ref.matmul_numpy(a, b))
    assert np.array_equal(flat, cpu_ref.matmul_k_ascending(a, b, threads=1))


def test_empty_and_zero_k() -> None:
    f16 = np.float16
    assert cpu_ref.matmul_k_ascending(np.zeros((0, 4), f16), np.zeros((4, 5), f16)).shape == (0, 5)
    assert cpu_ref.matmul_k_ascending(np.zeros((3, 4), f16), np.zeros((4, 0), f16)).shape == (3, 0)
    out = cpu_ref.matmul_k_ascending(np.zeros((3, 0), f16), np.zeros((0, 5), f16))
    assert out.shape == (3, 5) and not out.any()
    assert np.array_equal(out, cpu_ref.matmul_tiled(np.zeros((3, 0), f16), np.zeros((0, 5), f16)))


def test_row_sample_matches_full_product() -> None:
    rng = np.random.default_rng(11)
    a = rng.standard_normal((50, 64)).astype(np.float16)
    b = rng.standard_normal((64, 33)).astype(np.float16)
    full = cpu_ref.matmul_k_ascending(a, b)
    part = cpu_ref.matmul_k_ascending(a, b, rows=(10, 25))
    assert np.array_equal(part[10:25], full[10:25])
    assert not part[:10].any() and not part[25:].any()


def test_every_16_bit_pattern_widens_exactly() -> None:
    one = np.ones((1, 1), np.float16)
    for dtype in ("float16", "bfloat16"):
        values = np.arange(65536, dtype=np.uint16).view(np_dtype(dtype)).reshape(1, -1)
        with np.errstate(all="ignore"):
            out = cpu_ref.matmul_k_ascending(one.astype(np_dtype(dtype)), values)
        ref = values.astype(np.float32)
        finite = ~np.isnan(ref)
        assert np.array_equal(out[finite], ref[finite] + np.float32(0))
        assert np.array_equal(np.isnan(out), np.isnan(ref))


def test_rejects_mismatched_inputs() -> None:
    with pytest.raises(ValueError):
        cpu_ref.matmul_k_ascending(np.zeros((2, 3), np.float16), np.zeros((4, 2), np.float16))
    with pytest.raises(ValueError):
        cpu_ref.matmul_k_ascending(np.zeros((2, 3), np.float32), np.zeros((3, 2), np.float32))


@pytest.mark.skipif(not REFERENCE.exists(), reason="the reference checkout is not on this machine")
def test_reference_simulator_reproduces_a_fixture_and_runs_our_example() -> None:
    """Re-runs the unmodified reference simulator (with the two stand-in dependencies) on the
    ragged fixture, and runs this repository's example kernel through it as well: both must
    reproduce the stored output bit for bit."""
    script = r"""
import importlib.util, sys
import numpy as np
import hc.simulator as sim
from examples.amdgpu_gfx11_wmma_matmul import simulate_gfx11_wmma_matmul
data = np.load(sys.argv[1])
a = data["a_bits"].view(np.float16); b = data["b_bits"].view(np.float16)
assert np.array_equal(simulate_gfx11_wmma_matmul(a, b), data["c"])
spec = importlib.util.spec_from_file_location("b200_example", sys.argv[2])
mod = importlib.util.module_from_spec(spec); mod.__package__ = "loaded_by_test"
sys.modules["b200_example"] = mod; spec.loader.exec_module(mod)
c = np.zeros_like(data["c"])
sim.launch(mod.tiled_wmma_matmul_for("float16"), a, b, c)
assert np.array_equal(c, data["c"])
print("ok")
"""
    env = dict(os.environ)
    env["HC_IXSIMPL_VENDOR_DIR"] = str(REPO / "oracle" / "standins" / "ixsimpl_vendor")
    env["PYTHONPATH"] = os.pathsep.join([str(REFERENCE), str(REPO / "oracle" / "standins")])
    result = subprocess.run(
        [sys.executable, "-c", script, str(GOLDEN / "sim_f16_m17_n19_k18_seed7.npz"),
         str(REPO / "5_b200" / "examples" / "b200_wmma_matmul.py")],
        env=env, capture_output=True, text=True, timeout=120, cwd=str(REPO / "tests"))
    assert result.returncode == 0, result.stderr
    assert result.stdout.strip() == "ok"


def test_elementwise_map_fixture() -> None:
    """The masked element-wise kernels as the reference simulator executed them: the oracle's
    statement-by-statement float32 restatement gives the same bits (NaN where it gave NaN), and
    nothing was written past the operations the recogniser lists for these kernels."""
    with np.load(GOLDEN / "simmap_f32_seed15.npz") as data:
        fixture = {key: data[key] for key in data.files}
    assert np.array_equal(fixture["add_two_y"], fixture["add_two_x"] + 2)  # the reference test's own assertion
    assert np.array_equal(cpu_ref.map_elementwise(fixture["add_two_x"], (("add", 2.0),)), fixture["add_two_y"])
    ops = (("scale", 0.5), ("add", -1.0), ("rsub_other",), ("max", 0.25), ("scale", -1.0), ("scale", 3.0),
           ("add_other",))
    out = cpu_ref.map_elementwise(fixture["x"], ops, other=fixture["y"])
    want = fixture["out"]
    assert np.isnan(want).sum() >= 3 and np.isinf(want).any() and not (want == -7.0).any()
    assert np.array_equal(np.isnan(out), np.isnan(want))
    keep = ~np.isnan(want)
    assert np.array_equal(out[keep].view(np.uint32), want[keep].view(np.uint32))
    # The two-dimensional kernel (8 x 32 tiles over 37 x 70): element-wise, so the same restatement on the
    # flattened matrices; np.maximum(0.0, v) returns v when neither is greater, so -0.0 survives.
    ops2 = (("scale", 2.0), ("add_other",), ("rmax", 0.0))
    out2 = cpu_ref.map_elementwise(fixture["x_2d"].reshape(-1), ops2, other=fixture["shift_2d"].reshape(-1))
    want2 = fixture["out_2d"].reshape(-1)
    assert np.signbit(want2[1]) and want2[1] == 0 and not np.signbit(want2[0]) and not (want2 == -7.0).any()
    keep2 = ~np.isnan(want2)
    assert np.array_equal(np.isnan(out2), ~keep2)
    assert np.array_equal(out2[keep2].view(np.uint32), want2[keep2].view(np.uint32))
    # The one-element-per-work-item form (11 elements, groups of 4): every element written, once.
    assert np.array_equal(cpu_ref.map_elementwise(fixture["workitem_x"], (("add", 2.0),)), fixture["workitem_y"])


def test_float8_kernel_fixtures() -> None:
    """The float8 members as the reference simulator executed them (e4m3fn with B stored [K, N],
    e5m2 with B stored [N, K]): every form of the oracle reproduces the outputs bit for bit, and the
    8-bit decoders agree with ml_dtypes on all 256 patterns of each format."""
    import ctypes

    import ml_dtypes

    a, b, c_sim = load_golden("simf8_e4m3fn_m33_n17_k40_seed16")
    assert a.dtype == ml_dtypes.float8_e4m3fn and a.shape == (33, 40) and not (c_sim == -7.0).any()
    for fn in (cpu_ref.matmul_k_ascending, cpu_ref.matmul_tiled, cpu_ref.matmul_numpy):
        assert np.array_equal(fn(a, b).view(np.uint32), c_sim.view(np.uint32)), fn.__name__
    a, bt, c_sim = load_golden("simf8_e5m2_bt_m17_n19_k18_seed17")
    assert a.dtype == ml_dtypes.float8_e5m2 and bt.shape == (19, 18)
    b = np.ascontiguousarray(bt.T)
    for fn in (cpu_ref.matmul_k_ascending, cpu_ref.matmul_tiled, cpu_ref.matmul_numpy):
        assert np.array_equal(fn(a, b).view(np.uint32), c_sim.view(np.uint32)), fn.__name__
    lib = cpu_ref.load()
    lib.hc_oracle_widen.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                    ctypes.c_int]
    for dtype in (ml_dtypes.float8_e4m3fn, ml_dtypes.float8_e5m2):
        every = np.arange(256, dtype=np.uint8).view(dtype).reshape(16, 16)
        out = np.zeros((16, 16), np.float32)
        lib.hc_oracle_widen(every.ctypes.data, 16, out.ctypes.data, 16, 16, cpu_ref.dtype_code(dtype))
        want = every.astype(np.float32)
        assert np.array_equal(np.isnan(out), np.isnan(want))
        assert np.array_equal(out[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
