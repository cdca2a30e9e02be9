"""The row-sum kernel class on a B200: bit-identical to the reference simulator's stored outputs
and to the NumPy oracle, through the `hc.compile(..., target="nvidia-sm100a")` handle and through
`hc.cuda` (the C ABI)."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import GOLDEN
from examples import b200_rowsum as examples
from hc import cuda
from hc.errors import DeviceError
from oracle import cpu_ref

pytestmark = pytest.mark.gpu


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    """Equal bit for bit; a NaN must be a NaN (its sign and payload are not part of the value)."""
    if got.shape != want.shape:
        return False
    nan = np.isnan(want)
    return bool(np.array_equal(np.isnan(got), nan) and np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]))


def test_handle_matches_the_reference_simulator_bit_for_bit() -> None:
    with np.load(GOLDEN / "simrow_f32_seed19.npz") as data:
        cases = [("row_sums", data["x"], data["sums"]), ("row_sums", data["few_x"], data["few_sums"]),
                 ("row_norms", data["norm_x"], data["norms"]), ("row_energy", data["energy_x"], data["energy"])]
    for name, x, want in cases:
        out = np.full(want.shape, np.float32(-7.0))
        assert examples.compiled(name)(x, out) is None
        assert same_bits(out, want), name
    # (The row of -0.0 values sums to +0.0, as in the simulator.)
    assert not np.signbit(cases[1][2][4])


@pytest.mark.parametrize("h", [1, 5, 7, 8, 9, 15, 16, 31, 33, 127, 128, 129, 150, 256, 257, 300, 1031, 4100, 70000])
def test_every_summation_shape_matches_numpy(h: int, gpu_ctx) -> None:
    """The order of NumPy's float32 sum changes with the number of values (fewer than 8, up to 128,
    recursive halves, which the kernel cuts into 2 to 16 ranges per row): each regime, with a row
    count no CTA size divides, against the oracle."""
    rng = np.random.default_rng([h, 31])
    w = 301 if h < 10000 else 37
    x = (rng.standard_normal((w, h)) * rng.choice([1e-3, 1.0, 50.0], size=(w, h))).astype(np.float32)
    x[5, :] = -0.0
    dx = gpu_ctx.to_device(x)
    for square, take_sqrt in ((False, False), (True, False), (True, True)):
        want = cpu_ref.row_sums(x, square=square, take_sqrt=take_sqrt)
        dout = gpu_ctx.empty((w,), np.float32)
        dout.fill_bytes(0xFF)
        gpu_ctx.row_sum(dx, dout, square=square, take_sqrt=take_sqrt)
        gpu_ctx.synchronize()
        assert same_bits(dout.to_numpy(), want), (h, square, take_sqrt)
        dout.free()
    dx.free()


def test_restated_order_on_the_gpu_for_small_rows(gpu_ctx) -> None:
    """Against the oracle's written-out summation order (not NumPy's own sum) on a few shapes."""
    rng = np.random.default_rng(32)
    for h in (3, 100, 129, 700):
        x = (rng.standard_normal((9, h)) * 1e3).astype(np.float32)
        dx, dout = gpu_ctx.to_device(x), gpu_ctx.empty((9,), np.float32)
        gpu_ctx.row_sum(dx, dout)
        gpu_ctx.synchronize()
        assert same_bits(dout.to_numpy(), cpu_ref.row_sums(x, restated=True)), h
        dx.free()
        dout.free()


def test_padded_pitches_unaligned_bases_and_guard_bands(gpu_ctx) -> None:
    rng = np.random.default_rng(33)
    w, h = 200, 333
    x = rng.standard_normal((w, h)).astype(np.float32)
    want = cpu_ref.row_sums(x)
    for pad, shift in ((0, 0), (1, 1), (3, 2), (7, 3), (3, 0)):
        frame_x = cuda.DeviceBuffer(gpu_ctx, (w + 1, h + pad + 4), np.float32)
        frame_x.fill_bytes(0x7F)  # (large finite values around the matrix: a stray read would show)
        dx = cuda.DeviceBuffer.wrap(gpu_ctx, frame_x.ptr + shift * 4, (w, h), np.float32, ld=frame_x.ld)
        dx.copy_from_host(x)
        # `out` is a window inside a longer vector: nothing around it may change.
        frame = cuda.DeviceBuffer(gpu_ctx, (w + 16,), np.float32)
        frame.fill_bytes(0x7F)
        before = frame.to_numpy()
        window = cuda.DeviceBuffer.wrap(gpu_ctx, frame.ptr + (5 + shift) * 4, (w,), np.float32)
        gpu_ctx.row_sum(dx, window)
        gpu_ctx.synchronize()
        after = frame.to_numpy()
        assert same_bits(np.ascontiguousarray(after[5 + shift : 5 + shift + w]), want), (pad, shift)
        after[5 + shift : 5 + shift + w] = before[5 + shift : 5 + shift + w]
        assert np.array_equal(after.view(np.uint32), before.view(np.uint32)), (pad, shift)
        frame_x.free()
        frame.free()


def test_host_arrays_views_and_empty_reductions() -> None:
    rng = np.random.default_rng(34)
    big = rng.standard_normal((90, 300)).astype(np.float32)
    out_frame = np.full((120,), np.float32(-3.0))
    # Padded rows, written into a window of a longer vector.
    x, out = big[3:80, 10:210], out_frame[7:84]
    assert examples.compiled("row_sums")(x, out) is None
    assert same_bits(np.ascontiguousarray(out), cpu_ref.row_sums(x))
    out_frame[7:84] = -3.0
    assert (out_frame == -3.0).all()
    # Every other row and every other output (neither is contiguous: staged).
    x, out = big[::2, 5:205], out_frame[10:100:2]
    assert examples.compiled("row_norms")(x, out) is None
    assert same_bits(np.ascontiguousarray(out), cpu_ref.row_sums(x, square=True, take_sqrt=True))
    assert (out_frame[11:100:2] == -3.0).all()
    # No values to reduce: every result is inactive in the simulator, so nothing is stored.
    untouched = np.full((4,), np.float32(5.0))
    assert examples.compiled("row_sums")(np.zeros((4, 0), np.float32), untouched) is None
    assert (untouched == 5.0).all()
    # No rows: nothing to do.
    assert examples.compiled("row_sums")(np.zeros((0, 8), np.float32), np.zeros((0,), np.float32)) is None


def test_a_larger_problem_on_device_buffers_through_the_handle(gpu_ctx) -> None:
    rng = np.random.default_rng(35)
    w, h = 40001, 520
    x = rng.standard_normal((w, h)).astype(np.float32)
    x[17, 100], x[30000, 3] = np.inf, np.nan
    dx, dout = gpu_ctx.to_device(x), gpu_ctx.empty((w,), np.float32)
    dout.fill_bytes(0xFF)
    assert examples.compiled("row_energy")(dx, dout) is None  # (synchronises)
    got = dout.to_numpy()
    with np.errstate(invalid="ignore"):
        want = cpu_ref.row_sums(x, square=True)
    assert same_bits(got, want) and np.isinf(got[17]) and np.isnan(got[30000])
    dx.free()
    dout.free()


def test_many_rows_of_several_leaves(gpu_ctx) -> None:
    """More rows than the GPU holds at once, each of four leaves of NumPy's recursion (four pairs of
    lanes per row), and the row count not a multiple of the rows of a CTA."""
    rng = np.random.default_rng(36)
    w, h = 330001, 300
    x = rng.standard_normal((w, h)).astype(np.float32)
    dx, dout = gpu_ctx.to_device(x), gpu_ctx.empty((w,), np.float32)
    dout.fill_bytes(0xFF)
    gpu_ctx.row_sum(dx, dout)
    gpu_ctx.synchronize()
    assert same_bits(dout.to_numpy(), cpu_ref.row_sums(x))
    dx.free()
    dout.free()


def test_random_shapes_pitches_and_forms_match_numpy(gpu_ctx) -> None:
    """Eighty random problems (rows from 1 to 20000, values from 1 to 30000, padded and odd pitches,
    rows of -0.0, all three forms), each against NumPy's own sum row by row."""
    rng = np.random.default_rng(37)
    for case in range(80):
        kind = case % 4
        if kind == 0:
            w, h = int(rng.integers(1, 3000)), int(rng.integers(1, 300))
        elif kind == 1:
            w, h = int(rng.integers(1, 100)), int(rng.integers(1, 30000))
        elif kind == 2:
            w, h = int(rng.integers(1, 20000)), int(rng.integers(1, 140))
        else:
            w, h = int(rng.integers(1, 1000)), 8 * int(rng.integers(1, 400))
        pad = int(rng.choice([0, 0, 1, 3, 4, 8]))
        x = (rng.standard_normal((w, h)) * rng.choice([1e-3, 1.0, 1e3], size=(w, h))).astype(np.float32)
        if case % 3 == 0:
            x[int(rng.integers(0, w)), :] = -0.0
        dx = cuda.DeviceBuffer(gpu_ctx, (w, h), np.float32, ld=h + pad)
        dx.copy_from_host(x)
        dout = gpu_ctx.empty((w,), np.float32)
        square, take_sqrt = bool(case & 1), bool(case & 1) and bool(case & 2)
        gpu_ctx.row_sum(dx, dout, square=square, take_sqrt=take_sqrt)
        gpu_ctx.synchronize()
        values = x * x if square else x
        want = np.array([np.sum(row) for row in values], np.float32)
        if take_sqrt:
            want = np.sqrt(want)
        assert same_bits(dout.to_numpy(), want), (w, h, pad, square, take_sqrt)
        dx.free()
        dout.free()


def test_bad_arguments_are_rejected(gpu_ctx) -> None:
    dx, dout = gpu_ctx.empty((4, 8), np.float32), gpu_ctx.empty((4,), np.float32)
    with pytest.raises(ValueError, match="do not fit"):
        gpu_ctx.row_sum(dx, gpu_ctx.empty((5,), np.float32))
    with pytest.raises(DeviceError, match="must not overlap"):
        gpu_ctx.row_sum(dx, cuda.DeviceBuffer.wrap(gpu_ctx, dx.ptr + 16, (4,), np.float32))
    gpu_ctx.row_sum(dx, dout)  # still usable
    gpu_ctx.synchronize()
