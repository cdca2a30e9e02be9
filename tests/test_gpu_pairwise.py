"""The pairwise-distance kernel class on a B200: bit-identical to the reference simulator's stored
outputs and to the NumPy oracle, through the `hc.compile(..., target="nvidia-sm100a")` handle and
through `hc.cuda` (the C ABI)."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import GOLDEN
from examples import b200_pairwise as examples
from hc import cuda
from hc.errors import DeviceError
from oracle import cpu_ref

pytestmark = pytest.mark.gpu


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    """Equal bit for bit; a NaN must be a NaN (its sign and payload are not part of the value: x86
    and the GPU choose different ones)."""
    if got.shape != want.shape:
        return False
    nan = np.isnan(want)
    return bool(np.array_equal(np.isnan(got), nan) and np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]))


def test_handle_matches_the_reference_simulator_bit_for_bit() -> None:
    with np.load(GOLDEN / "simpair_f32_seed18.npz") as data:
        cases = [("pairwise", data["test_x1"], data["test_x2"], data["test_out"]),
                 ("pairwise", data["x1"], data["x2"], data["out"]),
                 ("pairwise_squared", data["sq_x1"], data["sq_x2"], data["sq_out"])]
    for name, x1, x2, want in cases:
        out = np.full(want.shape, np.float32(-7.0))
        assert examples.compiled(name)(x1, x2, out) is None
        assert same_bits(out, want), name


@pytest.mark.parametrize("h", [1, 5, 7, 8, 9, 31, 32, 33, 127, 128, 129, 150, 256, 257, 300, 1031, 4100])
def test_every_summation_shape_matches_numpy(h: int, gpu_ctx) -> None:
    """The order of NumPy's float32 sum changes with the number of values (fewer than 8, up to 128,
    recursive halves): each regime, with edges on both output axes, against the oracle."""
    rng = np.random.default_rng([h, 21])
    w1, w2 = 67, 131
    x1 = (rng.standard_normal((w1, h)) * rng.choice([1e-3, 1.0, 50.0], size=(w1, h))).astype(np.float32)
    x2 = (rng.standard_normal((w2, h)) * rng.choice([1e-3, 1.0, 50.0], size=(w2, h))).astype(np.float32)
    for take_sqrt in (True, False):
        want = cpu_ref.pairwise_distance(x1, x2, take_sqrt=take_sqrt)
        d1, d2 = gpu_ctx.to_device(x1), gpu_ctx.to_device(x2)
        dout = gpu_ctx.empty((w1, w2), np.float32)
        dout.fill_bytes(0xFF)
        gpu_ctx.pairwise(d1, d2, dout, take_sqrt=take_sqrt)
        gpu_ctx.synchronize()
        assert same_bits(dout.to_numpy(), want), (h, take_sqrt)
        for buf in (d1, d2, dout):
            buf.free()


def test_padded_pitches_unaligned_bases_and_guard_bands(gpu_ctx) -> None:
    rng = np.random.default_rng(22)
    w1, w2, h = 45, 70, 77
    x1 = rng.standard_normal((w1, h)).astype(np.float32)
    x2 = rng.standard_normal((w2, h)).astype(np.float32)
    want = cpu_ref.pairwise_distance(x1, x2)
    for pads in ((0, 0, 0), (1, 3, 1), (3, 0, 7), (4, 8, 12)):
        d1 = cuda.DeviceBuffer(gpu_ctx, (w1, h), np.float32, ld=h + pads[0])
        d2 = cuda.DeviceBuffer(gpu_ctx, (w2, h), np.float32, ld=h + pads[1])
        # `out` is a window inside a larger matrix: nothing around it may change.
        frame = cuda.DeviceBuffer(gpu_ctx, (w1 + 4, w2 + pads[2] + 6), np.float32)
        frame.fill_bytes(0x7F)
        before = frame.to_numpy()
        window = cuda.DeviceBuffer.wrap(gpu_ctx, frame.ptr + (2 * frame.ld + 3) * 4, (w1, w2), np.float32, ld=frame.ld)
        d1.copy_from_host(x1)
        d2.copy_from_host(x2)
        gpu_ctx.pairwise(d1, d2, window)
        gpu_ctx.synchronize()
        after = frame.to_numpy()
        assert same_bits(np.ascontiguousarray(after[2 : 2 + w1, 3 : 3 + w2]), want), pads
        after[2 : 2 + w1, 3 : 3 + w2] = before[2 : 2 + w1, 3 : 3 + w2]
        assert np.array_equal(after.view(np.uint32), before.view(np.uint32)), pads
        for buf in (d1, d2, frame):
            buf.free()


def test_host_arrays_views_and_empty_reductions() -> None:
    rng = np.random.default_rng(23)
    big1 = rng.standard_normal((50, 300)).astype(np.float32)
    big2 = rng.standard_normal((90, 300)).astype(np.float32)
    x1, x2 = big1[3:40, 10:210], big2[::2, 10:210]  # padded rows; every other row (not row-major: staged)
    out_frame = np.full((40, 60), np.float32(-3.0))
    out = out_frame[1:38, 5:50]
    want = cpu_ref.pairwise_distance(x1, x2)
    assert examples.compiled("pairwise")(x1, x2, out) is None
    assert same_bits(np.ascontiguousarray(out), want)
    out_frame[1:38, 5:50] = -3.0
    assert (out_frame == -3.0).all()
    # No values to reduce: every result is inactive in the simulator, so nothing is stored.
    untouched = np.full((4, 6), np.float32(5.0))
    assert examples.compiled("pairwise")(np.zeros((4, 0), np.float32), np.zeros((6, 0), np.float32), untouched) is None
    assert (untouched == 5.0).all()


def test_a_larger_problem_against_sampled_rows(gpu_ctx) -> None:
    rng = np.random.default_rng(24)
    w1, w2, h = 2050, 1537, 260
    x1 = rng.standard_normal((w1, h)).astype(np.float32)
    x2 = rng.standard_normal((w2, h)).astype(np.float32)
    x1[17, 100], x2[1500, 3] = np.inf, np.nan
    d1, d2 = gpu_ctx.to_device(x1), gpu_ctx.to_device(x2)
    dout = gpu_ctx.empty((w1, w2), np.float32)
    dout.fill_bytes(0xFF)
    gpu_ctx.pairwise(d1, d2, dout)
    gpu_ctx.synchronize()
    got = dout.to_numpy()
    rows = np.unique(np.concatenate([np.arange(0, 40), [17, 1023, 1024, 1025], np.arange(w1 - 40, w1)]))
    with np.errstate(invalid="ignore"):
        want = cpu_ref.pairwise_distance(x1[rows], x2)
    assert same_bits(np.ascontiguousarray(got[rows]), want)
    assert np.isnan(got[:, 1500]).all() and np.isinf(got[17, :1500]).all()
    for buf in (d1, d2, dout):
        buf.free()


def test_bad_arguments_are_rejected(gpu_ctx) -> None:
    d1, d2 = gpu_ctx.empty((4, 8), np.float32), gpu_ctx.empty((6, 8), np.float32)
    dout = gpu_ctx.empty((4, 6), np.float32)
    with pytest.raises(ValueError, match="do not fit"):
        gpu_ctx.pairwise(d1, d2, gpu_ctx.empty((6, 4), np.float32))
    with pytest.raises(DeviceError, match="must not overlap"):
        gpu_ctx.pairwise(d1, d2, cuda.DeviceBuffer.wrap(gpu_ctx, d1.ptr, (4, 6), np.float32, ld=8))
    gpu_ctx.pairwise(d1, d2, dout)  # still usable
    gpu_ctx.synchronize()
