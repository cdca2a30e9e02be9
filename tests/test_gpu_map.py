"""GPU parity of the masked element-wise kernel class: bit-identical to the reference simulator's
stored outputs and to the NumPy oracle, through the compiled handle (host arrays and device
buffers) and through the C ABI."""

import numpy as np
import pytest

from hc import cuda

from conftest import GOLDEN
from examples.b200_elementwise import compiled, scaled_clamp_numpy
from oracle import cpu_ref

pytestmark = pytest.mark.gpu

OPS = (("scale", 0.5), ("add", -1.0), ("rsub_other",), ("max", 0.25), ("scale", -1.0), ("scale", 3.0), ("add_other",))


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    """Equal float32 bit patterns; NaN only has to be NaN in the same places."""
    nan = np.isnan(want)
    return bool(np.array_equal(np.isnan(got), nan) and np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)))


def test_simulator_fixture_through_the_handles() -> None:
    with np.load(GOLDEN / "simmap_f32_seed15.npz") as data:
        fixture = {key: data[key] for key in data.files}
    y = np.zeros(6, np.float32)
    compiled("add_two")(fixture["add_two_x"], y)
    assert np.array_equal(y, fixture["add_two_y"])
    out = np.full(1003, np.float32(-7.0))
    compiled("scaled_clamp")(fixture["x"], fixture["y"], out)
    assert same_bits(out, fixture["out"])
    # A strided output array is staged; an in-place call reads the array it writes.
    wide = np.full(2006, np.float32(-7.0))
    compiled("scaled_clamp")(fixture["x"], fixture["y"], wide[::2])
    assert same_bits(wide[::2], fixture["out"]) and (wide[1::2] == -7.0).all()
    x = fixture["add_two_x"].copy()
    compiled("add_two")(x, x)
    assert np.array_equal(x, fixture["add_two_y"])
    # The one-element-per-work-item form of the same kernel.
    y = np.full(11, np.float32(-7.0))
    compiled("add_two_per_workitem")(fixture["workitem_x"], y)
    assert same_bits(y, fixture["workitem_y"])


def test_two_dimensional_kernel_matches_the_simulator(gpu_ctx) -> None:
    with np.load(GOLDEN / "simmap_f32_seed15.npz") as data:
        x, shift, want = data["x_2d"], data["shift_2d"], data["out_2d"]
    out = np.full(want.shape, np.float32(-7.0))
    compiled("affine_relu_2d")(x, shift, out)
    assert same_bits(out.reshape(-1), want.reshape(-1))
    # Views that are not contiguous are staged; the rest of the parent array stays as it was.
    parent = np.full((37, 80), np.float32(-7.0))
    compiled("affine_relu_2d")(np.asfortranarray(x), shift, parent[:, 5:75])
    assert same_bits(np.ascontiguousarray(parent[:, 5:75]).reshape(-1), want.reshape(-1))
    assert (parent[:, :5] == -7.0).all() and (parent[:, 75:] == -7.0).all()
    dx, ds, dout = gpu_ctx.to_device(x), gpu_ctx.to_device(shift), gpu_ctx.empty(want.shape, np.float32)
    compiled("affine_relu_2d")(dx, ds, dout)
    assert same_bits(dout.to_numpy().reshape(-1), want.reshape(-1))
    padded = cuda.DeviceBuffer(gpu_ctx, want.shape, np.float32, ld=72)
    with pytest.raises(Exception, match="without row padding"):
        compiled("affine_relu_2d")(dx, ds, padded)
    for buf in (dx, ds, dout, padded):
        buf.free()


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4096, 65537, 1 << 20, (1 << 22) + 3, 20_000_003])
def test_against_the_oracle_on_device_buffers(n: int, gpu_ctx) -> None:
    rng = np.random.default_rng([n, 41])
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    if n > 8:
        x[[1, n // 2]] = np.nan, np.inf
        y[[2, n - 1]] = -np.inf, np.nan
    want = cpu_ref.map_elementwise(x, OPS, other=y)
    assert same_bits(scaled_clamp_numpy(x, y), want)  # the kernel's statements on whole arrays
    dx, dy = gpu_ctx.to_device(x), gpu_ctx.to_device(y)
    guard = 8
    raw = gpu_ctx.empty((n + 2 * guard,), np.float32)
    raw.fill_bytes(0xFF)
    # Aligned output, then one that starts 4 bytes off a 16-byte boundary (the 4-byte path).
    for shift in (guard, guard + 1):
        dout = cuda.DeviceBuffer.wrap(gpu_ctx, raw.ptr + 4 * shift, (n,), np.float32)
        compiled("scaled_clamp")(dx, dy, dout)
        got = raw.to_numpy()
        assert same_bits(got[shift : shift + n], want)
        assert np.isnan(got[:shift]).all() and np.isnan(got[shift + n :]).all()  # nothing written outside
        raw.fill_bytes(0xFF)
    # In place on the first input, through the C ABI binding.
    gpu_ctx.map(dx, dx, OPS, other=dy)
    gpu_ctx.synchronize()
    assert same_bits(dx.to_numpy(), want)
    for buf in (dx, dy, raw):
        buf.free()


def test_every_operation_matches_numpy(gpu_ctx) -> None:
    n = 10007
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(n) * 100).astype(np.float32)
    y = (rng.standard_normal(n) * 100).astype(np.float32)
    x[:4] = np.nan, np.inf, -np.inf, -0.0
    y[:8] = 1.0, 2.0, 3.0, 0.0, np.nan, np.inf, -np.inf, -0.0
    dx, dy, dout = gpu_ctx.to_device(x), gpu_ctx.to_device(y), gpu_ctx.empty((n,), np.float32)
    # (x[3] is -0.0 where y[3] is 0.0, and x[7] is a number where y[7] is -0.0: maximum / minimum of two
    # zeros of opposite sign return the second operand in NumPy, in either order.)
    x[7] = 0.0
    dx.copy_from_host(x)
    for op in (("scale", 0.1), ("add", 0.1), ("max", 0.5), ("min", -0.5), ("rsub", 7.25), ("max", 0.0), ("rmax", 0.0),
               ("min", 0.0), ("rmin", 0.0), ("max", -0.0), ("rmin", -0.0), ("add_other",), ("sub_other",),
               ("rsub_other",), ("mul_other",), ("max_other",), ("min_other",), ("rmax_other",), ("rmin_other",)):
        gpu_ctx.map(dx, dout, (op,), other=dy)
        gpu_ctx.synchronize()
        assert same_bits(dout.to_numpy(), cpu_ref.map_elementwise(x, (op,), other=y)), op
    # A multiply followed by an add rounds twice (no fused multiply-add).
    ops = (("scale", 1.0000001), ("add", -1.0), ("mul_other",), ("add_other",))
    gpu_ctx.map(dx, dout, ops, other=dy)
    gpu_ctx.synchronize()
    assert same_bits(dout.to_numpy(), cpu_ref.map_elementwise(x, ops, other=y))
    gpu_ctx.map(dx, dout, ())  # no operation: a copy
    gpu_ctx.synchronize()
    assert same_bits(dout.to_numpy(), x)
    for buf in (dx, dy, dout):
        buf.free()


def test_host_arrays_travel_in_chunks(gpu_ctx) -> None:
    """More than one 16 MiB chunk, pageable and page-locked arrays, in place."""
    n = (9 << 20) + 5
    rng = np.random.default_rng(6)
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    want = cpu_ref.map_elementwise(x, OPS, other=y)
    out = np.zeros(n, np.float32)
    gpu_ctx.map_host(x, out, OPS, other=y)
    assert same_bits(out, want)
    px, py, pout = (cuda.pinned_empty((n,), np.float32) for _ in range(3))
    px[...], py[...], pout[...] = x, y, 0
    gpu_ctx.map_host(px, pout, OPS, other=py)
    assert same_bits(pout, want)
    gpu_ctx.map_host(px, px, OPS, other=py)
    assert same_bits(px, want)


def test_argument_checks(gpu_ctx) -> None:
    from hc.errors import DeviceError

    d = gpu_ctx.empty((64,), np.float32)
    overlapping = cuda.DeviceBuffer.wrap(gpu_ctx, d.ptr + 16, (32,), np.float32)
    head = cuda.DeviceBuffer.wrap(gpu_ctx, d.ptr, (32,), np.float32)
    with pytest.raises(DeviceError, match="must not partially overlap"):
        gpu_ctx.map(head, overlapping, (("add", 1.0),))
    with pytest.raises(DeviceError, match="must not be null"):
        gpu_ctx.map(head, head, (("add_other",),))
    with pytest.raises(ValueError, match="one length"):
        gpu_ctx.map(head, d, ())
    d.free()
