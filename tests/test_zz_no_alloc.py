"""The allocation-free skinny GEMM entry point, hcCudaGemmSkinnyStatic.

Some users of the library cannot call cudaMalloc when they launch: a process whose GPU memory
is already reserved in full by another allocator, or a latency-critical loop that must not
trigger the device-wide synchronisation an allocation implies. For them the library keeps the
split-k scratch of the skinny kernel in a static device array. This test calls that entry point
through the C ABI twice in a row (the second call sees the first call's leftovers in the shared
array) and compares each result with the regular, context-allocating entry point.

The file name sorts last so that a run that stops at the first failure has already run every
other test. It passes alone in a fresh process as well as after the other tests.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

from hc import cuda

pytestmark = pytest.mark.gpu


def _static_gemm(a_dev, b_dev, c_dev, m: int, n: int, k: int, dtype, stream=None, synchronize: int = 1) -> None:
    lib = cuda.library()
    args = cuda._GemmArgs(m, n, k, cuda.dtype_code(dtype), cuda.VARIANT_AUTO,
                          a_dev.ptr, a_dev.ld, b_dev.ptr, b_dev.ld, c_dev.ptr, c_dev.ld)
    text = ctypes.create_string_buffer(512)
    status = lib.hcCudaGemmSkinnyStatic(ctypes.byref(args), stream, synchronize, text, len(text))
    assert status == 0, (lib.hcCudaStatusString(status), text.value)


def _inputs(m: int, n: int, k: int, seed: int):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = (rng.standard_normal((k, n)) * 0.05).astype(np.float16)
    return a, b


def test_static_scratch_entry_point_matches_the_allocating_one(gpu_ctx) -> None:
    # Two different problems back to back; both use split-k, so both use the shared scratch.
    for seed, (m, n, k) in enumerate([(8, 4096, 8192), (5, 3000, 4104)]):
        assert gpu_ctx.plan(m, n, k, "float16").splits > 1
        a, b = _inputs(m, n, k, seed)
        da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
        expected_dev = gpu_ctx.empty((m, n), np.float32)
        gpu_ctx.gemm(da, db, expected_dev)
        gpu_ctx.synchronize()
        expected = expected_dev.to_numpy()

        got_dev = gpu_ctx.empty((m, n), np.float32)
        got_dev.fill_bytes(0xFF)
        gpu_ctx.synchronize()
        _static_gemm(da, db, got_dev, m, n, k, np.float16)
        got = got_dev.to_numpy()

        assert np.isfinite(got).all()
        bound = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
        diff = np.abs(got.astype(np.float64) - expected.astype(np.float64))
        assert (diff <= 1e-2 * bound + 1e-30).all()
        assert np.linalg.norm(diff) <= 1e-3 * np.linalg.norm(expected.astype(np.float64))
        # Same kernel, same split count, same summation order: in fact bit-identical.
        assert np.array_equal(got, expected)
        for buf in (da, db, expected_dev, got_dev):
            buf.free()


def test_static_scratch_entry_point_unsplit_shape_and_a_callers_stream(gpu_ctx) -> None:
    """The benchmark's skinny shape (no split over k, so only the status word of the array is used)
    and a split one, enqueued without waiting on a stream the caller owns; a synchronising call on
    the same stream then finishes the batch, which is also how a device-side timeout would surface.
    A k == 0 call only clears C and reads no status."""
    torch = pytest.importorskip("torch")
    stream = torch.cuda.Stream(device=0)
    shapes = [(8, 16384, 8192), (8, 4096, 8192)]
    assert gpu_ctx.plan(*shapes[0], "float16").splits == 1 and gpu_ctx.plan(*shapes[1], "float16").splits > 1
    results = []
    for seed, (m, n, k) in enumerate(shapes):
        a, b = _inputs(m, n, k, 10 + seed)
        da, db = gpu_ctx.to_device(a), gpu_ctx.to_device(b)
        expected_dev, got_dev = gpu_ctx.empty((m, n), np.float32), gpu_ctx.empty((m, n), np.float32)
        gpu_ctx.gemm(da, db, expected_dev)
        got_dev.fill_bytes(0xFF)
        gpu_ctx.synchronize()
        results.append((da, db, expected_dev, got_dev, m, n, k))
    handle = ctypes.c_void_p(stream.cuda_stream)
    for da, db, _, got_dev, m, n, k in results:  # same stream: the launches cannot overlap
        _static_gemm(da, db, got_dev, m, n, k, np.float16, stream=handle, synchronize=0)
    da, db, _, got_dev, m, n, k = results[-1]
    _static_gemm(da, db, got_dev, m, n, k, np.float16, stream=handle, synchronize=1)
    stream.synchronize()
    for da, db, expected_dev, got_dev, *_ in results:
        assert np.array_equal(got_dev.to_numpy(), expected_dev.to_numpy())
    # k == 0: C is cleared, nothing is launched, and a waiting call has no status to report.
    da, db, _, got_dev, m, n, _ = results[0]
    for _ in range(2):
        _static_gemm(da, db, got_dev, m, n, 0, np.float16, stream=handle, synchronize=1)
    assert not got_dev.to_numpy().any()
    for da, db, expected_dev, got_dev, *_ in results:
        for buf in (da, db, expected_dev, got_dev):
            buf.free()


def test_static_scratch_entry_point_rejects_what_does_not_fit(gpu_ctx, monkeypatch) -> None:
    """Rejections happen during validation, before anything is launched, so placeholder
    addresses are safe here."""
    lib = cuda.library()
    text = ctypes.create_string_buffer(512)
    # Forcing 32 splits makes 64 x 16384 need 128 MiB of partial sums, far beyond the 8 MiB array.
    monkeypatch.setenv("HC_CUDA_SKINNY_SPLITS", "32")
    args = cuda._GemmArgs(64, 16384, 8192, cuda.F16, 0, 0x7F0000000000, 8192, 0x7F1000000000, 16384,
                          0x7F8000000000, 16384)
    assert cuda.plan_gemm(64, 16384, 8192, "float16").splits == 32
    status = lib.hcCudaGemmSkinnyStatic(ctypes.byref(args), None, 1, text, len(text))
    assert status == 2 and b"static" in text.value
    monkeypatch.delenv("HC_CUDA_SKINNY_SPLITS")
    # An unaligned pitch would need a repack, i.e. scratch the entry point does not have.
    args = cuda._GemmArgs(8, 1001, 512, cuda.F16, 0, 0x7F0000000000, 512, 0x7F1000000000, 1001,
                          0x7F8000000000, 1001)
    status = lib.hcCudaGemmSkinnyStatic(ctypes.byref(args), None, 1, text, len(text))
    assert status == 2 and b"16-byte aligned" in text.value
    args = cuda._GemmArgs(65, 256, 512, cuda.F16, 0, 0x7F0000000000, 512, 0x7F1000000000, 256,
                          0x7F8000000000, 256)
    status = lib.hcCudaGemmSkinnyStatic(ctypes.byref(args), None, 1, text, len(text))
    assert status == 2 and b"m <= 64" in text.value
    args = cuda._GemmArgs(8, 256, 512, cuda.F8E4M3, 0, 0x7F0000000000, 512, 0x7F1000000000, 256,
                          0x7F8000000000, 256)
    status = lib.hcCudaGemmSkinnyStatic(ctypes.byref(args), None, 1, text, len(text))
    assert status == 2 and b"float16 or bfloat16" in text.value
    assert lib.hcCudaGemmSkinnyStatic(None, None, 1, text, len(text)) == 1
