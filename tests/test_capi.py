"""The C ABI on a machine without a GPU: the library loads, exports every declared symbol,
and its host-side validation / planning behaves. No compute call is made here."""

from __future__ import annotations

import ctypes
import re

import pytest

from conftest import REPO
from hc import cuda
from hc.errors import DeviceError

HEADER = REPO / "include" / "hc-c" / "Cuda.h"


def _declared_functions() -> list[str]:
    text = HEADER.read_text(encoding="utf-8")
    return re.findall(r"HC_CUDA_CAPI_EXPORTED\s+[\w\s\*]+?\b(hcCuda\w+)\s*\(", text)


def test_library_exports_every_declared_symbol() -> None:
    lib = cuda.library()
    declared = _declared_functions()
    assert len(declared) >= 28 and len(set(declared)) == len(declared)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in hc-c/Cuda.h but not exported"
    assert set(declared) == set(cuda.EXPORTS)
    assert lib.hcCudaApiVersion() == cuda.API_VERSION


def test_every_declaration_cites_or_describes_its_reference_counterpart() -> None:
    text = HEADER.read_text(encoding="utf-8")
    for anchor in ("hc/_compile.py:57-62", "hc/simulator.py:165-186", "hc/simulator.py:752-768",
                   "include/hc-c/HC.h", "lib/CAPI/HC.cpp:22-29"):
        assert anchor in text


def test_status_strings() -> None:
    lib = cuda.library()
    assert lib.hcCudaStatusString(0) == b"HC_CUDA_OK"
    assert lib.hcCudaStatusString(5) == b"HC_CUDA_ERR_DEVICE_TIMEOUT"
    assert lib.hcCudaStatusString(99) == b"HC_CUDA_ERR_UNKNOWN"


def test_missing_device_is_reported_not_papered_over() -> None:
    if cuda.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(DeviceError, match="HC_CUDA_ERR_NO_DEVICE"):
        cuda.Context(0)
    lib = cuda.library()
    assert lib.hcCudaContextCreate(0, None) == 1  # null out-pointer
    assert lib.hcCudaContextSynchronize(None) == 1
    assert lib.hcCudaGemm(None, None) == 1


def skinny_tile_n_is_zero() -> bool:
    return cuda.plan_gemm(8, 16384, 8192, "float16").tile_n == 0


def test_plan_chooses_variants() -> None:
    dense = cuda.plan_gemm(8192, 8192, 8192, "float16")
    assert (dense.variant, dense.tiles_m, dense.tiles_n, dense.grid, dense.splits) == ("dense", 16, 32, 148, 1)  # 512x256 tiles
    # The 512x256 tiles need a long k-loop, several rounds of tiles, and an epilogue that never reads C
    # with ordinary loads; otherwise the 256x256 pair tiles (or 128x256 single-CTA tiles) run.
    assert cuda.plan_gemm(8192, 8192, 512, "float16").tiles_m == 32
    assert cuda.plan_gemm(4096, 4096, 4096, "float16").tiles_m == 16
    assert cuda.plan_gemm(8192, 8192, 8192, "float16", accumulate=True).tiles_m == 16
    assert cuda.plan_gemm(8192, 8192, 8192, "float16", accumulate=True, epilogue=(("scale", 2.0),)).tiles_m == 32
    assert cuda.plan_gemm(8192, 8192, 8192, "float16", accumulate=True, ldc=8193).tiles_m == 32
    assert cuda.plan_gemm(8192, 8192, 8192, "float16", ldc=8193).tiles_m == 16
    assert dense.kernel_launches == 1 and dense.scratch_bytes == 0 and not dense.repack_a
    small = cuda.plan_gemm(100, 300, 64, "bfloat16")
    assert (small.variant, small.tiles_m, small.tiles_n, small.grid, small.tile_n) == ("dense", 1, 3, 3, 128)
    # 128-wide tiles for small unsplit products that would otherwise leave most SMs idle.
    little = cuda.plan_gemm(1024, 1024, 1024, "float16")
    assert (little.tile_n, little.tiles_m, little.tiles_n, little.grid, little.splits) == (128, 8, 8, 64, 1)
    assert cuda.plan_gemm(1024, 1024, 4096, "float16").tile_n == 256  # a long k: shared among clusters instead
    # One round of 128 x 256 tiles and a moderate k: single CTAs, not pairs (a cluster launch costs more);
    # 72 tiles are split in two over k and the halves meet in a cluster of two.
    mid = cuda.plan_gemm(1536, 1536, 1536, "float16")
    assert (mid.tile_n, mid.tiles_m, mid.tiles_n, mid.grid, mid.splits, mid.cluster_size) == (256, 12, 6, 144, 2, 2)
    square = cuda.plan_gemm(2048, 2048, 2048, "float16")
    assert (square.tile_n, square.tiles_m, square.tiles_n, square.grid, square.splits) == (256, 16, 8, 128, 1)
    assert cuda.plan_gemm(512, 8192, 8192, "float16").tiles_m == 2  # a long k: CTA pairs
    assert cuda.plan_gemm(2560, 2560, 2560, "float16").tile_n == 256  # more than a round of narrow tiles
    assert dense.tile_n == 256 and cuda.plan_gemm(4096, 4096, 1024, "float16").tile_n == 256
    assert cuda.plan_gemm(512, 512, 16384, "float16").tile_n == 256  # shared among clusters instead
    assert skinny_tile_n_is_zero()
    skinny = cuda.plan_gemm(8, 16384, 8192, "float16")
    assert (skinny.variant, skinny.tiles_n, skinny.splits, skinny.grid) == ("skinny", 128, 1, 128)
    assert skinny.scratch_bytes == 0  # enough column blocks to fill the GPU: no split over k
    narrow = cuda.plan_gemm(8, 2048, 8192, "float16")
    assert narrow.splits == 8 and narrow.grid == 128 and narrow.scratch_bytes == 8 * 8 * 2048 * 4
    assert cuda.plan_gemm(64, 512, 512, "float16").variant == "skinny"
    assert cuda.plan_gemm(65, 512, 512, "float16").variant == "dense"
    assert cuda.plan_gemm(8, 512, 512, "float16", variant=cuda.VARIANT_DENSE).variant == "dense"
    assert cuda.plan_gemm(8, 128, 64, "float16", variant=cuda.VARIANT_SKINNY).splits == 1


def test_plan_flags_pitches_that_need_a_repack() -> None:
    ragged = cuda.plan_gemm(4095, 3073, 1031, "bfloat16")
    assert ragged.variant == "dense" and ragged.repack_a and ragged.repack_b and ragged.kernel_launches == 2
    assert (ragged.tiles_m, ragged.tiles_n) == (16, 13)
    assert ragged.scratch_bytes >= 4095 * 1088 * 2 + 1031 * 3136 * 2
    padded = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", lda=1032, ldb=3080)
    assert not padded.repack_a and not padded.repack_b and padded.kernel_launches == 1
    misaligned_base = cuda.plan_gemm(128, 256, 64, "float16", a=0x1002)
    assert misaligned_base.repack_a and not misaligned_base.repack_b


def test_plan_with_b_stored_transposed() -> None:
    plan = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", b_transposed=True)
    assert plan.variant == "dense" and plan.repack_a and plan.repack_b and plan.kernel_launches == 2
    assert plan.scratch_bytes >= 4095 * 1088 * 2 + 3073 * 1088 * 2  # B is n rows of k as stored
    aligned = cuda.plan_gemm(512, 1000, 1024, "float16", b_transposed=True)
    assert not aligned.repack_b  # pitch k = 1024 is TMA-legal although n is not a multiple of 8
    with pytest.raises(DeviceError, match="ldb \\(63\\) must be at least k \\(64\\)"):
        cuda.plan_gemm(128, 256, 64, "float16", ldb=63, b_transposed=True)
    lib = cuda.library()
    args = cuda._GemmArgs(8, 8, 8, 0, 0, 0x1000, 8, 0x2000, 8, 0x3000, 8, 5, 0)
    info = cuda._PlanInfo()
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"b_layout" in lib.hcCudaContextLastError(None)
    args = cuda._GemmArgs(8, 8, 8, 0, 0, 0x1000, 8, 0x2000, 8, 0x3000, 8, 0, 0)
    args.c_dtype = 3
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"c_dtype" in lib.hcCudaContextLastError(None)


def test_plan_with_a_16_bit_c() -> None:
    """C may be float16 or bfloat16 (the float32 result rounded on store); it then needs only 2-byte
    alignment, and is not offered together with accumulation."""
    plan = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", lda=1031, ldb=3073, ldc=3073, c_dtype="bfloat16")
    plain = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", lda=1031, ldb=3073, ldc=3073)
    assert (plan.variant, plan.grid, plan.kernel_launches) == (plain.variant, plain.grid, plain.kernel_launches)
    assert cuda.plan_gemm(8, 512, 1024, "float16", c=0x80000002, c_dtype="float16").variant == "skinny"
    with pytest.raises(DeviceError, match="c must be 4-byte aligned"):
        cuda.plan_gemm(8, 512, 1024, "float16", c=0x80000002)
    with pytest.raises(DeviceError, match="c must be 2-byte aligned"):
        cuda.plan_gemm(8, 512, 1024, "float16", c=0x80000001, c_dtype="float16")
    with pytest.raises(DeviceError, match="HC_CUDA_ERR_UNSUPPORTED: accumulate needs a float32 C"):
        cuda.plan_gemm(64, 64, 64, "float16", accumulate=True, c_dtype="float16")
    assert cuda.plan_gemm(64, 64, 0, "float16", c_dtype="bfloat16").variant == "zero_fill"
    assert cuda.plan_gemm(64, 64, 0, "float16", c_dtype="bfloat16", epilogue=(("add", 1.0),)).variant == "elementwise"
    with pytest.raises(ValueError, match="C must be float32, float16 or bfloat16"):
        cuda.plan_gemm(64, 64, 64, "float16", c_dtype="float64")


def test_plan_with_accumulate_and_fused_operations() -> None:
    """The C += A.B member and the element-wise operations folded into the store."""
    assert ctypes.sizeof(cuda._GemmArgs) == 136  # the layout include/hc-c/Cuda.h declares
    plain = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", lda=1031, ldb=3073, ldc=3073)
    fused = cuda.plan_gemm(4095, 3073, 1031, "bfloat16", lda=1031, ldb=3073, ldc=3073, accumulate=True,
                           epilogue=(("scale", 0.5), ("bias",), ("max", 0.0), ("min", 6.0)))
    assert (fused.variant, fused.grid, fused.kernel_launches) == (plain.variant, plain.grid, plain.kernel_launches)
    # k == 0: nothing to add. C stays (accumulate), is zeroed, or only gets the element-wise work.
    assert cuda.plan_gemm(64, 64, 0, "float16", accumulate=True).variant == "noop"
    assert cuda.plan_gemm(64, 64, 0, "float16").variant == "zero_fill"
    only = cuda.plan_gemm(64, 64, 0, "float16", accumulate=True, epilogue=(("add", 1.0),))
    assert only.variant == "elementwise" and only.kernel_launches == 1
    with pytest.raises(DeviceError, match="at most one HC_CUDA_EPILOGUE_BIAS_COLUMN"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("bias",), ("bias",)))
    with pytest.raises(DeviceError, match="bias must be a 4-byte-aligned pointer"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("bias",),), bias=None)
    with pytest.raises(DeviceError, match="bias must be a 4-byte-aligned pointer"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("bias",),), bias=0xC0000002)
    with pytest.raises(DeviceError, match="c must not overlap bias"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("bias",),), bias=0x80000000 + 64)
    with pytest.raises(ValueError, match="at most 4 fused"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("add", 1.0),) * 5)
    with pytest.raises(ValueError, match="unknown fused operation"):
        cuda.plan_gemm(64, 64, 64, "float16", epilogue=(("divide", 2.0),))
    lib = cuda.library()
    info = cuda._PlanInfo()
    args = cuda._gemm_args(8, 8, 8, "float16", 0x1000, 8, 0x2000, 8, 0x3000, 8, 0)
    args.accumulate = 2
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"accumulate" in lib.hcCudaContextLastError(None)
    args.accumulate, args.epilogue_count = 0, 5
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"epilogue_count" in lib.hcCudaContextLastError(None)
    args.epilogue_count = 1
    args.epilogue_kind[0] = 9
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"epilogue_kind[0]" in lib.hcCudaContextLastError(None)


def test_plan_splits_dense_tiles_that_do_not_fill_a_round() -> None:
    """Few tiles and a long k: every tile is split. More tiles than CTAs with a small remainder and
    k >= 8192: only the last round's tiles. Otherwise nothing is split."""
    few = cuda.plan_gemm(128, 8192, 8192, "float16", ldc=8192 + 1)  # (a C that TMA cannot address)
    assert (few.variant, few.tiles_m, few.tiles_n, few.splits, few.first_split_tile, few.grid) == ("dense", 1, 32, 4, 0, 128)
    assert few.scratch_bytes == 32 * 4 * 128 * 256 * 4 and few.kernel_launches == 1 and few.cluster_size == 0
    one_tile = cuda.plan_gemm(256, 256, 32768, "bfloat16", c_dtype="bfloat16")
    assert one_tile.splits == 32 and one_tile.grid == 64 and one_tile.cluster_size == 0  # 32 CTA pairs
    tail = cuda.plan_gemm(4864, 1024, 8192, "float16")  # 19 x 4 pair tiles = one round of 74 + 2
    assert (tail.splits, tail.first_split_tile, tail.grid) == (8, 74, 148)
    assert tail.scratch_bytes == 2 * 8 * 256 * 256 * 4
    for shape in ((8192, 8192, 8192), (4096, 4096, 4096), (4095, 3073, 1031), (512, 8192, 8192), (1024, 1024, 1024)):
        plan = cuda.plan_gemm(*shape, "float16")
        assert plan.splits == 1 and plan.first_split_tile == 0 and plan.scratch_bytes % (1 << 10) == 0, (shape, plan)
    # Short k: the k-loop a split would shorten is not worth its partial tiles.
    assert cuda.plan_gemm(128, 8192, 512, "float16").splits == 1
    # Fewer SMs, more rounds.
    assert cuda.plan_gemm(128, 8192, 8192, "float16", sm_count=32).splits == 1


def test_plan_shares_few_tiles_among_clusters() -> None:
    """Few tiles, a long k and a float32 C that TMA can address: each 128x256 tile goes to one or several
    thread-block clusters, every CTA a range of k; partial tiles in global memory only between clusters."""
    few = cuda.plan_gemm(128, 8192, 8192, "float16")  # 32 tiles: clusters of four fill 128 SMs
    assert (few.cluster_size, few.splits, few.tiles_m, few.tiles_n, few.grid) == (4, 4, 1, 32, 128)
    assert few.scratch_bytes == 0 and few.first_split_tile == 0 and few.kernel_launches == 1
    one = cuda.plan_gemm(256, 256, 32768, "bfloat16")  # 2 tiles: seven clusters of eight each
    assert (one.cluster_size, one.splits, one.tiles_m, one.tiles_n, one.grid) == (8, 56, 2, 1, 112)
    assert one.scratch_bytes == 2 * 7 * 128 * 256 * 4
    mid = cuda.plan_gemm(512, 512, 16384, "float16", accumulate=True, epilogue=(("scale", 0.5),))
    assert (mid.cluster_size, mid.splits, mid.grid) == (4, 16, 128)
    # Products that fill the GPU with whole tiles, a short k, and the last round of a larger product
    # are not shared.
    for shape in ((8192, 8192, 8192), (2048, 2048, 2048), (128, 8192, 512), (4864, 1024, 8192)):
        assert cuda.plan_gemm(*shape, "float16").cluster_size == 0, shape
    # 8 < m <= 64 with few column blocks: the shared dense tiles instead of the skinny kernel's split;
    # not for m <= 8, not when there are column blocks enough, not when C rules the clusters out.
    assert (cuda.plan_gemm(64, 8192, 8192, "float16").variant, cuda.plan_gemm(64, 8192, 8192, "float16").cluster_size) == ("dense", 4)
    assert cuda.plan_gemm(33, 4096, 8192, "bfloat16").cluster_size == 4
    for kwargs in (dict(m=8, n=8192), dict(m=64, n=16384), dict(m=64, n=8192, ldc=8193), dict(m=64, n=8192, c_dtype="float16")):
        shape = dict(m=64, n=8192, k=8192) | {k_: v for k_, v in kwargs.items() if k_ in ("m", "n")}
        extra = {k_: v for k_, v in kwargs.items() if k_ not in ("m", "n")}
        plan = cuda.plan_gemm(shape["m"], shape["n"], shape["k"], "float16", **extra)
        assert (plan.variant, plan.cluster_size) == ("skinny", 0), (kwargs, plan)
    # A smaller device: fewer clusters at once.
    small = cuda.plan_gemm(256, 256, 32768, "float16", sm_count=64)
    assert small.cluster_size >= 2 and small.grid <= 64


def test_library_calls_from_threads() -> None:
    """Loading the library and planning are safe from several threads at once (one-time
    initialisation, thread-local error text)."""
    import threading

    seen: list = []

    def work(i: int) -> None:
        for _ in range(200):
            plan = cuda.plan_gemm(128 + i, 256, 512, "float16")
            assert plan.variant == "dense"
            try:
                cuda.plan_gemm(8, 8, 8, "float16", lda=4 + i % 3)
            except DeviceError as exc:
                assert f"lda ({4 + i % 3}) must be at least k (8)" in str(exc)  # this thread's own message
            else:  # pragma: no cover
                raise AssertionError("expected a DeviceError")
        seen.append(i)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert sorted(seen) == list(range(8))


def test_plan_degenerate_shapes() -> None:
    assert cuda.plan_gemm(0, 5, 7, "float16").variant == "noop"
    assert cuda.plan_gemm(5, 0, 7, "float16").kernel_launches == 0
    zero_k = cuda.plan_gemm(5, 6, 0, "float16")
    assert zero_k.variant == "zero_fill" and zero_k.kernel_launches == 0


@pytest.mark.parametrize(
    ("kwargs", "status", "message"),
    [
        ({"m": -1}, "INVALID_ARGUMENT", "non-negative"),
        ({"m": (1 << 30) + 1}, "UNSUPPORTED", "at most 2\\^30"),
        ({"a": 0}, "INVALID_ARGUMENT", "a and b must not be null"),
        ({"c": 0}, "INVALID_ARGUMENT", "c must not be null"),
        ({"c": 0x80000002}, "INVALID_ARGUMENT", "4-byte aligned"),
        ({"b": 0x40000001}, "INVALID_ARGUMENT", "aligned to their element size"),
        ({"lda": 63}, "INVALID_ARGUMENT", "lda \\(63\\) must be at least k \\(64\\)"),
        ({"ldb": 10}, "INVALID_ARGUMENT", "ldb"),
        ({"ldc": 10}, "INVALID_ARGUMENT", "ldc"),
        ({"c": 0x1000}, "INVALID_ARGUMENT", "must not overlap"),
        ({"c": 0x40000000 + 64}, "INVALID_ARGUMENT", "must not overlap"),
        ({"variant": 7}, "INVALID_ARGUMENT", "variant must be"),
        ({"m": 65, "variant": cuda.VARIANT_SKINNY}, "UNSUPPORTED", "skinny variant needs m <= 64"),
    ],
)
def test_plan_rejects_bad_arguments(kwargs: dict, status: str, message: str) -> None:
    args = {"m": 128, "n": 256, "k": 64, "dtype": "float16"}
    args.update(kwargs)
    with pytest.raises(DeviceError, match=message) as info:
        cuda.plan_gemm(args.pop("m"), args.pop("n"), args.pop("k"), args.pop("dtype"), **args)
    assert info.value.status_name == f"HC_CUDA_ERR_{status}"


def test_plan_rejects_unknown_dtype_code() -> None:
    lib = cuda.library()
    args = cuda._GemmArgs(1, 1, 1, 5, 0, 0x1000, 1, 0x2000, 1, 0x3000, 1)
    info = cuda._PlanInfo()
    assert lib.hcCudaGemmPlan(ctypes.byref(args), 148, ctypes.byref(info)) == 1
    assert b"dtype" in lib.hcCudaContextLastError(None)
    assert lib.hcCudaGemmPlan(None, 148, ctypes.byref(info)) == 1
    with pytest.raises(ValueError):
        cuda.plan_gemm(1, 1, 1, "float32")


def test_comm_entry_points_validate_before_touching_nccl() -> None:
    lib = cuda.library()
    assert lib.hcCudaCommGetUniqueId(None, 128) == 1
    buf = ctypes.create_string_buffer(16)
    assert lib.hcCudaCommGetUniqueId(buf, 16) == 1
    assert lib.hcCudaCommAllGather(None, None, None, 0) == 1
    assert lib.hcCudaCommInitRank(None, buf, 16, 2, 0) == 1


def test_checked_build_exports_the_same_symbols() -> None:
    """`python 5_b200/build.py --checked` gives libhc_cuda_checked.so: the same C ABI, with index checks
    compiled into the kernels (a flag says which build a library is)."""
    import importlib

    checked = importlib.import_module("build").build(checked=True)  # (5_b200/ is on the path: conftest)
    assert checked.name == "libhc_cuda_checked.so" and checked.exists()
    lib = ctypes.CDLL(str(checked))
    for name in cuda.EXPORTS:
        assert hasattr(lib, name), name
    assert lib.hcCudaBuildFlags() & 1 and not cuda.library_is_checked()
    assert lib.hcCudaApiVersion() == cuda.API_VERSION
    lib.hcCudaStatusString.restype = ctypes.c_char_p
    assert lib.hcCudaStatusString(8) == b"HC_CUDA_ERR_DEVICE_CHECK"


def test_plan_sends_one_small_tile_with_a_short_k_to_the_tiny_variant() -> None:
    """m, n <= 64 and k <= 128 (benchmark configuration 1 and every matmul fixture): the float32 kernel
    that is bit-identical to the reference simulator; it needs no repack and no scratch whatever the
    pitches, takes no float8, and can be asked for on any shape."""
    plan = cuda.plan_gemm(64, 64, 64, "float16")
    assert (plan.variant, plan.tiles_m, plan.tiles_n, plan.grid, plan.splits, plan.kernel_launches) == ("tiny", 4, 4, 16, 1, 1)
    odd = cuda.plan_gemm(33, 17, 40, "bfloat16", lda=41, ldb=19, ldc=23, a=0x1002)
    assert (odd.variant, odd.repack_a, odd.repack_b, odd.scratch_bytes) == ("tiny", False, False, 0)
    for shape in ((65, 64, 64), (64, 65, 64), (64, 64, 129)):
        assert cuda.plan_gemm(*shape, "float16").variant != "tiny", shape
    assert cuda.plan_gemm(64, 64, 64, "float8_e5m2", b_transposed=True).variant == "skinny"
    forced = cuda.plan_gemm(300, 500, 700, "float16", variant=cuda.VARIANT_TINY)
    assert (forced.variant, forced.tiles_m, forced.tiles_n, forced.grid) == ("tiny", 19, 32, 19 * 32)
    with pytest.raises(DeviceError, match="16-bit operands"):
        cuda.plan_gemm(64, 64, 64, "float8_e5m2", b_transposed=True, variant=cuda.VARIANT_TINY)
    with pytest.raises(DeviceError, match="variant must be AUTO, DENSE, SKINNY or TINY"):
        cuda.plan_gemm(64, 64, 64, "float16", variant=7)
