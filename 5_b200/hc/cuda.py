"""ctypes binding of include/hc-c/Cuda.h plus the small device-memory objects a launch needs.

Host code stays NumPy: a `DeviceBuffer` is a (pointer, shape, dtype, pitch) record whose
memory lives on the GPU, and `pinned_empty` gives NumPy arrays in page-locked memory so that
host<->device copies run at full PCIe speed. There is no CPU fallback anywhere in this
module: when the shared library is missing or no sm_100 device is present, the calls raise.

The library is looked up at `$HC_CUDA_LIB`, else at `lib/libhc_cuda.so` beside this package
(built by `5_b200/build.py`).
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from collections.abc import Sequence
from typing import Any

import numpy as np

from .errors import DeviceError

__all__ = [
    "Context",
    "DeviceBuffer",
    "GemmPlan",
    "BoundGemm",
    "default_context",
    "device_count",
    "library",
    "library_path",
    "pinned_empty",
    "plan_gemm",
]

F16, BF16, F8E4M3, F8E5M2 = 0, 1, 2, 3  # HcCudaDType
VARIANT_AUTO, VARIANT_DENSE, VARIANT_SKINNY, VARIANT_NOOP, VARIANT_ZERO_FILL, VARIANT_ELEMENTWISE = 0, 1, 2, 3, 4, 5
VARIANT_TINY = 6  # float32 pipes, bit-identical to the reference simulator; AUTO picks it for m, n <= 64, k <= 128
VARIANT_NAMES = {0: "auto", 1: "dense", 2: "skinny", 3: "noop", 4: "zero_fill", 5: "elementwise", 6: "tiny"}
API_VERSION = 8
# Element-wise operations fused into the store of C: ("scale", x), ("add", x), ("max", x),
# ("min", x) and ("bias",) -- the last adds bias[column].
EPILOGUE_KINDS = {"scale": 1, "add": 2, "max": 3, "min": 4, "bias": 5}
MAX_EPILOGUE_OPS = 4
COMM_ID_BYTES = 128
IPC_HANDLE_BYTES = 64
MAX_PUSH_TARGETS = 7

EXPORTS = (
    "hcCudaApiVersion", "hcCudaStatusString", "hcCudaGetDeviceCount", "hcCudaContextCreate",
    "hcCudaContextDestroy", "hcCudaContextLastError", "hcCudaContextGetDeviceInfo",
    "hcCudaContextSynchronize", "hcCudaMalloc", "hcCudaFree", "hcCudaHostAlloc", "hcCudaHostFree",
    "hcCudaMemcpyHtoD", "hcCudaMemcpyDtoH", "hcCudaMemcpy2DHtoD", "hcCudaMemcpy2DDtoH",
    "hcCudaMemset", "hcCudaGemmPlan", "hcCudaGemm", "hcCudaGemmHost", "hcCudaEventCreate",
    "hcCudaEventDestroy", "hcCudaEventRecord", "hcCudaEventElapsedMs", "hcCudaCommGetUniqueId",
    "hcCudaCommInitRank", "hcCudaCommAllGather", "hcCudaCommDestroy", "hcCudaGemmSkinnyStatic", "hcCudaSelfTestDeviceTimeout", "hcCudaGemmPush", "hcCudaIpcExport",
    "hcCudaIpcOpen", "hcCudaIpcClose", "hcCudaMap", "hcCudaMapHost",
    "hcCudaGemmHostDeviceA", "hcCudaPairwise", "hcCudaPairwiseHost", "hcCudaRowSum", "hcCudaRowSumHost", "hcCudaBuildFlags", "hcCudaSelfTestDeviceCheck",
)


class _GemmArgs(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("dtype", ctypes.c_int32), ("variant", ctypes.c_int32),
        ("a", ctypes.c_void_p), ("lda", ctypes.c_int64),
        ("b", ctypes.c_void_p), ("ldb", ctypes.c_int64),
        ("c", ctypes.c_void_p), ("ldc", ctypes.c_int64),
        ("b_layout", ctypes.c_int32), ("accumulate", ctypes.c_int32),
        ("epilogue_count", ctypes.c_int32), ("epilogue_kind", ctypes.c_int32 * 4),
        ("epilogue_value", ctypes.c_float * 4), ("c_dtype", ctypes.c_int32),
        ("bias", ctypes.c_void_p),
    ]


# Operations of the element-wise map (HcCudaMapOp): with a float32 constant, or with the element of
# the second input ("..._other").
MAP_KINDS = {"scale": 1, "add": 2, "max": 3, "min": 4, "rsub": 5, "add_other": 6, "sub_other": 7,
             "rsub_other": 8, "mul_other": 9, "max_other": 10, "min_other": 11, "rmax": 12, "rmin": 13,
             "rmax_other": 14, "rmin_other": 15}
MAX_MAP_OPS = 8


class _MapArgs(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_int64), ("x", ctypes.c_void_p), ("y", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("op_count", ctypes.c_int32), ("op_kind", ctypes.c_int32 * 8), ("op_value", ctypes.c_float * 8),
    ]


def _map_args(n: int, x: int | None, y: int | None, out: int | None, ops: Sequence[tuple]) -> _MapArgs:
    ops = tuple(ops)
    if len(ops) > MAX_MAP_OPS:
        raise ValueError(f"at most {MAX_MAP_OPS} element-wise operations are supported")
    args = _MapArgs(n=n, x=x, y=y, out=out, op_count=len(ops))
    for i, op in enumerate(ops):
        if op[0] not in MAP_KINDS:
            raise ValueError(f"unknown element-wise operation {op[0]!r}; known: {sorted(MAP_KINDS)}")
        args.op_kind[i] = MAP_KINDS[op[0]]
        args.op_value[i] = float(op[1]) if len(op) > 1 else 0.0
    return args


class _PlanInfo(ctypes.Structure):
    _fields_ = [
        ("variant", ctypes.c_int32), ("tiles_m", ctypes.c_int32), ("tiles_n", ctypes.c_int32),
        ("splits", ctypes.c_int32), ("grid", ctypes.c_int32), ("repack_a", ctypes.c_int32),
        ("repack_b", ctypes.c_int32), ("kernel_launches", ctypes.c_int32),
        ("scratch_bytes", ctypes.c_int64), ("first_split_tile", ctypes.c_int32), ("ring_stages", ctypes.c_int32),
        ("cluster_size", ctypes.c_int32), ("tile_n", ctypes.c_int32),
    ]


class _PairwiseArgs(ctypes.Structure):
    _fields_ = [
        ("w1", ctypes.c_int64), ("w2", ctypes.c_int64), ("h", ctypes.c_int64),
        ("x1", ctypes.c_void_p), ("ld1", ctypes.c_int64), ("x2", ctypes.c_void_p), ("ld2", ctypes.c_int64),
        ("out", ctypes.c_void_p), ("ldo", ctypes.c_int64), ("op", ctypes.c_int32),
    ]


PAIRWISE_EUCLIDEAN, PAIRWISE_SQUARED = 0, 1


class _RowSumArgs(ctypes.Structure):
    _fields_ = [("w", ctypes.c_int64), ("h", ctypes.c_int64), ("x", ctypes.c_void_p), ("ldx", ctypes.c_int64),
                ("out", ctypes.c_void_p), ("flags", ctypes.c_int32)]


ROW_SUM_SQUARE, ROW_SUM_SQRT = 1, 2


class _DeviceInfo(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 128), ("device", ctypes.c_int32), ("cc_major", ctypes.c_int32),
        ("cc_minor", ctypes.c_int32), ("sm_count", ctypes.c_int32),
        ("total_memory_bytes", ctypes.c_int64), ("l2_bytes", ctypes.c_int32),
        ("sm_clock_khz", ctypes.c_int32),
    ]


_LIB: ctypes.CDLL | None = None
_LIB_LOCK = threading.Lock()


def library_path() -> Path:
    override = os.environ.get("HC_CUDA_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent.parent / "lib" / "libhc_cuda.so"


def library() -> ctypes.CDLL:
    """Loads libhc_cuda.so once. Raises ImportError (never falls back) when it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LIB_LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not path.exists():
            raise ImportError(
                f"the hc CUDA library was not found at {path}; build it with "
                "`python 5_b200/build.py` or point HC_CUDA_LIB at it"
            )
        lib = ctypes.CDLL(str(path))
        vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        pvp = ctypes.POINTER(ctypes.c_void_p)
        lib.hcCudaApiVersion.restype = i
        lib.hcCudaStatusString.restype = ctypes.c_char_p
        lib.hcCudaStatusString.argtypes = [i]
        lib.hcCudaGetDeviceCount.argtypes = [ctypes.POINTER(i)]
        lib.hcCudaContextCreate.argtypes = [i, pvp]
        lib.hcCudaContextDestroy.argtypes = [vp]
        lib.hcCudaContextLastError.restype = ctypes.c_char_p
        lib.hcCudaContextLastError.argtypes = [vp]
        lib.hcCudaContextGetDeviceInfo.argtypes = [vp, ctypes.POINTER(_DeviceInfo)]
        lib.hcCudaContextSynchronize.argtypes = [vp]
        lib.hcCudaMalloc.argtypes = [vp, sz, pvp]
        lib.hcCudaFree.argtypes = [vp, vp]
        lib.hcCudaHostAlloc.argtypes = [sz, pvp]
        lib.hcCudaHostFree.argtypes = [vp]
        lib.hcCudaMemcpyHtoD.argtypes = [vp, vp, vp, sz]
        lib.hcCudaMemcpyDtoH.argtypes = [vp, vp, vp, sz]
        lib.hcCudaMemcpy2DHtoD.argtypes = [vp, vp, sz, vp, sz, sz, sz]
        lib.hcCudaMemcpy2DDtoH.argtypes = [vp, vp, sz, vp, sz, sz, sz]
        lib.hcCudaMemset.argtypes = [vp, vp, i, sz]
        lib.hcCudaGemmPlan.argtypes = [ctypes.POINTER(_GemmArgs), i, ctypes.POINTER(_PlanInfo)]
        lib.hcCudaGemm.argtypes = [vp, ctypes.POINTER(_GemmArgs)]
        lib.hcCudaGemmHost.argtypes = [vp, ctypes.POINTER(_GemmArgs)]
        lib.hcCudaGemmHostDeviceA.argtypes = [vp, ctypes.POINTER(_GemmArgs)]
        lib.hcCudaEventCreate.argtypes = [vp, pvp]
        lib.hcCudaEventDestroy.argtypes = [vp, vp]
        lib.hcCudaEventRecord.argtypes = [vp, vp]
        lib.hcCudaEventElapsedMs.argtypes = [vp, vp, vp, ctypes.POINTER(ctypes.c_float)]
        lib.hcCudaCommGetUniqueId.argtypes = [vp, sz]
        lib.hcCudaCommInitRank.argtypes = [vp, vp, sz, i, i]
        lib.hcCudaCommAllGather.argtypes = [vp, vp, vp, sz]
        lib.hcCudaCommDestroy.argtypes = [vp]
        lib.hcCudaSelfTestDeviceTimeout.argtypes = [vp, ctypes.c_int64]
        lib.hcCudaGemmPush.argtypes = [vp, ctypes.POINTER(_GemmArgs), ctypes.POINTER(ctypes.c_void_p), i]
        lib.hcCudaIpcExport.argtypes = [vp, vp, vp, sz]
        lib.hcCudaIpcOpen.argtypes = [vp, vp, sz, pvp]
        lib.hcCudaIpcClose.argtypes = [vp, vp]
        lib.hcCudaGemmSkinnyStatic.argtypes = [ctypes.POINTER(_GemmArgs), vp, i, ctypes.c_char_p, sz]
        lib.hcCudaMap.argtypes = [vp, ctypes.POINTER(_MapArgs)]
        lib.hcCudaMapHost.argtypes = [vp, ctypes.POINTER(_MapArgs)]
        lib.hcCudaSelfTestDeviceCheck.argtypes = [vp]
        lib.hcCudaPairwise.argtypes = [vp, ctypes.POINTER(_PairwiseArgs)]
        lib.hcCudaPairwiseHost.argtypes = [vp, ctypes.POINTER(_PairwiseArgs)]
        lib.hcCudaRowSum.argtypes = [vp, ctypes.POINTER(_RowSumArgs)]
        lib.hcCudaRowSumHost.argtypes = [vp, ctypes.POINTER(_RowSumArgs)]
        for name in EXPORTS:
            getattr(lib, name)  # AttributeError here means a stale or foreign library
        _LIB = lib
    return _LIB


def library_is_checked() -> bool:
    """Whether the loaded library is the checked build (in-kernel index checks; `HC_CUDA_LIB` selects it)."""
    return bool(library().hcCudaBuildFlags() & 1)


def _raise(status: int, ctx_handle: Any = None) -> None:
    lib = library()
    name = lib.hcCudaStatusString(status).decode()
    detail = lib.hcCudaContextLastError(ctx_handle).decode(errors="replace")
    raise DeviceError(status, name, detail)


def device_count() -> int:
    count = ctypes.c_int(0)
    status = library().hcCudaGetDeviceCount(ctypes.byref(count))
    if status:
        _raise(status)
    return count.value


def dtype_code(dtype: Any) -> int:
    name = dtype if isinstance(dtype, str) else np.dtype(dtype).name
    codes = {"float16": F16, "bfloat16": BF16, "float8_e4m3fn": F8E4M3, "float8_e5m2": F8E5M2}
    if name not in codes:
        raise ValueError(f"the CUDA backend multiplies {sorted(codes)} matrices, got {name}")
    return codes[name]


C_F32, C_F16, C_BF16 = 0, 1, 2  # element type of C (HcCudaCType)


def c_dtype_code(dtype: Any) -> int:
    name = dtype if isinstance(dtype, str) else np.dtype(dtype).name
    codes = {"float32": C_F32, "float16": C_F16, "bfloat16": C_BF16}
    if name not in codes:
        raise ValueError(f"C must be float32, float16 or bfloat16, got {name}")
    return codes[name]


class GemmPlan:
    """What one GEMM call does on the device (`hcCudaGemmPlan`)."""

    def __init__(self, info: _PlanInfo) -> None:
        self.variant = VARIANT_NAMES.get(info.variant, str(info.variant))
        self.tiles_m = info.tiles_m
        self.tiles_n = info.tiles_n
        self.splits = info.splits
        self.grid = info.grid
        self.repack_a = bool(info.repack_a)
        self.repack_b = bool(info.repack_b)
        self.kernel_launches = info.kernel_launches
        self.scratch_bytes = info.scratch_bytes
        self.first_split_tile = info.first_split_tile
        self.ring_stages = info.ring_stages  # skinny: shared-memory ring depth of this grid; else 0
        self.cluster_size = info.cluster_size  # dense, few tiles: CTAs per cluster sharing a tile; else 0
        self.tile_n = info.tile_n  # dense: columns of a tile (256, or 128 for small products); else 0

    def __repr__(self) -> str:
        splits = f"{self.splits}" + (f" from tile {self.first_split_tile}" if self.first_split_tile else "")
        return (f"GemmPlan({self.variant}, tiles={self.tiles_m}x{self.tiles_n}, splits={splits}, "
                f"grid={self.grid}, repack=({self.repack_a}, {self.repack_b}), "
                f"launches={self.kernel_launches}, scratch={self.scratch_bytes})")


B_KN, B_NK = 0, 1  # B stored [k, n] (default) or transposed, [n, k]


def _gemm_args(m: int, n: int, k: int, dtype: Any, a: int | None, lda: int, b: int | None, ldb: int,
               c: int | None, ldc: int, variant: int, b_transposed: bool = False, accumulate: bool = False,
               epilogue: Sequence[tuple] = (), bias: int | None = None, c_dtype: Any = "float32") -> _GemmArgs:
    epilogue = tuple(epilogue)
    if len(epilogue) > MAX_EPILOGUE_OPS:
        raise ValueError(f"at most {MAX_EPILOGUE_OPS} fused element-wise operations are supported")
    kinds = (ctypes.c_int32 * 4)()
    values = (ctypes.c_float * 4)()
    for i, op in enumerate(epilogue):
        name = op[0]
        if name not in EPILOGUE_KINDS:
            raise ValueError(f"unknown fused operation {name!r}; expected one of {sorted(EPILOGUE_KINDS)}")
        kinds[i] = EPILOGUE_KINDS[name]
        values[i] = float(op[1]) if len(op) > 1 else 0.0
    return _GemmArgs(m, n, k, dtype_code(dtype), variant, a, lda, b, ldb, c, ldc,
                     B_NK if b_transposed else B_KN, 1 if accumulate else 0, len(epilogue), kinds, values,
                     c_dtype_code(c_dtype), bias)


def plan_gemm(m: int, n: int, k: int, dtype: Any, *, a: int = 0x1000, lda: int | None = None,
              b: int = 0x40000000, ldb: int | None = None, c: int = 0x80000000,
              ldc: int | None = None, variant: int = VARIANT_AUTO, sm_count: int = 148,
              b_transposed: bool = False, accumulate: bool = False, epilogue: Sequence[tuple] = (),
              bias: int | None = 0xC0000000, c_dtype: Any = "float32") -> GemmPlan:
    """Validates a problem and returns its launch plan without touching a device.

    The pointer arguments are plain integers that are only inspected (null, alignment,
    overlap); the defaults are well-aligned, far-apart placeholders.
    """
    args = _gemm_args(m, n, k, dtype, a, k if lda is None else lda, b,
                      (k if b_transposed else n) if ldb is None else ldb, c, n if ldc is None else ldc, variant,
                      b_transposed, accumulate, epilogue, bias, c_dtype)
    info = _PlanInfo()
    status = library().hcCudaGemmPlan(ctypes.byref(args), sm_count, ctypes.byref(info))
    if status:
        _raise(status)
    return GemmPlan(info)


class Context:
    """One device: its stream, scratch memory and (optionally) its NCCL communicator."""

    def __init__(self, device: int = 0) -> None:
        self._lib = library()
        handle = ctypes.c_void_p()
        status = self._lib.hcCudaContextCreate(device, ctypes.byref(handle))
        if status:
            _raise(status)
        self._handle = handle
        self.device = device
        info = _DeviceInfo()
        self._check(self._lib.hcCudaContextGetDeviceInfo(self._handle, ctypes.byref(info)))
        self.name = info.name.decode()
        self.sm_count = info.sm_count
        self.compute_capability = (info.cc_major, info.cc_minor)
        self.total_memory_bytes = info.total_memory_bytes
        self.l2_bytes = info.l2_bytes
        self.sm_clock_khz = info.sm_clock_khz

    # -- plumbing -----------------------------------------------------------------------
    def _check(self, status: int) -> None:
        if status:
            _raise(status, self._handle)

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.hcCudaContextDestroy(self._handle)
            self._handle = None

    def __del__(self) -> None:  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self) -> "Context":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    def synchronize(self) -> None:
        self._check(self._lib.hcCudaContextSynchronize(self._handle))

    # -- memory -------------------------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        ptr = ctypes.c_void_p()
        self._check(self._lib.hcCudaMalloc(self._handle, nbytes, ctypes.byref(ptr)))
        return ptr.value or 0

    def free(self, ptr: int) -> None:
        if ptr:
            self._check(self._lib.hcCudaFree(self._handle, ptr))

    def memset(self, ptr: int, byte_value: int, nbytes: int) -> None:
        self._check(self._lib.hcCudaMemset(self._handle, ptr, byte_value, nbytes))

    def empty(self, shape: tuple[int, ...], dtype: Any) -> "DeviceBuffer":
        return DeviceBuffer(self, shape, dtype)

    def to_device(self, array: np.ndarray) -> "DeviceBuffer":
        buf = DeviceBuffer(self, array.shape, array.dtype)
        buf.copy_from_host(array)
        return buf

    # -- the hot path -------------------------------------------------------------------
    def gemm(self, a: "DeviceBuffer", b: "DeviceBuffer", c: "DeviceBuffer", *,
             variant: int = VARIANT_AUTO, push: "list[DeviceBuffer] | None" = None,
             b_transposed: bool = False, accumulate: bool = False, epilogue: Sequence[tuple] = (),
             bias: "DeviceBuffer | None" = None) -> None:
        """Enqueues C = A @ B on device buffers (asynchronous; see `synchronize`).

        `c` is float32, or float16 / bfloat16 (the float32 result rounded to nearest even).
        `b_transposed`: `b` holds B transposed, shape (n, k).
        `accumulate`: C = C + A @ B (the previous contents of C start the sums).
        `epilogue`: element-wise operations applied in order before the store, e.g.
        `(("scale", 0.5), ("bias",), ("max", 0.0))`; `bias` is the float32 vector of n values
        that ("bias",) adds to every row.
        `push`: up to 7 more buffers shaped and pitched like `c` (typically windows of peer
        GPUs' copies of C, see `ipc_open`) that receive every tile of C as well.
        """
        m, k = a.shape
        n = b.shape[0] if b_transposed else b.shape[1]
        if bias is not None and (bias.dtype != np.float32 or bias.shape != (n,)):
            raise ValueError("bias must be a float32 buffer of n values")
        args = _gemm_args(m, n, k, a.dtype, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, variant, b_transposed,
                          accumulate, epilogue, None if bias is None else bias.ptr, c.dtype)
        if not push:
            self._check(self._lib.hcCudaGemm(self._handle, ctypes.byref(args)))
            return
        for target in push:
            if target.shape != c.shape or target.ld != c.ld or target.dtype != c.dtype:
                raise ValueError("push targets must have the shape, pitch and dtype of c")
        pointers = (ctypes.c_void_p * len(push))(*[t.ptr for t in push])
        self._check(self._lib.hcCudaGemmPush(self._handle, ctypes.byref(args), pointers, len(push)))

    def bind_gemm(self, a: "DeviceBuffer", b: "DeviceBuffer", c: "DeviceBuffer", *,
                  variant: int = VARIANT_AUTO, b_transposed: bool = False, accumulate: bool = False,
                  epilogue: Sequence[tuple] = (), bias: "DeviceBuffer | None" = None) -> "BoundGemm":
        """The same call as `gemm` with its arguments marshalled once: `launch()` on the result only
        crosses the C ABI, for loops in which the Python side of `gemm` (a few microseconds per call)
        would otherwise pace the GPU. The buffers must stay allocated while it is used."""
        m, k = a.shape
        n = b.shape[0] if b_transposed else b.shape[1]
        if bias is not None and (bias.dtype != np.float32 or bias.shape != (n,)):
            raise ValueError("bias must be a float32 buffer of n values")
        args = _gemm_args(m, n, k, a.dtype, a.ptr, a.ld, b.ptr, b.ld, c.ptr, c.ld, variant, b_transposed,
                          accumulate, epilogue, None if bias is None else bias.ptr, c.dtype)
        return BoundGemm(self, args, (a, b, c, bias))

    # -- sharing device memory between the processes of one node ----------------------------
    def ipc_export(self, buf: "DeviceBuffer") -> bytes:
        """Handle (64 bytes) of the allocation behind `buf`, for `ipc_open` in another process."""
        handle = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
        self._check(self._lib.hcCudaIpcExport(self._handle, buf.ptr, handle, IPC_HANDLE_BYTES))
        return handle.raw

    def ipc_open(self, handle: bytes) -> int:
        """Maps another process's allocation into this one; returns its device address here."""
        raw = ctypes.create_string_buffer(bytes(handle), IPC_HANDLE_BYTES)
        ptr = ctypes.c_void_p()
        self._check(self._lib.hcCudaIpcOpen(self._handle, raw, IPC_HANDLE_BYTES, ctypes.byref(ptr)))
        return ptr.value or 0

    def ipc_close(self, ptr: int) -> None:
        if ptr:
            self._check(self._lib.hcCudaIpcClose(self._handle, ptr))

    def gemm_host_device_a(self, a: "DeviceBuffer", b: np.ndarray, c: np.ndarray, *,
                           b_transposed: bool = False, epilogue: Sequence[tuple] = (),
                           bias: np.ndarray | None = None) -> None:
        """C = A @ B with A resident on the device and B, C host arrays (row-major): B travels in
        column panels while earlier panels are multiplied and their columns of C travel back."""
        m, k = a.shape
        n = b.shape[0] if b_transposed else b.shape[1]
        b_rows, b_cols = b.shape
        args = _gemm_args(m, n, k, a.dtype, a.ptr, a.ld, b.ctypes.data,
                          b.strides[0] // b.itemsize if b_rows > 1 else max(b_cols, 1), c.ctypes.data,
                          c.strides[0] // c.itemsize if m > 1 else max(n, 1), VARIANT_AUTO, b_transposed, False,
                          epilogue, None if bias is None else bias.ctypes.data, c.dtype)
        self._check(self._lib.hcCudaGemmHostDeviceA(self._handle, ctypes.byref(args)))

    def map(self, x: "DeviceBuffer", out: "DeviceBuffer", ops: Sequence[tuple], *,
            other: "DeviceBuffer | None" = None) -> None:
        """Enqueues out[i] = ops(x[i] [, other[i]]) on one-dimensional float32 device buffers
        (asynchronous). `ops` in order, e.g. `(("scale", 2.0), ("add_other",), ("max", 0.0))`."""
        for buf in (x, out) + (() if other is None else (other,)):
            if buf.dtype != np.float32 or buf.ndim != 1 or buf.shape != x.shape:
                raise ValueError("map() takes one-dimensional float32 buffers of one length")
        args = _map_args(x.shape[0], x.ptr, None if other is None else other.ptr, out.ptr, ops)
        self._check(self._lib.hcCudaMap(self._handle, ctypes.byref(args)))

    def map_host(self, x: np.ndarray, out: np.ndarray, ops: Sequence[tuple], *,
                 other: np.ndarray | None = None) -> None:
        """The same on contiguous one-dimensional float32 host arrays: copies in, runs, copies `out`
        back in place; returns when `out` is complete."""
        for arr in (x, out) + (() if other is None else (other,)):
            if arr.dtype != np.float32 or arr.ndim != 1 or arr.shape != x.shape or not arr.flags.c_contiguous:
                raise ValueError("map_host() takes contiguous one-dimensional float32 arrays of one length")
        args = _map_args(x.shape[0], x.ctypes.data, None if other is None else other.ctypes.data,
                         out.ctypes.data, ops)
        self._check(self._lib.hcCudaMapHost(self._handle, ctypes.byref(args)))

    def pairwise(self, x1: "DeviceBuffer", x2: "DeviceBuffer", out: "DeviceBuffer", *, take_sqrt: bool = True) -> None:
        """Enqueues out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h])**2) (the sum itself with `take_sqrt`
        off) on float32 device matrices x1 (w1, h), x2 (w2, h), out (w1, w2): the pairwise kernel
        class, bit-identical to the reference simulator (asynchronous; see `synchronize`)."""
        for buf in (x1, x2, out):
            if buf.dtype != np.float32 or len(buf.shape) != 2:
                raise ValueError("pairwise() takes two-dimensional float32 device buffers")
        (w1, h), (w2, h2) = x1.shape, x2.shape
        if h != h2 or out.shape != (w1, w2):
            raise ValueError(f"pairwise(): shapes {x1.shape}, {x2.shape} -> {out.shape} do not fit")
        args = _PairwiseArgs(w1, w2, h, x1.ptr, x1.ld, x2.ptr, x2.ld, out.ptr, out.ld,
                             PAIRWISE_EUCLIDEAN if take_sqrt else PAIRWISE_SQUARED)
        self._check(self._lib.hcCudaPairwise(self._handle, ctypes.byref(args)))

    def pairwise_host(self, x1: np.ndarray, x2: np.ndarray, out: np.ndarray, *, take_sqrt: bool = True) -> None:
        """The same on row-major float32 host matrices (rows may be padded): copies in, runs, copies
        `out` back in place; returns when `out` is complete."""
        for arr in (x1, x2, out):
            if arr.dtype != np.float32 or arr.ndim != 2 or (arr.shape[1] > 1 and arr.strides[1] != 4):
                raise ValueError("pairwise_host() takes row-major two-dimensional float32 arrays")
        (w1, h), (w2, h2) = x1.shape, x2.shape
        if h != h2 or out.shape != (w1, w2):
            raise ValueError(f"pairwise_host(): shapes {x1.shape}, {x2.shape} -> {out.shape} do not fit")

        def pitch(arr: np.ndarray) -> int:
            return arr.strides[0] // 4 if arr.shape[0] > 1 else max(arr.shape[1], 1)

        args = _PairwiseArgs(w1, w2, h, x1.ctypes.data, pitch(x1), x2.ctypes.data, pitch(x2), out.ctypes.data,
                             pitch(out), PAIRWISE_EUCLIDEAN if take_sqrt else PAIRWISE_SQUARED)
        self._check(self._lib.hcCudaPairwiseHost(self._handle, ctypes.byref(args)))

    def row_sum(self, x: "DeviceBuffer", out: "DeviceBuffer", *, square: bool = False, take_sqrt: bool = False) -> None:
        """Enqueues out[i] = sum_h x[i, h] on a float32 device matrix x (w, h) and vector out (w,),
        with every value squared first (`square`) and the square root of the sum stored (`take_sqrt`)
        if asked: the row-sum kernel class, bit-identical to the reference simulator (asynchronous;
        see `synchronize`)."""
        if x.dtype != np.float32 or out.dtype != np.float32 or len(x.shape) != 2 or len(out.shape) != 1:
            raise ValueError("row_sum() takes a two-dimensional and a one-dimensional float32 device buffer")
        w, h = x.shape
        if out.shape != (w,):
            raise ValueError(f"row_sum(): shapes {x.shape} -> {out.shape} do not fit")
        flags = (ROW_SUM_SQUARE if square else 0) | (ROW_SUM_SQRT if take_sqrt else 0)
        args = _RowSumArgs(w, h, x.ptr, x.ld, out.ptr, flags)
        self._check(self._lib.hcCudaRowSum(self._handle, ctypes.byref(args)))

    def row_sum_host(self, x: np.ndarray, out: np.ndarray, *, square: bool = False, take_sqrt: bool = False) -> None:
        """The same on a row-major float32 host matrix (rows may be padded) and a contiguous float32
        host vector: copies in, runs, copies `out` back in place; returns when `out` is complete."""
        if (x.dtype != np.float32 or x.ndim != 2 or (x.shape[1] > 1 and x.strides[1] != 4) or out.dtype != np.float32
                or out.ndim != 1 or (out.shape[0] > 1 and out.strides[0] != 4)):
            raise ValueError("row_sum_host() takes a row-major float32 matrix and a contiguous float32 vector")
        w, h = x.shape
        if out.shape != (w,):
            raise ValueError(f"row_sum_host(): shapes {x.shape} -> {out.shape} do not fit")
        pitch = x.strides[0] // 4 if w > 1 else max(h, 1)
        flags = (ROW_SUM_SQUARE if square else 0) | (ROW_SUM_SQRT if take_sqrt else 0)
        args = _RowSumArgs(w, h, x.ctypes.data, pitch, out.ctypes.data, flags)
        self._check(self._lib.hcCudaRowSumHost(self._handle, ctypes.byref(args)))

    def gemm_host(self, a: np.ndarray, b: np.ndarray, c: np.ndarray, *,
                  variant: int = VARIANT_AUTO, b_transposed: bool = False, accumulate: bool = False,
                  epilogue: Sequence[tuple] = (), bias: np.ndarray | None = None) -> None:
        """C = A @ B on host arrays: copies in, multiplies on the GPU, copies C back in place.
        With `b_transposed`, `b` holds B transposed, shape (n, k). `accumulate`, `epilogue` and
        `bias` (a contiguous float32 host vector) as for `gemm`."""
        m, k = a.shape
        n = b.shape[0] if b_transposed else b.shape[1]
        b_rows, b_cols = b.shape
        args = _gemm_args(m, n, k, a.dtype, a.ctypes.data, a.strides[0] // a.itemsize if m > 1 else max(k, 1),
                          b.ctypes.data, b.strides[0] // b.itemsize if b_rows > 1 else max(b_cols, 1),
                          c.ctypes.data, c.strides[0] // c.itemsize if m > 1 else max(n, 1), variant,
                          b_transposed, accumulate, epilogue, None if bias is None else bias.ctypes.data, c.dtype)
        if bias is not None and (bias.dtype != np.float32 or bias.shape != (n,) or not bias.flags.c_contiguous):
            raise ValueError("bias must be a contiguous float32 vector of n values")
        self._check(self._lib.hcCudaGemmHost(self._handle, ctypes.byref(args)))

    def selftest_device_check(self) -> None:
        """Checked build only: enqueues a kernel whose index check fails (the access is skipped); the
        next `synchronize` raises DeviceError (HC_CUDA_ERR_DEVICE_CHECK) and the context stays usable."""
        self._check(self._lib.hcCudaSelfTestDeviceCheck(self._handle))

    def selftest_device_timeout(self, budget_cycles: int = 2_000_000) -> None:
        """Enqueues a kernel whose bounded wait runs out; the next `synchronize` raises
        DeviceError (HC_CUDA_ERR_DEVICE_TIMEOUT) and the context stays usable."""
        self._check(self._lib.hcCudaSelfTestDeviceTimeout(self._handle, budget_cycles))

    def plan(self, m: int, n: int, k: int, dtype: Any, **kwargs: Any) -> GemmPlan:
        kwargs.setdefault("sm_count", self.sm_count)
        return plan_gemm(m, n, k, dtype, **kwargs)

    # -- timing -------------------------------------------------------------------------
    def event(self) -> "Event":
        return Event(self)

    # -- multi-GPU ----------------------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(COMM_ID_BYTES)
        status = library().hcCudaCommGetUniqueId(buf, COMM_ID_BYTES)
        if status:
            _raise(status)
        return buf.raw

    def comm_init(self, unique_id: bytes, world_size: int, rank: int) -> None:
        buf = ctypes.create_string_buffer(bytes(unique_id), COMM_ID_BYTES)
        self._check(self._lib.hcCudaCommInitRank(self._handle, buf, COMM_ID_BYTES, world_size, rank))

    def all_gather(self, send: "DeviceBuffer", recv: "DeviceBuffer") -> None:
        """Asynchronous all-gather of whole buffers; `recv` holds world_size copies of `send`."""
        self._check(self._lib.hcCudaCommAllGather(self._handle, send.ptr, recv.ptr, send.nbytes))

    def comm_destroy(self) -> None:
        self._check(self._lib.hcCudaCommDestroy(self._handle))


class Event:
    def __init__(self, ctx: Context) -> None:
        self._ctx = ctx
        handle = ctypes.c_void_p()
        ctx._check(ctx._lib.hcCudaEventCreate(ctx._handle, ctypes.byref(handle)))
        self._handle = handle

    def record(self) -> None:
        self._ctx._check(self._ctx._lib.hcCudaEventRecord(self._ctx._handle, self._handle))

    def elapsed_ms_since(self, start: "Event") -> float:
        """Waits for this event, then returns the device time since `start` in milliseconds."""
        ms = ctypes.c_float()
        self._ctx._check(self._ctx._lib.hcCudaEventElapsedMs(self._ctx._handle, start._handle,
                                                             self._handle, ctypes.byref(ms)))
        return ms.value

    def close(self) -> None:
        if self._handle and self._ctx._handle:
            self._ctx._lib.hcCudaEventDestroy(self._ctx._handle, self._handle)
        self._handle = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


class BoundGemm:
    """A GEMM on device buffers with its C-ABI arguments already built (`Context.bind_gemm`)."""

    __slots__ = ("_ctx", "_args", "_ref", "_buffers", "_call", "_handle")

    def __init__(self, ctx: Context, args: _GemmArgs, buffers: tuple) -> None:
        self._ctx = ctx
        self._args = args
        self._ref = ctypes.byref(args)
        self._buffers = buffers  # kept alive with the call
        self._call = ctx._lib.hcCudaGemm
        self._handle = ctx._handle

    def launch(self) -> None:
        """Enqueues the product (asynchronous, like `Context.gemm`)."""
        status = self._call(self._handle, self._ref)
        if status:
            self._ctx._check(status)


class DeviceBuffer:
    """A row-major matrix (or vector) in device memory. `ld` is the row pitch in elements."""

    def __init__(self, ctx: Context, shape: tuple[int, ...], dtype: Any, *, ld: int | None = None) -> None:
        self.ctx = ctx
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.ndim = len(self.shape)
        cols = self.shape[-1] if self.shape else 1
        self.ld = int(cols if ld is None else ld)
        if self.ld < cols:
            raise ValueError("ld must be at least the number of columns")
        rows = int(np.prod(self.shape[:-1])) if self.ndim > 1 else 1
        self._rows = rows
        self.nbytes = rows * self.ld * self.dtype.itemsize
        self.ptr = ctx.malloc(self.nbytes) if self.nbytes else 0
        self._owned = True

    @classmethod
    def wrap(cls, ctx: Context, ptr: int, shape: tuple[int, ...], dtype: Any, *, ld: int | None = None) -> "DeviceBuffer":
        """A buffer object over device memory it does not own (a window of another buffer, or
        memory opened with `Context.ipc_open`); `free` and garbage collection leave it alone."""
        self = cls.__new__(cls)
        self.ctx = ctx
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.ndim = len(self.shape)
        cols = self.shape[-1] if self.shape else 1
        self.ld = int(cols if ld is None else ld)
        self._rows = int(np.prod(self.shape[:-1])) if self.ndim > 1 else 1
        self.nbytes = self._rows * self.ld * self.dtype.itemsize
        self.ptr = int(ptr)
        self._owned = False
        return self

    def window(self, row0: int, row1: int, col0: int, col1: int) -> "DeviceBuffer":
        """Non-owning view of rows [row0, row1), columns [col0, col1) of a matrix."""
        if self.ndim != 2 or not (0 <= row0 <= row1 <= self.shape[0] and 0 <= col0 <= col1 <= self.shape[1]):
            raise ValueError("window out of range")
        offset = (row0 * self.ld + col0) * self.dtype.itemsize
        return DeviceBuffer.wrap(self.ctx, self.ptr + offset, (row1 - row0, col1 - col0), self.dtype, ld=self.ld)

    def copy_from_host(self, array: np.ndarray) -> None:
        if tuple(array.shape) != self.shape or array.dtype != self.dtype:
            raise ValueError("host array does not match the device buffer")
        if not self.nbytes:
            return
        src = np.ascontiguousarray(array)
        width = self.shape[-1] * self.dtype.itemsize
        self.ctx._check(self.ctx._lib.hcCudaMemcpy2DHtoD(
            self.ctx._handle, self.ptr, self.ld * self.dtype.itemsize, src.ctypes.data, width, width,
            self._rows))

    def copy_from_host_columns(self, array: np.ndarray, col_begin: int, col_end: int) -> None:
        """Fills the buffer from columns [col_begin, col_end) of a wider row-major host matrix."""
        if array.ndim != 2 or array.dtype != self.dtype or self.shape != (array.shape[0], col_end - col_begin):
            raise ValueError("host slab does not match the device buffer")
        if not array.flags.c_contiguous:
            array = np.ascontiguousarray(array)
        item = self.dtype.itemsize
        self.ctx._check(self.ctx._lib.hcCudaMemcpy2DHtoD(
            self.ctx._handle, self.ptr, self.ld * item, array.ctypes.data + col_begin * item,
            array.shape[1] * item, (col_end - col_begin) * item, array.shape[0]))

    def to_numpy(self, out: np.ndarray | None = None) -> np.ndarray:
        if out is None:
            out = np.empty(self.shape, self.dtype)
        if tuple(out.shape) != self.shape or out.dtype != self.dtype or not out.flags.c_contiguous:
            raise ValueError("output array must be C-contiguous and match the device buffer")
        if self.nbytes:
            width = self.shape[-1] * self.dtype.itemsize
            self.ctx._check(self.ctx._lib.hcCudaMemcpy2DDtoH(
                self.ctx._handle, out.ctypes.data, width, self.ptr, self.ld * self.dtype.itemsize,
                width, self._rows))
        return out

    def fill_bytes(self, byte_value: int) -> None:
        if self.nbytes:
            self.ctx.memset(self.ptr, byte_value, self.nbytes)

    def free(self) -> None:
        if self.ptr and getattr(self, "_owned", True) and self.ctx._handle:
            self.ctx.free(self.ptr)
        self.ptr = 0

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.free()
        except Exception:
            pass

    def __repr__(self) -> str:
        return f"DeviceBuffer(shape={self.shape}, dtype={self.dtype.name}, ld={self.ld}, device={self.ctx.device})"


class _PinnedOwner:
    """Keeps a page-locked allocation alive for the NumPy arrays that view it."""

    def __init__(self, nbytes: int) -> None:
        ptr = ctypes.c_void_p()
        status = library().hcCudaHostAlloc(nbytes, ctypes.byref(ptr))
        if status:
            _raise(status)
        self.ptr = ptr.value
        self.nbytes = nbytes
        self.__array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3,
        }

    def __del__(self) -> None:  # pragma: no cover
        try:
            if self.ptr:
                library().hcCudaHostFree(self.ptr)
        except Exception:
            pass
        self.ptr = None


def pinned_empty(shape: tuple[int, ...], dtype: Any) -> np.ndarray:
    """NumPy array in page-locked host memory (needs a CUDA driver)."""
    dtype = np.dtype(dtype)
    nbytes = int(np.prod(shape)) * dtype.itemsize
    if nbytes == 0:
        return np.empty(shape, dtype)
    owner = _PinnedOwner(nbytes)
    return np.asarray(owner).view(dtype).reshape(shape)


_DEFAULT: dict[int, Context] = {}
_DEFAULT_LOCK = threading.Lock()


def default_context(device: int | None = None) -> Context:
    """Process-wide context of a device; `device=None` means `$HC_CUDA_DEVICE` or 0."""
    if device is None:
        device = int(os.environ.get("HC_CUDA_DEVICE", "0"))
    with _DEFAULT_LOCK:
        ctx = _DEFAULT.get(device)
        if ctx is None or not ctx._handle:
            ctx = _DEFAULT[device] = Context(device)
        return ctx
