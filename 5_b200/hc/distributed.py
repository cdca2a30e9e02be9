"""N-sharding of the matmul across the GPUs of one box: one process per GPU.

The product splits by columns with no exchange: rank r owns the column slab
`B[:, lo:hi]` and writes `C[:, lo:hi]`; A is replicated. A slab is just a matmul with a
smaller N, so each rank launches the same compiled handle on its own buffers. Gathering C on
every rank is optional and comes in two forms: an NCCL all-gather of the finished slabs (C
arrives slab-major, `[rank][M][slab columns]`; `assemble_row_major` turns that into a row-major
matrix on the host), or `PushedMatmul`, where the GEMM's own epilogue stores each tile into all
ranks' row-major C over NVLink while the rest of the product is still running. The reference has no multi-device notion at all;
this module is the whole of it here.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import numpy as np

__all__ = ["ColumnSlab", "PushedMatmul", "ShardedMatmul", "assemble_row_major", "column_slab", "init_communicator",
           "row_shard"]


@dataclass(frozen=True)
class ColumnSlab:
    rank: int
    world_size: int
    begin: int
    end: int

    @property
    def width(self) -> int:
        return self.end - self.begin


def column_slab(n: int, world_size: int, rank: int, *, align: int = 1) -> ColumnSlab:
    """Columns [begin, end) of rank `rank` when `n` columns are split over `world_size`.

    Slabs are contiguous and cover [0, n) exactly once. The columns are dealt out in blocks
    of `align` (the last block may be partial), so boundaries are multiples of `align` (use
    the CTA tile width, 256, to keep every slab tile-aligned) and slabs differ by at most one
    block. Ranks past the last column get an empty slab.
    """
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} is not in [0, {world_size})")
    if n < 0 or align < 1:
        raise ValueError("n must be non-negative and align positive")
    blocks = -(-n // align)
    base, extra = divmod(blocks, world_size)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    begin = min(first * align, n)
    end = min((first + count) * align, n)
    return ColumnSlab(rank, world_size, begin, end)


def row_shard(m: int, world_size: int, rank: int) -> ColumnSlab:
    """Rows [begin, end) of A that rank `rank` uploads from the host when the ranks share that work
    (`ShardedMatmul.host_product`): equal, contiguous shares when `world_size` divides `m`."""
    return column_slab(m, world_size, rank, align=1)


def init_communicator(ctx: Any, world_size: int, rank: int,
                      broadcast: Callable[[bytes | None], bytes]) -> None:
    """Joins `ctx` to a NCCL communicator of `world_size` ranks.

    `broadcast(payload)` must return rank 0's payload on every rank (rank 0 passes the id it
    created, the others pass None); any host channel will do, e.g. a `torch.distributed`
    object broadcast or a file.
    """
    payload = ctx.comm_unique_id() if rank == 0 else None
    unique_id = broadcast(payload)
    if not isinstance(unique_id, (bytes, bytearray)) or len(unique_id) == 0:
        raise RuntimeError("broadcast() did not deliver rank 0's communicator id")
    ctx.comm_init(bytes(unique_id), world_size, rank)


class ShardedMatmul:
    """Per-rank driver of the N-sharded product."""

    def __init__(self, handle: Any, ctx: Any, n: int, world_size: int, rank: int, *, align: int = 256) -> None:
        self.handle = handle
        self.ctx = ctx
        self.n = n
        self.slab = column_slab(n, world_size, rank, align=align)
        self.world_size = world_size
        self.rank = rank
        self._device_a: Any = None  # A gathered on the device, kept between host_product calls

    def upload(self, a: np.ndarray, b: np.ndarray) -> tuple[Any, Any, Any]:
        """Device copies of A (whole), this rank's slab of B, and an empty slab of C."""
        if b.shape[1] != self.n:
            raise ValueError(f"B has {b.shape[1]} columns, the sharding was built for {self.n}")
        da = self.ctx.to_device(a)
        db = self.ctx.empty((b.shape[0], self.slab.width), b.dtype)
        db.copy_from_host_columns(b, self.slab.begin, self.slab.end)
        dc = self.ctx.empty((a.shape[0], self.slab.width), np.float32)
        return da, db, dc

    def run(self, da: Any, db_slab: Any, dc_slab: Any) -> None:
        """C slab = A @ B slab (asynchronous on the rank's stream)."""
        if self.slab.width:
            self.ctx.gemm(da, db_slab, dc_slab)

    def host_product(self, a: np.ndarray, b_slab: np.ndarray, c_slab: np.ndarray) -> None:
        """C slab = A @ B slab from host arrays, without sending A over PCIe once per rank.

        `a` is the whole row-major A as this rank's host sees it; the rank uploads only its share
        of the rows (`row_shard`), the ranks exchange the shares over NVLink with one in-place
        all-gather (the context must have joined the communicator, `init_communicator`), and the
        gathered A is multiplied with the rank's own slab of B, which travels in column panels
        while earlier panels are multiplied and their columns of C travel back
        (`hcCudaGemmHostDeviceA`). Collective: every rank calls it for every product. Returns when
        this rank's `c_slab` is complete. Page-locked arrays make the copies asynchronous."""
        m, k = a.shape
        if b_slab.shape != (k, self.slab.width) or c_slab.shape != (m, self.slab.width):
            raise ValueError("b_slab / c_slab do not match this rank's column slab")
        if self._device_a is None or self._device_a.shape != (m, k) or self._device_a.dtype != a.dtype:
            if self._device_a is not None:
                self._device_a.free()
            self._device_a = self.ctx.empty((m, k), a.dtype)
        da = self._device_a
        share = row_shard(m, self.world_size, self.rank)
        if m % self.world_size == 0 and self.world_size > 1:
            mine = da.window(share.begin, share.end, 0, k)
            mine.copy_from_host(a[share.begin : share.end])
            self.ctx.all_gather(mine, da)  # in place: the send buffer is this rank's part of `da`
        else:
            da.copy_from_host(a)  # shares of unequal size: every rank sends the whole of A
        if self.slab.width:
            self.ctx.gemm_host_device_a(da, b_slab, c_slab)
        else:
            self.ctx.synchronize()

    def all_gather(self, dc_slab: Any, gathered: Any) -> None:
        """Gathers equal-width C slabs into `gathered`, shape (world_size, M, slab width)."""
        if self.n % self.world_size != 0 or self.slab.width * self.world_size != self.n:
            raise ValueError("all_gather needs equal slabs (n divisible by world_size * align)")
        self.ctx.all_gather(dc_slab, gathered)


class PushedMatmul:
    """The N-sharded product with the gather fused into the GEMM's epilogue.

    Every rank holds a full row-major C[M, N]. Rank r computes its column slab and its kernel
    stores each finished tile into the slab's window of *every* rank's C: locally, and over NVLink
    through pointers opened with CUDA IPC. Transfers overlap the remaining tiles' math, and the
    result is row-major everywhere (the NCCL all-gather yields slab-major C and runs after the
    product). Usage per rank: `setup` (collective), then `run` + `ctx.synchronize()` + a host
    barrier per product, `close` (collective) at the end.
    """

    def __init__(self, ctx: Any, m: int, n: int, world_size: int, rank: int, *, align: int = 256) -> None:
        if world_size - 1 > 7:
            raise ValueError("at most 8 ranks (7 push targets)")
        self.ctx = ctx
        self.m, self.n = m, n
        self.world_size, self.rank = world_size, rank
        self.slab = column_slab(n, world_size, rank, align=align)
        self.full_c: Any = None
        self._peer_ptrs: list[int] = []
        self._targets: list[Any] = []

    def setup(self, all_gather: Callable[[bytes], "list[bytes]"]) -> Any:
        """Allocates this rank's full C and maps the peers'. `all_gather(payload)` must return
        the payloads of all ranks in rank order (any host channel). Returns the full C."""
        import numpy as _np

        self.full_c = self.ctx.empty((self.m, self.n), _np.float32)
        handles = all_gather(self.ctx.ipc_export(self.full_c))
        if len(handles) != self.world_size:
            raise RuntimeError("all_gather() must return one handle per rank")
        for peer, handle in enumerate(handles):
            if peer == self.rank:
                continue
            ptr = self.ctx.ipc_open(handle)
            self._peer_ptrs.append(ptr)
            whole = type(self.full_c).wrap(self.ctx, ptr, (self.m, self.n), _np.float32)
            self._targets.append(whole.window(0, self.m, self.slab.begin, self.slab.end))
        return self.full_c

    def run(self, da: Any, db_slab: Any) -> None:
        """Enqueues the slab product; its tiles go to this rank's C and to all peers'."""
        if self.slab.width == 0:
            return
        local = self.full_c.window(0, self.m, self.slab.begin, self.slab.end)
        self.ctx.gemm(da, db_slab, local, push=self._targets)

    def close(self) -> None:
        """Unmaps the peers' memory. Call on every rank before any rank frees its C."""
        self.ctx.synchronize()
        for ptr in self._peer_ptrs:
            self.ctx.ipc_close(ptr)
        self._peer_ptrs, self._targets = [], []


def assemble_row_major(gathered: np.ndarray) -> np.ndarray:
    """(world, M, w) slab-major array -> (M, world * w) row-major matrix (host-side copy)."""
    world, m, width = gathered.shape
    return np.ascontiguousarray(gathered.transpose(1, 0, 2)).reshape(m, world * width)
