"""Host logic of the N-sharded product, on CPU: slab arithmetic, and a world-size-2 run over
`gloo` in which each rank handles its own column slab and the communicator id travels from
rank 0 by broadcast. The GEMM itself is stood in for by the CPU oracle (this file tests the
plumbing around it, not the kernels)."""

from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest

from conftest import PACKAGE, REPO
from hc.distributed import ShardedMatmul, assemble_row_major, column_slab, init_communicator


@pytest.mark.parametrize("n,world,align", [(32768, 8, 256), (32768, 1, 256), (3073, 4, 256), (1000, 8, 1),
                                           (5, 8, 1), (0, 2, 256), (4096, 3, 2048)])
def test_column_slabs_partition_the_columns(n: int, world: int, align: int) -> None:
    slabs = [column_slab(n, world, r, align=align) for r in range(world)]
    assert slabs[0].begin == 0 and slabs[-1].end == n
    for left, right in zip(slabs, slabs[1:]):
        assert left.end == right.begin
    for slab in slabs:
        assert 0 <= slab.begin <= slab.end <= n
        assert slab.begin % align == 0 or slab.begin == n
    widths = [s.width for s in slabs]
    assert sum(widths) == n
    full = [w for w in widths if w]
    assert not full or max(full) - min(full) < 2 * align


def test_column_slab_rejects_bad_ranks() -> None:
    with pytest.raises(ValueError):
        column_slab(10, 2, 2)
    with pytest.raises(ValueError):
        column_slab(10, 0, 0)
    with pytest.raises(ValueError):
        column_slab(-1, 2, 0)


def test_config5_slabs() -> None:
    for world in (1, 2, 4, 8):
        widths = {column_slab(32768, world, r, align=256).width for r in range(world)}
        assert widths == {32768 // world}


def test_assemble_row_major() -> None:
    gathered = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    full = assemble_row_major(gathered)
    assert full.shape == (3, 8)
    assert np.array_equal(full[:, :4], gathered[0]) and np.array_equal(full[:, 4:], gathered[1])


class _FakeContext:
    """Records what the communicator set-up asks of a context."""

    def __init__(self) -> None:
        self.joined = None

    def comm_unique_id(self) -> bytes:
        return bytes(range(128))

    def comm_init(self, unique_id: bytes, world_size: int, rank: int) -> None:
        self.joined = (unique_id, world_size, rank)


def test_init_communicator_needs_rank0_payload() -> None:
    ctx = _FakeContext()
    with pytest.raises(RuntimeError, match="did not deliver"):
        init_communicator(ctx, 2, 1, lambda payload: b"")
    init_communicator(ctx, 1, 0, lambda payload: payload)
    assert ctx.joined == (bytes(range(128)), 1, 0)


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    for entry in (str(REPO), str(PACKAGE)):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    import torch.distributed as dist

    import workloads
    from hc.distributed import column_slab, init_communicator
    from oracle import cpu_ref

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def broadcast(payload):
            box = [payload]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        ctx = _FakeContext()
        init_communicator(ctx, world, rank, broadcast)
        assert ctx.joined == (bytes(range(128)), world, rank)

        n, m, k = 4096, 48, 96
        slab = column_slab(n, world, rank, align=2048)
        a, b_slab = workloads.make_sharded_inputs(slab.begin, slab.end, m=m, k=k)
        c_slab = cpu_ref.matmul_k_ascending(a, b_slab, threads=1)
        np.save(os.path.join(out_dir, f"c_{rank}.npy"), c_slab)

        # host_product's plumbing on stand-in device memory: the rank uploads only its rows of A,
        # the in-place all-gather (here over gloo) completes A, the slab product follows.
        import torch

        from hc.distributed import ShardedMatmul, row_shard

        class Buffer:
            def __init__(self, array, row0=0):
                self.array, self.row0 = array, row0
                self.shape, self.dtype = array.shape, array.dtype

            def window(self, r0, r1, c0, c1):
                return Buffer(self.array[r0:r1, c0:c1], r0)

            def copy_from_host(self, host):
                self.array[...] = host

            def free(self):
                pass

        class Device(_FakeContext):
            uploads = 0

            def empty(self, shape, dtype):
                return Buffer(np.full(shape, 7, dtype))

            def all_gather(self, send, recv):
                assert send.array.base is not None and np.shares_memory(send.array, recv.array)  # in place
                Device.uploads += send.array.shape[0]
                parts = [torch.zeros(send.shape, dtype=torch.float16) for _ in range(world)]
                dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(send.array)))
                recv.array[...] = np.concatenate([p.numpy() for p in parts])

            def gemm_host_device_a(self, da, b, c):
                c[...] = cpu_ref.matmul_k_ascending(da.array, b, threads=1)

            def synchronize(self):
                pass

        device = Device()
        sharded = ShardedMatmul(None, device, n, world, rank, align=2048)
        out = np.zeros((m, slab.width), np.float32)
        scrambled = a.copy()
        share = row_shard(m, world, rank)
        scrambled[: share.begin] = 0  # rows of other ranks must come from them, not from this host copy
        scrambled[share.end :] = 0
        sharded.host_product(scrambled, b_slab, out)
        assert Device.uploads == m // world and np.array_equal(out, c_slab)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo_cover_the_product(tmp_path) -> None:
    import torch.multiprocessing as mp

    import workloads
    from oracle import cpu_ref

    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    slabs = np.stack([np.load(tmp_path / f"c_{r}.npy") for r in range(world)])
    a, b = workloads.make_sharded_inputs(0, 4096, m=48, k=96)
    assert np.array_equal(assemble_row_major(slabs), cpu_ref.matmul_k_ascending(a, b))


def test_sharded_matmul_checks_its_inputs() -> None:
    sharded = ShardedMatmul(handle=None, ctx=None, n=4096, world_size=2, rank=1, align=256)
    assert (sharded.slab.begin, sharded.slab.end) == (2048, 4096)
    with pytest.raises(ValueError, match="columns"):
        sharded.upload(np.zeros((4, 4), np.float16), np.zeros((4, 100), np.float16))
    with pytest.raises(ValueError, match="do not match this rank's column slab"):
        sharded.host_product(np.zeros((4, 8), np.float16), np.zeros((8, 100), np.float16), np.zeros((4, 100), np.float32))
    uneven = ShardedMatmul(handle=None, ctx=None, n=3073, world_size=2, rank=0, align=256)
    with pytest.raises(ValueError, match="equal slabs"):
        uneven.all_gather(None, None)
