"""The N-sharded product on two GPUs of one box: one process per GPU, each computing its own
column slab through the C ABI, then an NCCL all-gather of the C slabs; and the same product with
the gather fused into the GEMM epilogue (tiles pushed to the peer over NVLink, CUDA IPC). Skipped on a box with
fewer than two GPUs. NVLS is switched off so that a rank that dies never leaves NVLink multicast
state behind."""

from __future__ import annotations

import multiprocessing as mp
import os
import sys
import time
from pathlib import Path

import numpy as np
import pytest

from conftest import PACKAGE, REPO

pytestmark = pytest.mark.gpu

M, K, N = 512, 1024, 4096


def _rank_main(rank: int, world: int, out_dir: str) -> None:
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for entry in (str(REPO), str(PACKAGE)):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    import workloads
    from examples.b200_wmma_matmul import compiled_for
    from hc import cuda
    from hc.distributed import ShardedMatmul, init_communicator

    ctx = cuda.Context(rank)
    id_file = Path(out_dir) / "nccl_id.bin"

    def broadcast(payload):
        if payload is not None:
            tmp = id_file.with_suffix(".tmp")
            tmp.write_bytes(payload)
            tmp.rename(id_file)
            return payload
        deadline = time.time() + 60
        while not id_file.exists():
            if time.time() > deadline:
                raise TimeoutError("rank 0 never published the communicator id")
            time.sleep(0.05)
        return id_file.read_bytes()

    init_communicator(ctx, world, rank, broadcast)
    sharded = ShardedMatmul(compiled_for("float16"), ctx, N, world, rank, align=workloads.SHARDED_BLOCK_COLUMNS)
    a, b_slab = workloads.make_sharded_inputs(sharded.slab.begin, sharded.slab.end, m=M, k=K)
    da = ctx.to_device(a)
    db = ctx.to_device(b_slab)
    dc = ctx.empty((M, sharded.slab.width), np.float32)
    sharded.run(da, db, dc)
    gathered = ctx.empty((world, M, sharded.slab.width), np.float32)
    sharded.all_gather(dc, gathered)
    ctx.synchronize()
    np.save(Path(out_dir) / f"gathered_{rank}.npy", gathered.to_numpy())
    # The same slab from host arrays: each rank uploads half of A's rows, the halves are exchanged
    # over NVLink, B travels in column panels. A larger problem so that the panel pipeline runs.
    big_m, big_k = 2048, 1024
    big_a, big_b = workloads.make_sharded_inputs(sharded.slab.begin, sharded.slab.end, m=big_m, k=big_k)
    pa, pb = cuda.pinned_empty(big_a.shape, big_a.dtype), cuda.pinned_empty(big_b.shape, big_b.dtype)
    pa[...], pb[...] = big_a, big_b
    pc = cuda.pinned_empty((big_m, sharded.slab.width), np.float32)
    pc[...] = np.nan
    for _ in range(2):  # the gathered A is kept between calls
        sharded.host_product(pa, pb, pc)
    np.save(Path(out_dir) / f"host_slab_{rank}.npy", np.array(pc))
    dbig_a, dbig_b = ctx.to_device(big_a), ctx.to_device(big_b)
    dbig_c = ctx.empty((big_m, sharded.slab.width), np.float32)
    sharded.run(dbig_a, dbig_b, dbig_c)
    ctx.synchronize()
    np.save(Path(out_dir) / f"device_slab_{rank}.npy", dbig_c.to_numpy())
    ctx.comm_destroy()

    # The same product with the gather fused into the epilogue: tiles are pushed into every
    # rank's row-major C through CUDA IPC pointers.
    from hc.distributed import PushedMatmul

    def exchange(tag: str, payload: bytes) -> list[bytes]:
        mine = Path(out_dir) / f"{tag}_{rank}.bin"
        tmp = mine.with_suffix(".tmp")
        tmp.write_bytes(payload)
        tmp.rename(mine)
        out = []
        for r in range(world):
            path = Path(out_dir) / f"{tag}_{r}.bin"
            deadline = time.time() + 60
            while not path.exists():
                if time.time() > deadline:
                    raise TimeoutError(f"rank {r} never published {tag}")
                time.sleep(0.02)
            out.append(path.read_bytes())
        return out

    pushed = PushedMatmul(ctx, M, N, world, rank, align=workloads.SHARDED_BLOCK_COLUMNS)
    full_c = pushed.setup(lambda payload: exchange("ipc", payload))
    full_c.fill_bytes(0xFF)
    ctx.synchronize()
    exchange("ready", b"1")          # nobody pushes before every C has been poisoned
    pushed.run(da, db)
    ctx.synchronize()
    exchange("done", b"1")           # every rank's pushes have landed
    np.save(Path(out_dir) / f"pushed_{rank}.npy", full_c.to_numpy())
    exchange("saved", b"1")
    # The same push with the tiles handed to the TMA store engine once per destination.
    os.environ["HC_CUDA_PUSH_TMA"] = "1"
    full_c.fill_bytes(0xFF)
    ctx.synchronize()
    exchange("ready_tma", b"1")
    pushed.run(da, db)
    ctx.synchronize()
    exchange("done_tma", b"1")
    np.save(Path(out_dir) / f"pushed_tma_{rank}.npy", full_c.to_numpy())
    exchange("saved_tma", b"1")
    del os.environ["HC_CUDA_PUSH_TMA"]
    pushed.close()
    exchange("closed", b"1")         # no rank frees its C while a peer still maps it
    ctx.close()


def test_two_gpus_shard_and_gather(tmp_path) -> None:
    from hc import cuda

    if cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import workloads
    from hc.distributed import assemble_row_major
    from oracle import cpu_ref

    world = 2
    spawn = mp.get_context("spawn")
    procs = [spawn.Process(target=_rank_main, args=(r, world, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    a, b = workloads.make_sharded_inputs(0, N, m=M, k=K)
    expect = cpu_ref.matmul_k_ascending(a, b)
    bound = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
    first = None
    for r in range(world):
        full = assemble_row_major(np.load(tmp_path / f"gathered_{r}.npy"))
        assert (np.abs(full.astype(np.float64) - expect) <= 1e-2 * bound + 1e-30).all()
        assert workloads.check_against_float64(full, a, b)["ok"]
        first = full if first is None else first
        assert np.array_equal(full, first)  # every rank holds the same gathered C
        pushed = np.load(tmp_path / f"pushed_{r}.npy")
        assert np.array_equal(pushed, first)  # the fused push yields the same C, row-major, on every rank
        assert np.array_equal(np.load(tmp_path / f"pushed_tma_{r}.npy"), first)  # and so do TMA stores to the peers
        # The host-array path (rows of A shared out, gathered over NVLink) gives the bits of the
        # device-buffer product of the same slab.
        host_slab, device_slab = np.load(tmp_path / f"host_slab_{r}.npy"), np.load(tmp_path / f"device_slab_{r}.npy")
        assert np.isfinite(host_slab).all() and np.array_equal(host_slab, device_slab)
