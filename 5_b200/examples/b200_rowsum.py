"""Row-sum kernels in hc, launched on a B200.

    python 5_b200/examples/b200_rowsum.py [--w 262144 --h 512]

Kernels of the one-dimensional workgroup class that reduces the rows it loads -- the load of the
reference simulator's first test (tests/test_simulator.py:153-154) followed by the reduction of
its value type (hc/_sim_types.py:338-351):

  row_sums     out[i] = sum_h x[i, h], 4 rows per workgroup;
  row_norms    out[i] = sqrt(sum_h x[i, h]**2), 16 rows per workgroup, written with temporaries;
  row_energy   out[i] = sum_h x[i, h] * x[i, h], 8 rows per workgroup.

The file only uses the public `hc` surface, so it means the same thing under either `hc` package:
with the reference's, `hc.simulator.launch(row_sums, x, out)` interprets the body on the host; with
this repository's, `hc.compile(row_sums, target="nvidia-sm100a")` recognises the kernel and runs it
as one CUDA kernel whose float32 result is bit-identical (the additions follow the order of NumPy's
sum). Rows past the end of the buffer are inactive and the store is clipped, so exactly the W
outputs are written.
"""

import argparse
import functools
import sys
from pathlib import Path

import numpy as np

if __package__ in (None, ""):  # run as a script: make the sibling `hc` package importable
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import hc
from hc import Buffer, kernel, sym

W, H = sym.W, sym.H
NVIDIA_TARGET = "nvidia-sm100a"


@kernel(work_shape=(W,), group_shape=(4,))
def row_sums(group, x: Buffer[W, H], out: Buffer[W]) -> None:
    r0 = group.work_offset[0]
    rows = group.load(x[r0:], shape=(group.shape[0], x.shape[1]))
    group.store(out[r0:], rows.sum(axis=1))


@kernel(work_shape=(W,), group_shape=(16,))
def row_norms(group, x: Buffer[W, H, np.float32], out: Buffer[W, np.float32]) -> None:
    gid = group.work_offset
    rows = group.load(x[gid[0] :], shape=(16, x.shape[1]))
    squares = rows**2
    energy = squares.sum(axis=1)
    group.store(out[gid[0] :], np.sqrt(energy))


@kernel(work_shape=(W,), group_shape=(8,))
def row_energy(group, x: Buffer[W, H], out: Buffer[W]) -> None:
    first = group.work_offset[0]
    rows = group.load(x[first:], shape=(group.shape[0], x.shape[1]))
    group.store(out[first:], (rows * rows).sum(axis=-1))


@functools.cache
def compiled(name: str = "row_sums", device: int | None = None):
    return hc.compile(globals()[name], target=NVIDIA_TARGET, device=device)


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--w", type=int, default=262144)
    parser.add_argument("--h", type=int, default=512)
    parser.add_argument("--device", type=int, default=None)
    args = parser.parse_args()
    rng = np.random.default_rng(0)
    x = rng.standard_normal((args.w, args.h)).astype(np.float32)
    out = np.empty((args.w,), np.float32)
    compiled("row_sums", args.device)(x, out)
    rows = slice(0, min(args.w, 4096))
    want = np.array([np.sum(row) for row in x[rows]], np.float32)
    same = np.array_equal(out[rows].view(np.uint32), want.view(np.uint32))
    print(f"row_sums of {args.w} rows of {args.h}: first {rows.stop} rows "
          f"{'bit-identical to' if same else 'DIFFER from'} NumPy's float32 sums")
    return 0 if same else 1


if __name__ == "__main__":
    raise SystemExit(main())
