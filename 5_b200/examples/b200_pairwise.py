"""The pairwise-distance kernel in hc, launched on a B200.

    python 5_b200/examples/b200_pairwise.py [--w1 4096 --w2 4096 --h 128]

Kernels of the two-dimensional workgroup class that opens the reference simulator's own tests
(tests/test_simulator.py:142-167):

  pairwise          out[i, j] = sqrt(sum_h (x1[i, h] - x2[j, h])**2), 4 x 4 outputs per workgroup --
                    the reference's kernel as it stands;
  pairwise_squared  the same without the square root, 8 x 16 outputs per workgroup, written with
                    temporaries and the subtraction the other way round.

The file only uses the public `hc` surface, so it means the same thing under either `hc` package:
with the reference's, `hc.simulator.launch(pairwise, x1, x2, out)` interprets the body on the host;
with this repository's, `hc.compile(pairwise, target="nvidia-sm100a")` recognises the kernel and
runs it as one CUDA kernel whose float32 result is bit-identical. Rows past the end of a buffer
are inactive and stores are clipped, so exactly the W1 x W2 outputs are written.
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

W1, W2, H = sym.W1, sym.W2, sym.H
NVIDIA_TARGET = "nvidia-sm100a"


@kernel(work_shape=(W1, W2), group_shape=(4, 4))
def pairwise(group, x1: Buffer[W1, H], x2: Buffer[W2, H], out: Buffer[W1, W2]) -> None:
    gid = group.work_offset
    lhs = group.load(x1[gid[0] :], shape=(group.shape[0], x1.shape[1]))
    rhs = group.load(x2[gid[1] :], shape=(group.shape[1], x2.shape[1]))
    diff = ((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2)
    group.store(out[gid[0] :, gid[1] :], np.sqrt(diff))


@kernel(work_shape=(W1, W2), group_shape=(8, 16))
def pairwise_squared(group, x1: Buffer[W1, H, np.float32], x2: Buffer[W2, H, np.float32],
                     out: Buffer[W1, W2, np.float32]) -> None:
    r0, c0 = group.work_offset
    rows = group.load(x1[r0:], shape=(8, x1.shape[1]))
    cols = group.load(x2[c0:], shape=(16, x2.shape[1]))
    delta = cols[None, :, :] - rows[:, None, :]
    squares = delta**2
    group.store(out[r0:, c0:], squares.sum(axis=2))


@functools.cache
def compiled(name: str = "pairwise", device: int | None = None):
    return hc.compile(globals()[name], target=NVIDIA_TARGET, device=device)


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--w1", type=int, default=4096)
    parser.add_argument("--w2", type=int, default=4096)
    parser.add_argument("--h", type=int, default=128)
    parser.add_argument("--device", type=int, default=None)
    args = parser.parse_args()
    rng = np.random.default_rng(0)
    x1 = rng.standard_normal((args.w1, args.h)).astype(np.float32)
    x2 = rng.standard_normal((args.w2, args.h)).astype(np.float32)
    out = np.empty((args.w1, args.w2), np.float32)
    compiled("pairwise", args.device)(x1, x2, out)
    rows = slice(0, min(args.w1, 64))
    want = np.sqrt(((x1[rows, None, :] - x2[None, :, :]) ** 2).sum(axis=2))
    same = np.array_equal(out[rows].view(np.uint32), want.view(np.uint32))
    print(f"pairwise {args.w1} x {args.w2} over h = {args.h}: first {rows.stop} rows "
          f"{'bit-identical to' if same else 'DIFFER from'} NumPy's float32 result")
    return 0 if same else 1


if __name__ == "__main__":
    raise SystemExit(main())
