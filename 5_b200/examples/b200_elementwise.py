"""Masked element-wise kernels in hc, launched on a B200.

    python 5_b200/examples/b200_elementwise.py [--n 1000003]

Kernels of the masked load / element-wise / store class:

  add_two       the reference simulator's own masked vector test
                (tests/test_simulator.py:210-224): y = x + 2, four elements per workgroup;
  add_two_per_workitem  the same written one element per work-item inside `@group.workitems`
                (tests/test_simulator.py:901-917);
  scaled_clamp  out = maximum(y - (0.5 * x - 1), 0.25) * -3 + y on float32 buffers, 64 elements
                per workgroup: a chain of element-wise statements with a second input;
  affine_relu_2d  out = maximum(0, 2 * x + shift) on matrices, one 8 x 32 tile per workgroup.

The file only uses the public `hc` surface, so it means the same thing under either `hc` package:
with the reference's, `hc.simulator.launch(add_two, x, y)` interprets the body on the host; with
this repository's, `hc.compile(add_two, target="nvidia-sm100a")` recognises the kernel and runs it
as one bandwidth-bound CUDA kernel. Loads past the end of a buffer are inactive and stores are
clipped, so exactly the first W elements are read and written, whatever W is.
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

W = sym.W
NVIDIA_TARGET = "nvidia-sm100a"
HALF = 0.5
FLOOR = np.float32(0.25)


@kernel(work_shape=(W,), group_shape=(4,))
def add_two(group, x: Buffer[W], y: Buffer[W]) -> None:
    gid = group.work_offset[0]
    vec = group.vload(x[gid:], shape=(4,))
    group.store(y[gid:], vec + 2)


@kernel(work_shape=(W,), group_shape=(64,))
def scaled_clamp(group, x: Buffer[W, np.float32], y: Buffer[W, np.float32], out: Buffer[W, np.float32]) -> None:
    gid = group.work_offset[0]
    xv = group.vload(x[gid:], shape=(64,))
    yv = group.vload(y[gid : gid + 64], shape=(64,))
    t = HALF * xv - 1
    t = np.maximum(yv - t, FLOOR)
    group.store(out[gid:], -t * 3 + yv)


@kernel(work_shape=(W,), group_shape=(4,))
def add_two_per_workitem(group, src: Buffer[W], dst: Buffer[W]) -> None:
    @group.workitems
    def inner(wi) -> None:
        gid = wi.global_id()[0]
        vec = group.vload(src[gid:], shape=(1,))
        group.store(dst[gid:], vec + 2)

    inner()


M, N = sym.M, sym.N


@kernel(work_shape=(M, N), group_shape=(8, 32))
def affine_relu_2d(group, x: Buffer[M, N, np.float32], shift: Buffer[M, N, np.float32], out: Buffer[M, N, np.float32]) -> None:
    """out = maximum(0, 2 * x + shift) on matrices, one 8 x 32 tile per workgroup."""
    r0, c0 = group.work_offset
    tile = group.load(x[r0 : r0 + 8, c0 : c0 + 32], shape=(8, 32))
    other = group.load(shift[r0:, c0:], shape=(8, 32))
    group.store(out[r0:, c0:], np.maximum(0.0, tile * 2 + other))


def scaled_clamp_numpy(x, y):
    """The same statements on whole float32 arrays (what the kernel computes element by element)."""
    t = np.float32(HALF) * x - np.float32(1)
    t = np.maximum(y - t, FLOOR)
    return -t * np.float32(3) + y


@functools.lru_cache(maxsize=None)
def compiled(name, device=None):
    kernels = {
        "add_two": add_two,
        "scaled_clamp": scaled_clamp,
        "add_two_per_workitem": add_two_per_workitem,
        "affine_relu_2d": affine_relu_2d,
    }
    return hc.compile(kernels[name], target=NVIDIA_TARGET, device=device)


def main(argv=None):
    parser = argparse.ArgumentParser(description="hc element-wise kernels on a B200")
    parser.add_argument("--n", type=int, default=1000003)
    parser.add_argument("--device", action="store_true",
                        help="keep the buffers on the GPU: one launch over all n elements per kernel (for profiling)")
    args = parser.parse_args(argv)
    rng = np.random.default_rng(0)
    x = rng.standard_normal(args.n).astype(np.float32)
    y = rng.standard_normal(args.n).astype(np.float32)
    out = np.zeros_like(x)
    if args.device:
        from hc import cuda

        ctx = cuda.default_context()
        dx, dy, dout = ctx.to_device(x), ctx.to_device(y), ctx.empty((args.n,), np.float32)
        compiled("add_two")(dx, dout)
        if not np.array_equal(dout.to_numpy(), x + np.float32(2)):
            raise SystemExit("add_two differs")
        compiled("scaled_clamp")(dx, dy, dout)
        out = dout.to_numpy()
    else:
        compiled("scaled_clamp")(x, y, out)
    print(f"{compiled('scaled_clamp')!r}")
    same = np.array_equal(out, scaled_clamp_numpy(x, y))
    print(f"n={args.n}: bit-identical to NumPy: {same}")
    if not same:
        raise SystemExit("result differs")


if __name__ == "__main__":
    main()
