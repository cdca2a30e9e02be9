"""Tiled WMMA matmul in hc, parametrised by element type, launched on a B200.

    python 5_b200/examples/b200_wmma_matmul.py [--dtype float16|bfloat16] [--m 64 --n 64 --k 64]

The kernel is the one the reference ships as examples/amdgpu_gfx11_wmma_matmul.py: one wave
of 32 workitems per 16x16 tile of C, a k-loop of masked 16x16 tile loads, a per-lane
16x16x16 multiply-accumulate intrinsic that keeps 8 fp32 accumulator values per lane, and a
masked strided store. The reference hard-codes float16; here `build_tiled_wmma_matmul`
produces the same kernel for float16 or bfloat16 (both are in the language's minimum dtype
set, doc/langref.md:526-527).

The file only uses the public `hc` surface, so it means the same thing under either `hc`
package: with the reference's, `hc.simulator.launch(tiled_wmma_matmul, a, b, c)` interprets
the body on the host (the intrinsic's Python body below is that simulator fallback); with
this repository's, `hc.compile(tiled_wmma_matmul, target="nvidia-sm100a")` recognises the
kernel and runs it on the GPU, where the tile distribution written here is re-tiled to
128x256 CTA tiles with accumulators in tensor memory.
"""

import argparse
import functools
import sys
from pathlib import Path

import numpy as np

if __package__ in (None, ""):  # run as a script: make the sibling `hc` package importable
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import hc
from hc import Buffer, WorkGroup, WorkItem, idx_type, kernel, sym, tensor_type, undef_type, vector_type
from hc.symbols import ceil_div

WAVE_LANES = 32
TILE_M = 16
TILE_N = 16
TILE_K = 16
ACC_PER_LANE = TILE_M * TILE_N // WAVE_LANES  # 8 fp32 values per lane
ARCH = "wave32-16x16x16"
NVIDIA_TARGET = "nvidia-sm100a"

M = sym.M
N = sym.N
K = sym.K


def _tile_origin(tile_row, tile_col):
    return tile_row * TILE_M, tile_col * TILE_N


MEMBERS = ("plain", "accumulate", "fused", "narrow")
FUSED_SCALE = 0.125  # the constant the "fused" member multiplies its accumulators by


def _helpers(element_type, b_transposed):
    """The pieces every member of the family shares: the 16x16x16 intrinsic with its NVIDIA
    lowering hook, and the workgroup functions around it. With `b_transposed` the B tile is
    indexed (n, k)."""
    b_tile_shape = (TILE_N, TILE_K) if b_transposed else (TILE_K, TILE_N)

    @kernel.intrinsic(
        scope=WorkItem,
        effects="pure",
        const_attrs={"wave_size", "arch"},
        operand_types=(
            undef_type(),
            tensor_type((TILE_M, TILE_K), element_type),
            tensor_type(b_tile_shape, element_type),
            vector_type((TILE_K,), element_type),
            vector_type((TILE_K,), element_type),
            vector_type((ACC_PER_LANE,), np.float32),
            idx_type(),
        ),
        result_types=(vector_type((ACC_PER_LANE,), np.float32),),
    )
    def wmma_16x16x16(group, a_tile, b_tile, a_frag, b_frag, acc_frag, *, lane, wave_size, arch):
        """Host-simulator body: the lane's share of D = A.B + C for one 16x16x16 step.

        Lane l owns column l % 16 and rows l // 16, l // 16 + 2, ... of the tile; each value
        is accumulated over k ascending in fp32. Masked-off tile elements count as zero.
        """
        del a_frag, b_frag, arch  # the staged tiles carry the same data as the fragments
        a_vals = a_tile.with_inactive(value=element_type(0))
        b_vals = b_tile.with_inactive(value=element_type(0))
        col = lane % TILE_N
        row_step = wave_size // TILE_N
        out = np.empty((ACC_PER_LANE,), dtype=np.float32)
        for slot in range(ACC_PER_LANE):
            row = lane // TILE_N + slot * row_step
            total = np.float32(acc_frag[slot])
            for kk in range(TILE_K):
                b_value = b_vals[col, kk] if b_transposed else b_vals[kk, col]
                total += np.float32(a_vals[row, kk]) * np.float32(b_value)
            out[slot] = total
        return group.vload(out, shape=(ACC_PER_LANE,))

    @wmma_16x16x16.lower(target=NVIDIA_TARGET)
    def _lower_to_umma(ctx, *operands, **attrs):
        """What the NVIDIA target does with this intrinsic instead of emitting a per-lane op: the
        whole k-loop of 16x16x16 steps becomes tcgen05.mma instructions on CTA tiles. The hook
        may steer the kernel family; here it leaves the choice to the launcher."""
        del operands, attrs
        return {
            "variant": "auto",
            "instruction": getattr(ctx, "instruction", "tcgen05.mma.kind::f16"),
            "accumulator": "tensor memory, fp32",
            "cta_tiles": getattr(ctx, "cta_tiles", ()),
            "b_operand": "K-major" if b_transposed else "MN-major",
            "input_dtype": np.dtype(element_type).name,
        }

    @kernel.func(scope=WorkItem)
    def a_fragment(wi, a_tile):
        return a_tile[wi.local_id()[0] % TILE_M, :].vec().with_inactive(value=element_type(0))

    @kernel.func(scope=WorkItem)
    def b_fragment(wi, b_tile):
        lane_col = wi.local_id()[0] % TILE_N
        column = b_tile[lane_col, :] if b_transposed else b_tile[:, lane_col]
        return column.vec().with_inactive(value=element_type(0))

    @kernel.func(scope=WorkGroup)
    def zero_accumulators(group):
        @group.workitems
        def per_lane(wi):
            del wi
            return group.vzeros(shape=(ACC_PER_LANE,), dtype=np.float32)

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def load_accumulators(group, c, row0, col0):
        """The lanes' accumulators start from the C tile (elements outside C read as 0)."""
        c_tile = group.load(c[row0 : row0 + TILE_M, col0 : col0 + TILE_N], shape=(TILE_M, TILE_N))

        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            rows = c_tile[lane // TILE_N :: WAVE_LANES // TILE_N, lane % TILE_N]
            return rows.vec().with_inactive(value=np.float32(0))

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def multiply_accumulate(group, a_tile, b_tile, acc):
        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            return wmma_16x16x16(
                group,
                a_tile,
                b_tile,
                a_fragment(wi, a_tile),
                b_fragment(wi, b_tile),
                acc[:, lane, 0],
                lane=lane,
                wave_size=WAVE_LANES,
                arch=ARCH,
            )

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def add_column_bias(group, bias, col0, acc):
        """Adds bias[column] to every accumulator of that column."""
        bias_tile = group.load(bias[col0 : col0 + TILE_N], shape=(TILE_N,))

        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            value = bias_tile[lane % TILE_N : lane % TILE_N + 1].vec().with_inactive(value=np.float32(0))
            return acc[:, lane, 0] + value

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def store_accumulators(group, c, row0, col0, acc):
        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            col = col0 + lane % TILE_N
            first = row0 + lane // TILE_N
            # Slices, not scalar indices: on an edge tile they clip to an empty overlap.
            group.store(c[first : row0 + TILE_M : WAVE_LANES // TILE_N, col : col + 1], acc[:, lane, :])

        per_lane()

    return (zero_accumulators, load_accumulators, multiply_accumulate, add_column_bias, store_accumulators)


_LAUNCH = dict(
    work_shape=(ceil_div(M, TILE_M) * WAVE_LANES, ceil_div(N, TILE_N)),
    group_shape=(WAVE_LANES, 1),
    subgroup_size=WAVE_LANES,
)


def build_tiled_wmma_matmul(element_type, b_transposed=False, member="plain"):
    """Returns the `@kernel` function for A, B of `element_type` (np.float16 or bfloat16).

    With `b_transposed` the kernel takes B stored transposed, `b: Buffer[N, K]` (the usual layout
    of a weight matrix): its k-loop loads `b[col0:col0+16, k0:k0+16]` windows and the intrinsic's
    B tile is (n, k). The arithmetic is the same, C = A @ B^T-as-stored.

    `member` selects what surrounds the k-loop:
      "plain"       C = A @ B, the reference example itself;
      "accumulate"  C = C + A @ B: the accumulators are loaded from `c` instead of zeroed;
      "fused"       C = maximum(FUSED_SCALE * (A @ B) + bias, 0) with a fourth buffer
                    `bias: Buffer[N, float32]`: element-wise statements between the k-loop and
                    the store, which the NVIDIA target folds into the store of C;
      "narrow"      C = (A @ B).astype(element_type) with `c: Buffer[M, N, element_type]`: fp32
                    accumulation, 16-bit output.
    """
    element_type = np.dtype(element_type).type
    if member not in MEMBERS:
        raise ValueError(f"member must be one of {MEMBERS}")
    if b_transposed and member != "plain":
        raise ValueError("the transposed-B example is built as the plain member only")
    (zero_accumulators, load_accumulators, multiply_accumulate, add_column_bias,
     store_accumulators) = _helpers(element_type, b_transposed)
    suffix = np.dtype(element_type).name

    if b_transposed:

        @kernel(**_LAUNCH)
        def tiled_wmma_matmul_bt(
            group,
            a: Buffer[M, K, element_type],
            b: Buffer[N, K, element_type],
            c: Buffer[M, N, np.float32],
        ) -> None:
            row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])
            acc = zero_accumulators(group)
            for k0 in range(0, a.shape[1], TILE_K):
                a_tile = group.load(a[row0 : row0 + TILE_M, k0 : k0 + TILE_K], shape=(TILE_M, TILE_K))
                bt_tile = group.load(b[col0 : col0 + TILE_N, k0 : k0 + TILE_K], shape=(TILE_N, TILE_K))
                acc = multiply_accumulate(group, a_tile, bt_tile, acc)
            store_accumulators(group, c, row0, col0, acc)

        tiled_wmma_matmul_bt.__name__ = f"tiled_wmma_matmul_bt_{suffix}"
        return tiled_wmma_matmul_bt

    if member == "accumulate":

        @kernel(**_LAUNCH)
        def tiled_wmma_matmul_acc(
            group,
            a: Buffer[M, K, element_type],
            b: Buffer[K, N, element_type],
            c: Buffer[M, N, np.float32],
        ) -> None:
            row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])
            acc = load_accumulators(group, c, row0, col0)
            for k0 in range(0, a.shape[1], TILE_K):
                a_tile = group.load(a[row0 : row0 + TILE_M, k0 : k0 + TILE_K], shape=(TILE_M, TILE_K))
                b_tile = group.load(b[k0 : k0 + TILE_K, col0 : col0 + TILE_N], shape=(TILE_K, TILE_N))
                acc = multiply_accumulate(group, a_tile, b_tile, acc)
            store_accumulators(group, c, row0, col0, acc)

        tiled_wmma_matmul_acc.__name__ = f"tiled_wmma_matmul_acc_{suffix}"
        return tiled_wmma_matmul_acc

    if member == "fused":

        @kernel(**_LAUNCH)
        def tiled_wmma_matmul_fused(
            group,
            a: Buffer[M, K, element_type],
            b: Buffer[K, N, element_type],
            c: Buffer[M, N, np.float32],
            bias: Buffer[N, np.float32],
        ) -> None:
            row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])
            acc = zero_accumulators(group)
            for k0 in range(0, a.shape[1], TILE_K):
                a_tile = group.load(a[row0 : row0 + TILE_M, k0 : k0 + TILE_K], shape=(TILE_M, TILE_K))
                b_tile = group.load(b[k0 : k0 + TILE_K, col0 : col0 + TILE_N], shape=(TILE_K, TILE_N))
                acc = multiply_accumulate(group, a_tile, b_tile, acc)
            acc = acc * np.float32(FUSED_SCALE)
            acc = add_column_bias(group, bias, col0, acc)
            acc = np.maximum(acc, np.float32(0))
            store_accumulators(group, c, row0, col0, acc)

        tiled_wmma_matmul_fused.__name__ = f"tiled_wmma_matmul_fused_{suffix}"
        return tiled_wmma_matmul_fused

    if member == "narrow":

        @kernel(**_LAUNCH)
        def tiled_wmma_matmul_narrow(
            group,
            a: Buffer[M, K, element_type],
            b: Buffer[K, N, element_type],
            c: Buffer[M, N, element_type],
        ) -> None:
            row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])
            acc = zero_accumulators(group)
            for k0 in range(0, a.shape[1], TILE_K):
                a_tile = group.load(a[row0 : row0 + TILE_M, k0 : k0 + TILE_K], shape=(TILE_M, TILE_K))
                b_tile = group.load(b[k0 : k0 + TILE_K, col0 : col0 + TILE_N], shape=(TILE_K, TILE_N))
                acc = multiply_accumulate(group, a_tile, b_tile, acc)
            acc = acc.astype(element_type)
            store_accumulators(group, c, row0, col0, acc)

        tiled_wmma_matmul_narrow.__name__ = f"tiled_wmma_matmul_narrow_{suffix}"
        return tiled_wmma_matmul_narrow

    @kernel(**_LAUNCH)
    def tiled_wmma_matmul(
        group,
        a: Buffer[M, K, element_type],
        b: Buffer[K, N, element_type],
        c: Buffer[M, N, np.float32],
    ) -> None:
        row0, col0 = _tile_origin(group.group_id[0], group.group_id[1])
        acc = zero_accumulators(group)
        for k0 in range(0, a.shape[1], TILE_K):
            a_tile = group.load(a[row0 : row0 + TILE_M, k0 : k0 + TILE_K], shape=(TILE_M, TILE_K))
            b_tile = group.load(b[k0 : k0 + TILE_K, col0 : col0 + TILE_N], shape=(TILE_K, TILE_N))
            acc = multiply_accumulate(group, a_tile, b_tile, acc)
        store_accumulators(group, c, row0, col0, acc)

    tiled_wmma_matmul.__name__ = f"tiled_wmma_matmul_{suffix}"
    return tiled_wmma_matmul


@functools.lru_cache(maxsize=None)
def tiled_wmma_matmul_for(dtype_name, b_transposed=False, member="plain"):
    """The kernel for "float16", "bfloat16", "float8_e4m3fn" or "float8_e5m2" (built once per process)."""
    if dtype_name in ("bfloat16", "float8_e4m3fn", "float8_e5m2"):
        import ml_dtypes

        return build_tiled_wmma_matmul(getattr(ml_dtypes, dtype_name), b_transposed, member)
    if dtype_name == "float16":
        return build_tiled_wmma_matmul(np.float16, b_transposed, member)
    raise ValueError(f"unsupported element type {dtype_name!r}")


@functools.lru_cache(maxsize=None)
def compiled_for(dtype_name, device=None, b_transposed=False, member="plain"):
    """`hc.compile(..., target="nvidia-sm100a")` of the kernel for one element type."""
    return hc.compile(tiled_wmma_matmul_for(dtype_name, b_transposed, member), target=NVIDIA_TARGET,
                      device=device)


def gpu_wmma_matmul(a, b, *, device=None, b_transposed=False):
    """C = A @ B on the GPU; the counterpart of the reference's simulate_gfx11_wmma_matmul
    (examples/amdgpu_gfx11_wmma_matmul.py:338-348), with the same argument checks. With
    `b_transposed`, `b` holds B transposed (shape (n, k)) and the Buffer[N, K] kernel is used."""
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("A and B must be rank-2 matrices")
    if a.shape[1] != (b.shape[1] if b_transposed else b.shape[0]):
        raise ValueError("A.shape[1] must match B.shape[0]")
    if a.dtype != b.dtype or a.dtype.name not in ("float16", "bfloat16", "float8_e4m3fn", "float8_e5m2"):
        raise ValueError("this example expects float16, bfloat16 or float8 A and B operands of one type")
    c = np.zeros((a.shape[0], b.shape[0] if b_transposed else b.shape[1]), dtype=np.float32)
    compiled_for(a.dtype.name, device, b_transposed)(a, b, c)
    return c


def make_demo_inputs(*, m=32, n=32, k=32, seed=0, dtype=np.float16):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, size=(m, k)).astype(dtype)
    b = rng.uniform(-1.0, 1.0, size=(k, n)).astype(dtype)
    return a, b


def main(argv=None):
    parser = argparse.ArgumentParser(description="hc tiled WMMA matmul on a B200")
    parser.add_argument("--dtype", default="float16", choices=("float16", "bfloat16"))
    parser.add_argument("--m", type=int, default=64)
    parser.add_argument("--n", type=int, default=64)
    parser.add_argument("--k", type=int, default=64)
    args = parser.parse_args(argv)
    dtype = np.float16
    if args.dtype == "bfloat16":
        import ml_dtypes

        dtype = ml_dtypes.bfloat16
    a, b = make_demo_inputs(m=args.m, n=args.n, k=args.k, dtype=dtype)
    out = gpu_wmma_matmul(a, b)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    error = np.linalg.norm(out - exact) / max(np.linalg.norm(exact), 1e-30)
    print(f"{compiled_for(args.dtype)!r}")
    print(f"shape: A={a.shape}, B={b.shape}, C={out.shape}; relative Frobenius error vs float64: {error:.3e}")
    if error > 1e-3:
        raise SystemExit("result outside tolerance")


if __name__ == "__main__":
    main()
