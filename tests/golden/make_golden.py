"""Generates tests/golden/*.npz by running the UNMODIFIED reference simulator.

    python tests/golden/make_golden.py [--reference /path/to/reference]

The reference (a Python package) is imported from its own checkout; nothing of it is copied
here. Its two absent third-party dependencies are replaced by the stand-ins under
oracle/standins/ (an integer-expression evaluator for launch shapes, and run-to-completion
coroutines); neither carries any of the matmul arithmetic. Each fixture stores the inputs as
raw 16-bit patterns and the simulator's fp32 output, so the parity tests need neither the
reference nor the stand-ins.

Fixtures (all produced by `hc.simulator.launch` on the example kernel):
  sim_f16_m16_n16_k16_seed7, sim_f16_m32_n32_k32_seed7, sim_f16_m17_n19_k18_seed7
      the three shapes of the reference's tests/test_examples.py:22-33, inputs from its
      make_demo_inputs (uniform(-1, 1), seed 7)
  sim_f16_m32_n32_k32_seed0
      the example's own main() (examples/amdgpu_gfx11_wmma_matmul.py:438-441)
  sim_f16_m64_n64_k64_normal_seed0
      benchmark config 1: A, B ~ N(0, 1) from default_rng(0), A drawn first
  sim_bf16_m33_n17_k40_seed5
      a bfloat16 twin of the kernel: the example's source with its element type replaced,
      executed in memory by the same simulator
  simbt_f16_m17_n19_k18_seed9
      the transposed-B member of the family defined in 5_b200/examples/b200_wmma_matmul.py
      (b stored [N, K]); `b_bits` holds B as stored
  simacc_f16_m17_n19_k18_seed11
      the accumulating member of that family (C = C + A.B); `c0` holds C before the launch
  simfusednan_bf16_m33_n17_k40_seed14
      the fused member on inputs with infinities and a NaN (NaN must survive np.maximum)
  simfused_bf16_m33_n17_k40_seed12
      the fused member (C = maximum(0.125 * (A.B) + bias, 0)); `bias` holds the fourth buffer
  simnarrow_bf16_m33_n17_k40_seed13
      the narrow member (c: Buffer[M, N, bfloat16]); `c_bits` holds the 16-bit output
  simf8_e4m3fn_m33_n17_k40_seed16, simf8_e5m2_bt_m17_n19_k18_seed17
      the float8 members of that family (8-bit raw patterns in `a_bits`, `b_bits`): e4m3fn with B
      stored [K, N], e5m2 with B stored [N, K]
  simmap_f32_seed15
      the masked element-wise kernels of 5_b200/examples/b200_elementwise.py: `add_two_x/_y` the
      reference's own vector test (tests/test_simulator.py:210-224), `x`, `y`, `out` the
      scaled_clamp kernel on 1003 elements with NaN and infinities, `x_2d`, `shift_2d`, `out_2d` the
      two-dimensional affine_relu_2d kernel on a 37 x 70 matrix, `workitem_x/_y` the one-element-per-work-item
      form (tests/test_simulator.py:901-917) on 11 elements
  simpair_f32_seed18
      the pairwise-distance kernels of 5_b200/examples/b200_pairwise.py: `test_x1/_x2/_out` the
      reference's own test (tests/test_simulator.py:142-167), `x1`, `x2`, `out` the same kernel on
      37 x 29 outputs over 150 values, `sq_x1`, `sq_x2`, `sq_out` the squared-distance kernel on
      19 x 35 outputs over 333 values with an infinity and a NaN
  simrow_f32_seed19
      the row-sum kernels of 5_b200/examples/b200_rowsum.py: `x`, `sums` row_sums on 37 rows of 150
      values (scales from 1e-3 to 300, some -0.0), `few_x`, `few_sums` on 9 rows of 5 values (one row
      all -0.0), `norm_x`, `norms` row_norms on 21 rows of 333 values with an infinity and a NaN,
      `energy_x`, `energy` row_energy on 13 rows of 1000 values
The file blocked_reference.npz holds `reference_blocked_matmul` of the first four (the
reference test's own comparison value, atol 2e-6).
"""

from __future__ import annotations

import argparse
import importlib
import os
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def _import_reference(reference: Path):
    os.environ["HC_IXSIMPL_VENDOR_DIR"] = str(REPO / "oracle" / "standins" / "ixsimpl_vendor")
    sys.path.insert(0, str(REPO / "oracle" / "standins"))
    sys.path.insert(0, str(reference))
    return importlib.import_module("examples.amdgpu_gfx11_wmma_matmul")


def _bf16_twin(example_module):
    """The example kernel with bfloat16 operands, built from its source text in memory."""
    import ml_dtypes

    source = Path(example_module.__file__).read_text(encoding="utf-8")
    source = source.replace("np.float16", "BF16")
    twin = types.ModuleType("examples.amdgpu_gfx11_wmma_matmul_bf16")
    twin.__file__ = example_module.__file__
    twin.__dict__["BF16"] = ml_dtypes.bfloat16
    sys.modules[twin.__name__] = twin
    exec(compile(source, example_module.__file__, "exec"), twin.__dict__)
    return twin


def _save(name: str, a: np.ndarray, b: np.ndarray, c: np.ndarray, **extra: np.ndarray) -> None:
    np.savez_compressed(
        HERE / f"{name}.npz",
        a_bits=a.view(np.uint8 if a.dtype.itemsize == 1 else np.uint16),
        b_bits=b.view(np.uint8 if b.dtype.itemsize == 1 else np.uint16),
        c=c,
        dtype=np.array(a.dtype.name),
        **extra,
    )
    print(f"{name}: A{a.shape} B{b.shape} -> C{c.shape}", flush=True)


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("HC_REFERENCE_DIR"),
                        help="checkout of the reference project (default: $HC_REFERENCE_DIR, else the location "
                             "tests/conftest.py names)")
    args = parser.parse_args()
    if args.reference is None:
        sys.path.insert(0, str(HERE.parent))
        from conftest import REFERENCE  # the one place that names a default location

        args.reference = str(REFERENCE)
    ex = _import_reference(Path(args.reference))

    blocked = {}
    for m, n, k, seed in [(16, 16, 16, 7), (32, 32, 32, 7), (17, 19, 18, 7), (32, 32, 32, 0)]:
        a, b = ex.make_demo_inputs(m=m, n=n, k=k, seed=seed)
        c = ex.simulate_gfx11_wmma_matmul(a, b)
        name = f"sim_f16_m{m}_n{n}_k{k}_seed{seed}"
        _save(name, a, b, c)
        blocked[name] = ex.reference_blocked_matmul(a, b)
    np.savez_compressed(HERE / "blocked_reference.npz", **blocked)

    rng = np.random.default_rng(0)
    a = rng.standard_normal((64, 64)).astype(np.float16)
    b = rng.standard_normal((64, 64)).astype(np.float16)
    _save("sim_f16_m64_n64_k64_normal_seed0", a, b, ex.simulate_gfx11_wmma_matmul(a, b))

    import ml_dtypes

    twin = _bf16_twin(ex)
    rng = np.random.default_rng(5)
    a = rng.uniform(-1.0, 1.0, size=(33, 40)).astype(ml_dtypes.bfloat16)
    b = rng.uniform(-1.0, 1.0, size=(40, 17)).astype(ml_dtypes.bfloat16)
    c = np.zeros((33, 17), np.float32)
    twin.sim.launch(twin.tiled_gfx11_wmma_matmul, a, b, c)
    _save("sim_bf16_m33_n17_k40_seed5", a, b, c)

    # This repository's transposed-B member of the kernel family (b: Buffer[N, K]), executed by the
    # reference simulator: the file is loaded against the reference's `hc` package.
    import importlib.util

    path = REPO / "5_b200" / "examples" / "b200_wmma_matmul.py"
    spec = importlib.util.spec_from_file_location("b200_example_under_reference", path)
    mod = importlib.util.module_from_spec(spec)
    mod.__package__ = "loaded_by_make_golden"  # keeps the script-mode sys.path insertion off
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(9)
    a = rng.uniform(-1.0, 1.0, size=(17, 18)).astype(np.float16)
    bt = rng.uniform(-1.0, 1.0, size=(19, 18)).astype(np.float16)
    c = np.zeros((17, 19), np.float32)
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("float16", True), a, bt, c)
    _save("simbt_f16_m17_n19_k18_seed9", a, bt, c)

    rng = np.random.default_rng(11)
    a = rng.uniform(-1.0, 1.0, size=(17, 18)).astype(np.float16)
    b = rng.uniform(-1.0, 1.0, size=(18, 19)).astype(np.float16)
    c0 = rng.uniform(-2.0, 2.0, size=(17, 19)).astype(np.float32)
    c = c0.copy()
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("float16", False, "accumulate"), a, b, c)
    _save("simacc_f16_m17_n19_k18_seed11", a, b, c, c0=c0)

    rng = np.random.default_rng(12)
    a = rng.uniform(-1.0, 1.0, size=(33, 40)).astype(ml_dtypes.bfloat16)
    b = rng.uniform(-1.0, 1.0, size=(40, 17)).astype(ml_dtypes.bfloat16)
    bias = rng.uniform(-0.5, 0.5, size=(17,)).astype(np.float32)
    c = np.full((33, 17), np.float32(-7.0))  # every element must be overwritten
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("bfloat16", False, "fused"), a, b, c, bias)
    _save("simfused_bf16_m33_n17_k40_seed12", a, b, c, bias=bias)

    # The same member on inputs that hold infinities and a NaN: np.maximum propagates NaN (inf * 0
    # and inf - inf inside the k-sum), -inf becomes 0, +inf stays.
    rng = np.random.default_rng(14)
    a = rng.uniform(-1.0, 1.0, size=(33, 40)).astype(ml_dtypes.bfloat16)
    b = rng.uniform(-1.0, 1.0, size=(40, 17)).astype(ml_dtypes.bfloat16)
    a[3, 5] = np.inf
    b[5, 2] = 0.0
    a[7, 1] = np.nan
    a[11, 0], a[11, 39] = np.inf, -np.inf
    b[0, :], b[39, :] = 1.0, 1.0
    a[20, 8] = -np.inf
    bias = rng.uniform(-0.5, 0.5, size=(17,)).astype(np.float32)
    c = np.full((33, 17), np.float32(-7.0))
    with np.errstate(invalid="ignore"):
        mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("bfloat16", False, "fused"), a, b, c, bias)
    _save("simfusednan_bf16_m33_n17_k40_seed14", a, b, c, bias=bias)

    rng = np.random.default_rng(13)
    a = rng.uniform(-1.0, 1.0, size=(33, 40)).astype(ml_dtypes.bfloat16)
    b = rng.uniform(-1.0, 1.0, size=(40, 17)).astype(ml_dtypes.bfloat16)
    c = np.full((33, 17), 7.0).astype(ml_dtypes.bfloat16)
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("bfloat16", False, "narrow"), a, b, c)
    _save("simnarrow_bf16_m33_n17_k40_seed13", a, b, c.astype(np.float32), c_bits=c.view(np.uint16))
    # 8-bit float members of the family (the simulator widens any NumPy element type with
    # np.float32(...)): e4m3fn with B stored [K, N], e5m2 with B stored [N, K]. Values cover the
    # formats' subnormals as well as their normal range.
    rng = np.random.default_rng(16)
    a = (rng.standard_normal((33, 40)) * rng.choice([0.01, 1.0, 8.0], size=(33, 40))).astype(ml_dtypes.float8_e4m3fn)
    b = (rng.standard_normal((40, 17)) * rng.choice([0.01, 1.0, 8.0], size=(40, 17))).astype(ml_dtypes.float8_e4m3fn)
    c = np.full((33, 17), np.float32(-7.0))
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("float8_e4m3fn"), a, b, c)
    _save("simf8_e4m3fn_m33_n17_k40_seed16", a, b, c)
    rng = np.random.default_rng(17)
    a = (rng.standard_normal((17, 18)) * rng.choice([1e-4, 1.0, 100.0], size=(17, 18))).astype(ml_dtypes.float8_e5m2)
    bt = (rng.standard_normal((19, 18)) * rng.choice([1e-4, 1.0, 100.0], size=(19, 18))).astype(ml_dtypes.float8_e5m2)
    c = np.zeros((17, 19), np.float32)
    mod.hc.simulator.launch(mod.tiled_wmma_matmul_for("float8_e5m2", True), a, bt, c)
    _save("simf8_e5m2_bt_m17_n19_k18_seed17", a, bt, c)

    # The masked element-wise kernels of 5_b200/examples/b200_elementwise.py under the reference
    # simulator: the reference's own vector test (tests/test_simulator.py:210-224) and a chain of
    # statements with a second input, on a length that no group size divides, with NaN and
    # infinities among the values.
    path = REPO / "5_b200" / "examples" / "b200_elementwise.py"
    spec = importlib.util.spec_from_file_location("b200_elementwise_under_reference", path)
    ew = importlib.util.module_from_spec(spec)
    ew.__package__ = "loaded_by_make_golden"
    sys.modules[spec.name] = ew
    spec.loader.exec_module(ew)
    x = np.arange(6, dtype=np.float32)
    y = np.zeros((6,), dtype=np.float32)
    ew.hc.simulator.launch(ew.add_two, x, y)
    rng = np.random.default_rng(15)
    x2 = rng.standard_normal(1003).astype(np.float32)
    y2 = rng.standard_normal(1003).astype(np.float32)
    x2[[5, 700]] = np.nan, -np.inf
    y2[[64, 1002]] = np.inf, np.nan
    out2 = np.full((1003,), np.float32(-7.0))
    with np.errstate(invalid="ignore"):
        ew.hc.simulator.launch(ew.scaled_clamp, x2, y2, out2)
    # The two-dimensional member: 8 x 32 tiles over a 37 x 70 matrix (ragged on both axes), with zeros of
    # both signs where the maximum's tie rule shows.
    x3 = rng.standard_normal((37, 70)).astype(np.float32)
    s3 = rng.standard_normal((37, 70)).astype(np.float32)
    x3[0, :4] = 0.0, -0.0, np.nan, np.inf
    s3[0, :4] = -0.0, -0.0, 1.0, -np.inf
    out3 = np.full((37, 70), np.float32(-7.0))
    with np.errstate(invalid="ignore"):
        ew.hc.simulator.launch(ew.affine_relu_2d, x3, s3, out3)
    # The work-item form (tests/test_simulator.py:901-917) on a length the group size does not divide.
    wi_x = rng.standard_normal(11).astype(np.float32)
    wi_y = np.full((11,), np.float32(-7.0))
    ew.hc.simulator.launch(ew.add_two_per_workitem, wi_x, wi_y)
    np.savez_compressed(HERE / "simmap_f32_seed15.npz", add_two_x=x, add_two_y=y, x=x2, y=y2, out=out2,
                        x_2d=x3, shift_2d=s3, out_2d=out3, workitem_x=wi_x, workitem_y=wi_y)
    print(f"simmap_f32_seed15: add_two{ x.shape } scaled_clamp{ x2.shape } affine_relu_2d{ x3.shape }", flush=True)

    # The pairwise kernels of 5_b200/examples/b200_pairwise.py under the reference simulator: the
    # reference's own test (tests/test_simulator.py:142-167, 5 x 6 outputs over 3 values), and shapes
    # that no group shape divides with 150 values per row (NumPy's sum splits at 72, the tail has
    # 6 values) and with 333 (three levels of splitting), with an infinity and a NaN among them.
    path = REPO / "5_b200" / "examples" / "b200_pairwise.py"
    spec = importlib.util.spec_from_file_location("b200_pairwise_under_reference", path)
    pw = importlib.util.module_from_spec(spec)
    pw.__package__ = "loaded_by_make_golden"
    sys.modules[spec.name] = pw
    spec.loader.exec_module(pw)
    t1 = np.arange(15, dtype=np.float32).reshape(5, 3)
    t2 = np.arange(18, dtype=np.float32).reshape(6, 3) / 3.0
    t_out = np.zeros((5, 6), dtype=np.float32)
    pw.hc.simulator.launch(pw.pairwise, t1, t2, t_out)
    rng = np.random.default_rng(18)
    p1 = (rng.standard_normal((37, 150)) * rng.choice([1e-3, 1.0, 300.0], size=(37, 150))).astype(np.float32)
    p2 = (rng.standard_normal((29, 150)) * rng.choice([1e-3, 1.0, 300.0], size=(29, 150))).astype(np.float32)
    p_out = np.full((37, 29), np.float32(-7.0))
    pw.hc.simulator.launch(pw.pairwise, p1, p2, p_out)
    q1 = rng.standard_normal((19, 333)).astype(np.float32)
    q2 = rng.standard_normal((35, 333)).astype(np.float32)
    q1[3, 200], q2[7, 5] = np.inf, np.nan
    q_out = np.full((19, 35), np.float32(-7.0))
    with np.errstate(invalid="ignore"):
        pw.hc.simulator.launch(pw.pairwise_squared, q1, q2, q_out)
    np.savez_compressed(HERE / "simpair_f32_seed18.npz", test_x1=t1, test_x2=t2, test_out=t_out, x1=p1, x2=p2, out=p_out,
                        sq_x1=q1, sq_x2=q2, sq_out=q_out)
    print(f"simpair_f32_seed18: pairwise{t_out.shape} pairwise{p_out.shape} pairwise_squared{q_out.shape}", flush=True)

    # The row-sum kernels of 5_b200/examples/b200_rowsum.py under the reference simulator: row lengths
    # below eight (added in order), 150 (NumPy's sum splits at 72, the tail has 6 values), 333 and 1000
    # (three levels of splitting); no group size divides the row counts.
    path = REPO / "5_b200" / "examples" / "b200_rowsum.py"
    spec = importlib.util.spec_from_file_location("b200_rowsum_under_reference", path)
    rs = importlib.util.module_from_spec(spec)
    rs.__package__ = "loaded_by_make_golden"
    sys.modules[spec.name] = rs
    spec.loader.exec_module(rs)
    rng = np.random.default_rng(19)
    r1 = (rng.standard_normal((37, 150)) * rng.choice([1e-3, 1.0, 300.0], size=(37, 150))).astype(np.float32)
    r1[rng.integers(0, 37, 40), rng.integers(0, 150, 40)] = -0.0
    r1_out = np.full((37,), np.float32(-7.0))
    rs.hc.simulator.launch(rs.row_sums, r1, r1_out)
    r2 = rng.standard_normal((9, 5)).astype(np.float32)
    r2[4, :] = -0.0
    r2_out = np.full((9,), np.float32(-7.0))
    rs.hc.simulator.launch(rs.row_sums, r2, r2_out)
    r3 = rng.standard_normal((21, 333)).astype(np.float32)
    r3[3, 200], r3[7, 5] = np.inf, np.nan
    r3_out = np.full((21,), np.float32(-7.0))
    with np.errstate(invalid="ignore"):
        rs.hc.simulator.launch(rs.row_norms, r3, r3_out)
    r4 = (rng.standard_normal((13, 1000)) * 30.0).astype(np.float32)
    r4_out = np.full((13,), np.float32(-7.0))
    rs.hc.simulator.launch(rs.row_energy, r4, r4_out)
    np.savez_compressed(HERE / "simrow_f32_seed19.npz", x=r1, sums=r1_out, few_x=r2, few_sums=r2_out, norm_x=r3,
                        norms=r3_out, energy_x=r4, energy=r4_out)
    print(f"simrow_f32_seed19: row_sums{r1.shape} row_sums{r2.shape} row_norms{r3.shape} row_energy{r4.shape}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
