"""The pairwise-distance kernel class on the CPU side: the recogniser, the oracle against the
reference simulator's stored outputs, and launch binding (no GPU)."""

from __future__ import annotations

import numpy as np
import pytest

import hc
from conftest import GOLDEN as GOLDEN_DIR
from examples import b200_pairwise as examples
from hc import Buffer, kernel, sym
from hc._pairwise_kernels import PairwiseContract, recognise_pairwise
from hc.errors import LaunchError
from oracle import cpu_ref

W1, W2, H = sym.W1, sym.W2, sym.H
TARGET = "nvidia-sm100a"


def test_example_kernels_are_recognised() -> None:
    plan, diagnostics = recognise_pairwise(examples.pairwise)
    assert diagnostics == [] and plan == PairwiseContract(
        kernel_name="pairwise", lhs_param="x1", rhs_param="x2", out_param="out", extents=("W1", "W2", "H"),
        group_shape=(4, 4), take_sqrt=True)
    plan, diagnostics = recognise_pairwise(examples.pairwise_squared)
    assert diagnostics == [] and (plan.take_sqrt, plan.group_shape, plan.lhs_param, plan.rhs_param) == (False, (8, 16), "x1", "x2")
    handle = hc.compile(examples.pairwise, target=TARGET)
    assert isinstance(handle.plan, PairwiseContract) and handle.target == TARGET


def test_the_roles_follow_the_work_axes_not_the_parameter_order() -> None:
    @kernel(work_shape=(W1, W2), group_shape=(2, 8))
    def swapped(group, cols: Buffer[W2, H], result: Buffer[W1, W2], rows: Buffer[W1, H]) -> None:
        gid = group.work_offset
        b = group.load(cols[gid[1] :], shape=(8, cols.shape[1]))
        a = group.load(rows[gid[0] :], shape=(2, rows.shape[1]))
        group.store(result[gid[0] :, gid[1] :], np.sqrt(((a[:, None, :] - b[None, :, :]) ** 2).sum(axis=2)))

    plan, diagnostics = recognise_pairwise(swapped)
    assert diagnostics == [] and (plan.lhs_param, plan.rhs_param, plan.out_param) == ("rows", "cols", "result")
    assert plan.extents == ("W1", "W2", "H")


def _variant(body: str, *, header: str = "group, x1: Buffer[W1, H], x2: Buffer[W2, H], out: Buffer[W1, W2]",
             work: str = "(W1, W2)", groups: str = "(4, 4)"):
    source = (f"@kernel(work_shape={work}, group_shape={groups})\n"
              f"def variant({header}) -> None:\n" + "".join(f"    {line}\n" for line in body.strip().splitlines()))
    namespace = dict(kernel=kernel, Buffer=Buffer, W1=W1, W2=W2, H=H, np=np)
    import linecache

    filename = f"<pairwise-variant-{abs(hash(source))}>"
    linecache.cache[filename] = (len(source), None, source.splitlines(True), filename)
    exec(compile(source, filename, "exec"), namespace)  # noqa: S102 - test-local kernel text
    return namespace["variant"]


GOOD = """
gid = group.work_offset
lhs = group.load(x1[gid[0]:], shape=(group.shape[0], x1.shape[1]))
rhs = group.load(x2[gid[1]:], shape=(group.shape[1], x2.shape[1]))
diff = ((lhs[:, None, :] - rhs[None, :, :]) ** 2).sum(axis=2)
group.store(out[gid[0]:, gid[1]:], np.sqrt(diff))
"""


@pytest.mark.parametrize("change, why", [
    (("** 2", "** 3"), "is not `np.sqrt"),
    ((".sum(axis=2)", ".sum(axis=1)"), "is not `np.sqrt"),
    ((".sum(axis=2)", ".max(axis=2)"), "is not `np.sqrt"),
    (("np.sqrt(diff)", "np.exp(diff)"), "is not `np.sqrt"),
    (("lhs[:, None, :] - rhs[None, :, :]", "lhs[:, None, :] + rhs[None, :, :]"), "is not `np.sqrt"),
    (("lhs[:, None, :] - rhs[None, :, :]", "rhs[:, None, :] - lhs[None, :, :]"), "is not `np.sqrt"),
    (("x1[gid[0]:]", "x1[gid[1]:]"), "must load the group's rows"),  # (the shape names the other axis)
    (("x1[gid[0]:]", "x1[0:]"), "must load the group's rows"),
    (("shape=(group.shape[0], x1.shape[1])", "shape=(group.shape[0], 3)"), "must load the group's rows"),
    (("shape=(group.shape[0], x1.shape[1])", "shape=(5, x1.shape[1])"), "must load the group's rows"),
    (("out[gid[0]:, gid[1]:]", "out[gid[1]:, gid[0]:]"), "must store to the group's own window"),
    (("out[gid[0]:, gid[1]:]", "out[gid[0]:]"), "must store to the group's own window"),
    (("group.store(out[gid[0]:, gid[1]:], np.sqrt(diff))", "pass"), "not part of the load"),
])
def test_other_bodies_are_refused(change, why: str) -> None:
    assert change[0] in GOOD
    plan, diagnostics = recognise_pairwise(_variant(GOOD.replace(*change)))
    assert plan is None and why in diagnostics[0], diagnostics


def test_the_unchanged_body_of_those_variants_is_accepted() -> None:
    plan, diagnostics = recognise_pairwise(_variant(GOOD))
    assert plan is not None and diagnostics == []


@pytest.mark.parametrize("kwargs, why", [
    (dict(header="group, x1: Buffer[W1, H], x2: Buffer[W2, H], out: Buffer[W2, W1]"), "must be Buffer[W1, W2]"),
    (dict(header="group, x1: Buffer[W1, H], x2: Buffer[W2, W1], out: Buffer[W1, W2]"), "must share their second extent"),
    (dict(header="group, x1: Buffer[W1, H, np.float16], x2: Buffer[W2, H], out: Buffer[W1, W2]"), "float32"),
    (dict(header="group, x1: Buffer[W1, H], x2: Buffer[W2, H], out: Buffer[W1]"), "rank-2 Buffer"),
    (dict(work="(W1, W2 + 1)"), "work_shape must be the extents"),
    (dict(work="(W1,)", groups="(4,)"), "two axes"),
])
def test_other_signatures_and_geometries_are_refused(kwargs, why: str) -> None:
    plan, diagnostics = recognise_pairwise(_variant(GOOD, **kwargs))
    assert plan is None and why in diagnostics[0], diagnostics


def test_unrecognised_pairwise_kernels_report_why_through_compile() -> None:
    handle = hc.compile(_variant(GOOD.replace("** 2", "** 4")), target=TARGET)  # (still a `.sum(...)` of something)
    assert handle.plan is None and any("is not `np.sqrt" in text for text in handle.pipeline_diagnostics)
    with pytest.raises(NotImplementedError, match="cannot launch"):
        handle(np.zeros((2, 2), np.float32), np.zeros((2, 2), np.float32), np.zeros((2, 2), np.float32))


# ---------------------------------------------------------------- oracle ---------------


def test_oracle_is_bit_identical_to_the_reference_simulator() -> None:
    with np.load(GOLDEN_DIR / "simpair_f32_seed18.npz") as data:
        cases = [(data["test_x1"], data["test_x2"], data["test_out"], True), (data["x1"], data["x2"], data["out"], True),
                 (data["sq_x1"], data["sq_x2"], data["sq_out"], False)]
    # The reference's own expectation for its test (tests/test_simulator.py:165-167).
    t1, t2, t_out, _ = cases[0]
    assert np.allclose(t_out, np.sqrt(((t1[:, None, :] - t2[None, :, :]) ** 2).sum(axis=2)))
    for x1, x2, out, take_sqrt in cases:
        got = cpu_ref.pairwise_distance(x1, x2, take_sqrt=take_sqrt, rows_per_block=7)
        assert np.array_equal(got.view(np.uint32), out.view(np.uint32))
    assert np.isnan(cases[2][2][:, 7]).all() and np.isinf(cases[2][2][3, :7]).all()  # the NaN column, the infinite row


def test_summation_order_restatement_matches_numpy() -> None:
    rng = np.random.default_rng(3)
    for n in (0, 1, 5, 7, 8, 9, 15, 16, 17, 100, 127, 128, 129, 150, 255, 256, 257, 333, 1000, 1031, 4099):
        for scale in (1.0, 1e4):
            values = (rng.standard_normal(n) * scale).astype(np.float32) ** 2
            want = np.sum(values) if n else np.float32(0)
            assert cpu_ref.pairwise_sum_in_numpy_order(values) == want, n
    # Reducing the last axis of a contiguous block is that same sum per row.
    block = rng.standard_normal((5, 6, 333)).astype(np.float32) ** 2
    per_pair = np.array([[np.sum(block[i, j]) for j in range(6)] for i in range(5)], np.float32)
    assert np.array_equal(block.sum(axis=2), per_pair)


# ---------------------------------------------------------------- launch binding -------


def test_launch_checks_run_before_any_device_work() -> None:
    handle = examples.compiled("pairwise")
    assert handle(np.zeros((0, 3), np.float32), np.zeros((4, 3), np.float32), np.zeros((0, 4), np.float32)) is None
    with pytest.raises(LaunchError, match="conflicting binding for H"):
        handle(np.zeros((2, 3), np.float32), np.zeros((4, 5), np.float32), np.zeros((2, 4), np.float32))
    with pytest.raises(LaunchError, match="dtype expected float32"):
        handle(np.zeros((2, 3), np.float64), np.zeros((4, 3), np.float64), np.zeros((2, 4), np.float64))
