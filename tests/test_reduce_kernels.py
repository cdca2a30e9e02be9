"""The row-sum kernel class on the CPU side: the recogniser, the oracle against the reference
simulator's stored outputs, and what `hc.compile` reports for kernels outside the class (no GPU)."""

from __future__ import annotations

import numpy as np
import pytest

import hc
from conftest import GOLDEN as GOLDEN_DIR
from examples import b200_rowsum as examples
from hc import Buffer, kernel, sym
from hc._reduce_kernels import RowSumContract, recognise_row_sum
from oracle import cpu_ref

W, H = sym.W, sym.H
TARGET = "nvidia-sm100a"


def test_example_kernels_are_recognised() -> None:
    plan, diagnostics = recognise_row_sum(examples.row_sums)
    assert diagnostics == [] and plan == RowSumContract(
        kernel_name="row_sums", in_param="x", out_param="out", extents=("W", "H"), group_rows=4, square=False,
        take_sqrt=False)
    plan, diagnostics = recognise_row_sum(examples.row_norms)
    assert diagnostics == [] and (plan.square, plan.take_sqrt, plan.group_rows) == (True, True, 16)
    plan, diagnostics = recognise_row_sum(examples.row_energy)
    assert diagnostics == [] and (plan.square, plan.take_sqrt, plan.group_rows) == (True, False, 8)
    handle = hc.compile(examples.row_sums, target=TARGET)
    assert isinstance(handle.plan, RowSumContract) and handle.target == TARGET


def test_the_roles_follow_the_body_not_the_parameter_order() -> None:
    @kernel(work_shape=(W,), group_shape=(2,))
    def swapped(group, totals: Buffer[W], values: Buffer[W, H]) -> None:
        first = group.work_offset[0]
        rows = group.load(values[first:], shape=(2, values.shape[1]))
        group.store(totals[first:], rows.sum(axis=1))

    plan, diagnostics = recognise_row_sum(swapped)
    assert diagnostics == [] and (plan.in_param, plan.out_param, plan.extents) == ("values", "totals", ("W", "H"))


def _variant(body: str, *, header: str = "group, x: Buffer[W, H], out: Buffer[W]", work: str = "(W,)",
             groups: str = "(4,)"):
    source = (f"@kernel(work_shape={work}, group_shape={groups})\n"
              f"def variant({header}) -> None:\n" + "".join(f"    {line}\n" for line in body.strip().splitlines()))
    namespace = dict(kernel=kernel, Buffer=Buffer, W=W, H=H, np=np)
    import linecache

    filename = f"<row-sum-variant-{abs(hash(source))}>"
    linecache.cache[filename] = (len(source), None, source.splitlines(True), filename)
    exec(compile(source, filename, "exec"), namespace)  # noqa: S102 - test-local kernel text
    return namespace["variant"]


GOOD = """
r0 = group.work_offset[0]
rows = group.load(x[r0:], shape=(group.shape[0], x.shape[1]))
group.store(out[r0:], rows.sum(axis=1))
"""


@pytest.mark.parametrize("change, why", [
    ((".sum(axis=1)", ".sum(axis=0)"), "is not `rows.sum(axis=1)`"),
    ((".sum(axis=1)", ".max(axis=1)"), "is not `rows.sum(axis=1)`"),
    ((".sum(axis=1)", ".sum()"), "is not `rows.sum(axis=1)`"),
    (("rows.sum(axis=1)", "(rows * 2).sum(axis=1)"), "is not `rows.sum(axis=1)`"),
    (("rows.sum(axis=1)", "(rows ** 3).sum(axis=1)"), "is not `rows.sum(axis=1)`"),
    (("rows.sum(axis=1)", "np.exp(rows.sum(axis=1))"), "is not `rows.sum(axis=1)`"),
    (("rows.sum(axis=1)", "rows.sum(axis=1) + 1"), "is not `rows.sum(axis=1)`"),
    (("x[r0:]", "x[0:]"), "must load the group's rows"),
    (("x[r0:]", "x[r0:, 1:]"), "must load the group's rows"),
    (("shape=(group.shape[0], x.shape[1])", "shape=(group.shape[0], 3)"), "must load the group's rows"),
    (("shape=(group.shape[0], x.shape[1])", "shape=(5, x.shape[1])"), "must load the group's rows"),
    (("out[r0:]", "out[0:]"), "must store to the group's own window"),
    (("out[r0:]", "out[r0:r0 + 2]"), "must store to the group's own window"),
    (("r0 = group.work_offset[0]", "r0 = group.work_offset[0] + 1"), "must load the group's rows"),
    (("group.store(out[r0:], rows.sum(axis=1))", "pass"), "not part of the load"),
])
def test_other_bodies_are_refused(change, why: str) -> None:
    assert change[0] in GOOD
    plan, diagnostics = recognise_row_sum(_variant(GOOD.replace(*change)))
    assert plan is None and why in diagnostics[0], diagnostics


@pytest.mark.parametrize("body", [
    GOOD,
    GOOD.replace("rows.sum(axis=1)", "np.sqrt((rows ** 2).sum(axis=-1))"),
    GOOD.replace("rows.sum(axis=1)", "(rows * rows).sum(axis=1)"),
    GOOD.replace("r0 = group.work_offset[0]", "gid = group.work_offset\nr0 = gid[0]"),
    GOOD.replace("shape=(group.shape[0], x.shape[1])", "shape=(4, x.shape[1])"),
])
def test_the_forms_of_the_class_are_accepted(body: str) -> None:
    plan, diagnostics = recognise_row_sum(_variant(body))
    assert plan is not None and diagnostics == []


@pytest.mark.parametrize("kwargs, why", [
    (dict(header="group, x: Buffer[W, H], out: Buffer[H]"), "must be Buffer[W]"),
    (dict(header="group, x: Buffer[W, H, np.float16], out: Buffer[W]"), "float32"),
    (dict(header="group, x: Buffer[W, H], out: Buffer[W, H]"), "rank-1 Buffer"),
    (dict(header="group, x: Buffer[W, H], out: Buffer[W], extra: Buffer[W]"), "takes (group, x, out)"),
    (dict(work="(W + 1,)"), "work_shape must be the extent"),
    (dict(work="(W, H)", groups="(4, 4)"), "one axis"),
])
def test_other_signatures_and_geometries_are_refused(kwargs, why: str) -> None:
    plan, diagnostics = recognise_row_sum(_variant(GOOD, **kwargs))
    assert plan is None and why in diagnostics[0], diagnostics


def test_unrecognised_reductions_report_why_through_compile() -> None:
    handle = hc.compile(_variant(GOOD.replace(".sum(axis=1)", ".max(axis=1)")), target=TARGET)
    assert handle.plan is None and any("other reductions are not run" in text for text in handle.pipeline_diagnostics)
    with pytest.raises(NotImplementedError, match="cannot launch"):
        handle(np.zeros((2, 2), np.float32), np.zeros((2,), np.float32))


def test_the_other_classes_still_get_their_own_kernels() -> None:
    from examples import b200_elementwise, b200_pairwise
    from hc._map_kernels import MapContract
    from hc._pairwise_kernels import PairwiseContract

    assert isinstance(hc.compile(b200_elementwise.add_two, target=TARGET).plan, MapContract)
    assert isinstance(hc.compile(b200_pairwise.pairwise, target=TARGET).plan, PairwiseContract)


# ---------------------------------------------------------------- oracle ---------------


def test_oracle_is_bit_identical_to_the_reference_simulator() -> None:
    with np.load(GOLDEN_DIR / "simrow_f32_seed19.npz") as data:
        cases = [(data["x"], data["sums"], {}), (data["few_x"], data["few_sums"], {}),
                 (data["norm_x"], data["norms"], dict(square=True, take_sqrt=True)),
                 (data["energy_x"], data["energy"], dict(square=True))]
    for x, want, kwargs in cases:
        for restated in (False, True):
            got = cpu_ref.row_sums(x, restated=restated, **kwargs)
            nan = np.isnan(want)
            assert np.array_equal(np.isnan(got), nan)
            assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32)), (kwargs, restated)
    # A row of -0.0 sums to +0.0: the reduction starts from +0 (the fixture holds such a row).
    few_x, few_sums = cases[1][0], cases[1][1]
    assert np.signbit(few_x[4]).all() and few_sums[4] == 0 and not np.signbit(few_sums[4])
    assert np.isinf(cases[2][1][3]) and np.isnan(cases[2][1][7])  # the infinite row, the NaN row


def test_row_sum_restatement_matches_numpy_for_every_regime() -> None:
    rng = np.random.default_rng(4)
    for h in (1, 5, 7, 8, 9, 16, 100, 127, 128, 129, 150, 255, 256, 257, 333, 1000, 1031, 4099):
        x = (rng.standard_normal((6, h)) * rng.choice([1e-3, 1.0, 1e4], size=(6, h))).astype(np.float32)
        x[0, :] = -0.0
        want = np.array([np.sum(row) for row in x], np.float32)
        for restated in (False, True):
            assert np.array_equal(cpu_ref.row_sums(x, restated=restated).view(np.uint32), want.view(np.uint32)), h
