"""The masked element-wise kernel class of `hc.compile(..., target="nvidia-sm100a")`: recognition
(what is accepted, what is refused and why), launch binding, and the C ABI's argument checks that
need no device."""

import ctypes

import numpy as np
import pytest

import hc
from hc import Buffer, kernel, sym
from hc import cuda
from hc._map_kernels import MapContract, recognise_elementwise_map
from hc._pipeline import NVIDIA_SM100A

from examples.b200_elementwise import add_two, compiled, scaled_clamp

W, V = sym.W, sym.V
M_, N_ = sym.M, sym.N
THREE = 3
WIDE = np.float64(0.1)


def test_example_kernels_are_recognised() -> None:
    plan = compiled("add_two").plan
    assert isinstance(plan, MapContract)
    assert (plan.x_param, plan.other_param, plan.out_param, plan.extent, plan.group_size) == ("x", None, "y", "W", 4)
    assert plan.ops == (("add", 2.0),)
    plan = compiled("scaled_clamp").plan
    assert (plan.x_param, plan.other_param, plan.out_param, plan.group_size) == ("x", "y", "out", 64)
    assert plan.ops == (("scale", 0.5), ("add", -1.0), ("rsub_other",), ("max", 0.25), ("scale", -1.0),
                        ("scale", 3.0), ("add_other",))
    assert repr(compiled("add_two")).endswith("stage=nvidia-sm100a)")


def test_spellings() -> None:
    @kernel(work_shape=(W,), group_shape=(8,))
    def in_place(group, x: Buffer[W, np.float32]) -> None:
        """Doubles x where it stands."""
        start = group.work_offset[0]
        v = group.load(x[start : start + 8], shape=(8,))
        v = np.minimum(THREE - v, v * np.float32(2)).astype(np.float32)
        group.store(x[start:], v)
        return None

    plan, why = recognise_elementwise_map(in_place)
    assert plan is None and "combines two computed vectors" in why[0]

    @kernel(work_shape=(W,), group_shape=(8,))
    def doubled(group, x: Buffer[W, np.float32]) -> None:
        start = group.work_offset[0]
        v = group.load(x[start : start + 8], shape=(8,))
        v = np.minimum(THREE - v, 1.5).astype(np.float32)
        group.store(x[start:], v)
        return None

    plan, why = recognise_elementwise_map(doubled)
    assert plan is not None, why
    assert (plan.x_param, plan.out_param, plan.ops) == ("x", "x", (("rsub", 3.0), ("min", 1.5)))

    @kernel(work_shape=(W,), group_shape=(8,))
    def relu(group, x: Buffer[W, np.float32], y: Buffer[W, np.float32]) -> None:
        start = group.work_offset[0]
        v = group.load(x[start:], shape=(8,))
        group.store(y[start:], np.maximum(0.0, v))

    # np.maximum returns its second operand when neither is greater, so maximum(0.0, -0.0) is -0.0 but
    # maximum(-0.0, 0.0) is 0.0: the operand order is part of the operation.
    plan, why = recognise_elementwise_map(relu)
    assert plan is not None and plan.ops == (("rmax", 0.0),), why

    @kernel(work_shape=(16,), group_shape=(16,))
    def fixed(group, a: Buffer[16], b: Buffer[16], c: Buffer[16]) -> None:
        g = group.work_offset[0]
        left = group.vload(a[g:], shape=(16,))
        right = group.vload(b[g:], shape=(16,))
        group.store(c[g:], np.maximum(right, left) - right * 1)

    plan, why = recognise_elementwise_map(fixed)
    assert plan is None and "combines two computed vectors" in why[0]

    @kernel(work_shape=(16,), group_shape=(16,))
    def fixed_ok(group, a: Buffer[16], b: Buffer[16], c: Buffer[16]) -> None:
        g = group.work_offset[0]
        left = group.vload(a[g:], shape=(16,))
        right = group.vload(b[g:], shape=(16,))
        group.store(c[g:], np.maximum(left, right) - right)

    plan, why = recognise_elementwise_map(fixed_ok)
    assert plan is not None and plan.extent == 16, why
    assert (plan.x_param, plan.other_param, plan.ops) == ("a", "b", (("max_other",), ("sub_other",)))


def test_two_dimensional_kernels() -> None:
    from examples.b200_elementwise import affine_relu_2d

    plan = hc.compile(affine_relu_2d, target=NVIDIA_SM100A).plan
    assert isinstance(plan, MapContract) and plan.rank == 2
    assert (plan.x_param, plan.other_param, plan.out_param) == ("x", "shift", "out")
    assert plan.extent == ("M", "N") and plan.group_size == (8, 32)
    assert plan.ops == (("scale", 2.0), ("add_other",), ("rmax", 0.0))

    @kernel(work_shape=(M_, N_), group_shape=(8, 32))
    def swapped(group, x: Buffer[M_, N_], out: Buffer[M_, N_]) -> None:
        r0, c0 = group.work_offset
        tile = group.load(x[c0:, r0:], shape=(8, 32))
        group.store(out[r0:, c0:], tile + 1)

    plan, why = recognise_elementwise_map(swapped)
    assert plan is None and "must load the group's own window" in why[0]

    @kernel(work_shape=(M_, N_), group_shape=(8, 32))
    def wrong_shape(group, x: Buffer[M_, N_], out: Buffer[M_, N_]) -> None:
        r0 = group.work_offset[0]
        c0 = group.work_offset[1]
        tile = group.load(x[r0 : r0 + 8, c0 : c0 + 32], shape=(32, 8))
        group.store(out[r0:, c0:], tile + 1)

    plan, why = recognise_elementwise_map(wrong_shape)
    assert plan is None and "shape=(8, 32)" in why[0]

    @kernel(work_shape=(M_,), group_shape=(8,))
    def rank_mismatch(group, x: Buffer[M_, N_], out: Buffer[M_, N_]) -> None:
        r0 = group.work_offset[0]
        tile = group.load(x[r0:, r0:], shape=(8, 8))
        group.store(out[r0:, r0:], tile + 1)

    plan, why = recognise_elementwise_map(rank_mismatch)
    assert plan is None and "one axis per buffer axis" in why[0]
    handle = hc.compile(affine_relu_2d, target=NVIDIA_SM100A)
    launch = handle.prepare(np.zeros((5, 7), np.float32), np.zeros((5, 7), np.float32), np.zeros((5, 7), np.float32))
    assert launch.symbols == {"M": 5, "N": 7} and launch.group_counts == (1, 1)
    with pytest.raises(hc.LaunchError, match="conflicting binding for N"):
        handle(np.zeros((5, 7), np.float32), np.zeros((5, 8), np.float32), np.zeros((5, 7), np.float32))


def _kernel(body: str, *, params="x: Buffer[W], y: Buffer[W]", work="(W,)", group_shape="(4,)", tmp_path=None, name="k"):
    import importlib.util

    text = f'''
import numpy as np
from hc import Buffer, kernel, sym
W, V = sym.W, sym.V
WIDE = np.float64(0.1)

@kernel(work_shape={work}, group_shape={group_shape})
def kern(group, {params}) -> None:
{body}
'''
    path = tmp_path / f"{name}.py"
    path.write_text(text, encoding="utf-8")
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.kern


GOOD = "    gid = group.work_offset[0]\n    vec = group.vload(x[gid:], shape=(4,))\n    group.store(y[gid:], vec + 2)"


@pytest.mark.parametrize(
    ("name", "kwargs", "message"),
    [
        ("div", {"body": GOOD.replace("vec + 2", "vec / 2")}, "is not element-wise arithmetic this target runs"),
        ("square", {"body": GOOD.replace("vec + 2", "vec * vec")}, "combines two computed vectors"),
        ("f64", {"body": GOOD.replace("vec + 2", "vec * WIDE")}, "is not a loaded vector"),
        ("npf64", {"body": GOOD.replace("vec + 2", "vec * np.float64(2)")}, "is not element-wise arithmetic"),
        ("short", {"body": GOOD.replace("shape=(4,)", "shape=(2,)")}, "must load the group's own window"),
        ("shifted", {"body": GOOD.replace("x[gid:]", "x[gid + 1:]")}, "must load the group's own window"),
        ("whole", {"body": GOOD.replace("y[gid:]", "y")}, "must store to the group's own window"),
        ("other_offset", {"body": GOOD.replace("group.work_offset[0]", "group.group_id[0]")},
         "`group.group_id[0]` is not element-wise arithmetic"),
        ("tail", {"body": GOOD + "\n    group.store(y[gid:], vec)"}, "follows the store"),
        ("no_store", {"body": GOOD.rsplit("\n", 1)[0]}, "must end with"),
        ("loop", {"body": GOOD + "\n    for i in range(2):\n        pass"}, "follows the store"),
        ("extents", {"body": GOOD, "params": "x: Buffer[W], y: Buffer[V]"}, "must have the same extents"),
        ("dtype", {"body": GOOD, "params": "x: Buffer[W, np.float16], y: Buffer[W, np.float16]"},
         "runs element-wise kernels on float32"),
        ("rank", {"body": GOOD, "params": "x: Buffer[W, V], y: Buffer[W]"}, "must have the same extents"),
        ("rank3", {"body": GOOD, "params": "x: Buffer[W, V, 4], y: Buffer[W, V, 4]"}, "rank-1 or rank-2 Buffer"),
        ("work", {"body": GOOD, "work": "(W * 2,)"}, "work_shape must be the buffers' extent"),
        ("group", {"body": GOOD, "group_shape": "(W,)"}, "group_shape must be a positive constant"),
        ("many", {"body": GOOD.replace("vec + 2", "vec" + " + 1" * 9)}, "at most 8 element-wise operations"),
    ],
)
def test_other_kernels_are_refused_with_a_reason(tmp_path, name, kwargs, message) -> None:
    kern = _kernel(tmp_path=tmp_path, name=f"map_{name}", **kwargs)
    handle = hc.compile(kern, target=NVIDIA_SM100A)
    assert handle.plan is None
    assert any(message in line for line in handle.pipeline_diagnostics), handle.pipeline_diagnostics
    with pytest.raises(NotImplementedError, match="cannot launch"):
        handle(np.zeros(4, np.float32), np.zeros(4, np.float32))


WORKITEM = ("    @group.workitems\n    def inner(wi) -> None:\n        gid = wi.global_id()[0]\n"
            "        vec = group.vload(x[gid:], shape=(1,))\n        group.store(y[gid:], vec + 2)\n\n    inner()")


def test_one_element_per_workitem_is_the_same_map(tmp_path) -> None:
    """The kernel written inside `@group.workitems` (tests/test_simulator.py:901-917 in the reference):
    every work-item loads, transforms and stores the element at its global id."""
    from examples.b200_elementwise import add_two_per_workitem

    plan, diagnostics = recognise_elementwise_map(add_two_per_workitem)
    assert diagnostics == [] and (plan.x_param, plan.out_param, plan.ops, plan.extent) == ("src", "dst", (("add", 2.0),), "W")
    plan, diagnostics = recognise_elementwise_map(_kernel(WORKITEM, tmp_path=tmp_path, name="wi_good"))
    assert plan is not None and diagnostics == []
    for name, change, message in [
        ("wi_local", ("wi.global_id()[0]", "wi.local_id()[0]"), "is not element-wise arithmetic"),
        ("wi_wide", ("shape=(1,)", "shape=(4,)"), "must load the group's own window"),
        ("wi_group_offset", ("wi.global_id()[0]", "group.work_offset[0]"), "is not element-wise arithmetic"),
        ("wi_not_called", ("\n\n    inner()", ""), "not part of the load / element-wise / store form"),
        ("wi_subgroups", ("@group.workitems", "@group.subgroups"), "not part of the load / element-wise / store form"),
        ("wi_twice", ("    inner()", "    inner()\n    inner()"), "not part of the load / element-wise / store form"),
    ]:
        assert change[0] in WORKITEM
        plan, diagnostics = recognise_elementwise_map(_kernel(WORKITEM.replace(*change), tmp_path=tmp_path, name=name))
        assert plan is None and message in diagnostics[0], (name, diagnostics)


def test_launch_binding_uses_the_simulator_messages() -> None:
    handle = compiled("add_two")
    launch = handle.prepare(np.zeros(6, np.float32), np.zeros(6, np.float32))
    assert launch.symbols == {"W": 6} and launch.work_shape == (6,) and launch.group_shape == (4,)
    with pytest.raises(hc.LaunchError, match="conflicting binding for W: 4 from 'x.shape\\[0\\]' vs 5 from 'y.shape\\[0\\]'"):
        handle(np.zeros(4, np.float32), np.zeros(5, np.float32))
    with pytest.raises(hc.LaunchError, match="x dtype expected float32, got float64"):
        handle(np.zeros(4, np.float64), np.zeros(4, np.float64))
    typed = compiled("scaled_clamp")
    with pytest.raises(hc.LaunchError, match="y dtype expected float32, got int32"):
        typed(np.zeros(4, np.float32), np.zeros(4, np.int32), np.zeros(4, np.float32))
    with pytest.raises(hc.LaunchError, match="rank does not match"):
        typed(np.zeros((4, 1), np.float32), np.zeros(4, np.float32), np.zeros(4, np.float32))
    empty = np.zeros(0, np.float32)
    assert handle(empty, empty.copy()) is None  # zero-sized work: returns before any CUDA library is touched


def test_c_abi_rejects_bad_map_arguments_without_a_device() -> None:
    lib = cuda.library()
    assert lib.hcCudaMap(None, None) == 1 and lib.hcCudaMapHost(None, None) == 1
    args = cuda._map_args(4, 0x1000, None, 0x2000, (("add", 1.0),))
    assert lib.hcCudaMap(None, ctypes.byref(args)) == 1  # a context is required
    with pytest.raises(ValueError, match="at most 8"):
        cuda._map_args(4, 0x1000, None, 0x2000, (("add", 1.0),) * 9)
    with pytest.raises(ValueError, match="unknown element-wise operation"):
        cuda._map_args(4, 0x1000, None, 0x2000, (("divide", 1.0),))
    assert cuda.MAP_KINDS["min_other"] == 11 and cuda.MAP_KINDS["rmin_other"] == 15 and cuda.MAX_MAP_OPS == 8
