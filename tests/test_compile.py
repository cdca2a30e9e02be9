"""`hc.compile(..., target="nvidia-sm100a")`: argument checks, kernel recognition, launch binding."""

import subprocess
import sys
import os

import numpy as np
import pytest

import hc
from hc import Buffer, WorkGroup, WorkItem, idx_type, kernel, sym, tensor_type, undef_type, vector_type
from hc._pipeline import NVIDIA_SM100A, known_targets, recognise_tiled_matmul
from hc.symbols import ceil_div

from conftest import REFERENCE, REPO
from examples.b200_wmma_matmul import compiled_for, tiled_wmma_matmul_for

M, N, K = sym.M, sym.N, sym.K


def _helpers(tm, tn, tk, wave, acc, in_dtype, effects="pure", mma_body="matmul"):
    """Real helpers of a (tm, tn, tk) tile on `wave` lanes: lane l owns column l % tn and rows
    l // tn, l // tn + wave // tn, ... of the tile (`acc` values per lane)."""
    step_rows = max(wave // tn, 1)

    @kernel.intrinsic(
        scope=WorkItem, effects=effects, const_attrs={"wave_size", "arch"},
        operand_types=(undef_type(), tensor_type((tm, tk), in_dtype), tensor_type((tk, tn), in_dtype),
                       vector_type((tk,), in_dtype), vector_type((tk,), in_dtype),
                       vector_type((acc,), np.float32), idx_type()),
        result_types=(vector_type((acc,), np.float32),))
    def mma(group, a_tile, b_tile, a_frag, b_frag, acc_frag, *, lane, wave_size, arch):
        if mma_body == "identity":
            return acc_frag
        a_vals = a_tile.with_inactive(value=in_dtype(0))
        b_vals = b_tile.with_inactive(value=in_dtype(0))
        out = np.empty((acc,), dtype=np.float32)
        for slot in range(acc):
            total = np.float32(acc_frag[slot])
            for kk in range(tk):
                total += np.float32(a_vals[lane // tn + slot * step_rows, kk]) * np.float32(b_vals[kk, lane % tn])
            out[slot] = total
        return group.vload(out, shape=(acc,))

    @kernel.func(scope=WorkGroup)
    def zeros(group):
        @group.workitems
        def per_lane(wi):
            return group.vzeros(shape=(acc,), dtype=np.float32)

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def ones(group):
        @group.workitems
        def per_lane(wi):
            return group.vones(shape=(acc,), dtype=np.float32)

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def from_c(group, c, row0, col0):
        c_tile = group.load(c[row0 : row0 + tm, col0 : col0 + tn], shape=(tm, tn))

        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            return c_tile[lane // tn :: step_rows, lane % tn].vec().with_inactive(value=np.float32(0))

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def step_fn(group, a_tile, b_tile, acc_values):
        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            return mma(group, a_tile, b_tile, a_tile[lane % tm, :].vec(), b_tile[:, lane % tn].vec(),
                       acc_values[:, lane, 0], lane=lane, wave_size=wave, arch="x")

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def plus_bias(group, bias, col0, acc_values):
        bias_tile = group.load(bias[col0 : col0 + tn], shape=(tn,))

        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            return acc_values[:, lane, 0] + bias_tile[lane % tn : lane % tn + 1].vec().with_inactive(value=np.float32(0))

        return per_lane()

    @kernel.func(scope=WorkGroup)
    def store(group, c, row0, col0, acc_values):
        @group.workitems
        def per_lane(wi):
            lane = wi.local_id()[0]
            col = col0 + lane % tn
            group.store(c[row0 + lane // tn : row0 + tm : step_rows, col : col + 1], acc_values[:, lane, :])

        per_lane()

    return mma, zeros, ones, from_c, step_fn, plus_bias, store


def _family(*, tile=(16, 16, 16), wave=32, acc=8, in_dtype=np.float16, out_dtype=np.float32,
            effects="pure", k_step=None, work_shape=None, loop=True, b_dims=None, mma_body="matmul",
            windows="tile", store_at="tile", init="zeros"):
    """A matmul kernel of the example's family with one aspect varied (or broken)."""
    tm, tn, tk = tile
    step = tk if k_step is None else k_step
    mma, zeros, ones, from_c, step_fn, plus_bias, store = _helpers(tm, tn, tk, wave, acc, in_dtype, effects, mma_body)
    start = {"zeros": zeros, "ones": ones}[init]

    shape = work_shape if work_shape is not None else (ceil_div(M, tm) * wave, ceil_div(N, tn))
    bd = b_dims if b_dims is not None else (K, N)
    launch = dict(work_shape=shape, group_shape=(wave, 1), subgroup_size=wave)

    if not loop:
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            a_tile = group.load(a[row0 : row0 + tm, 0:tk], shape=(tm, tk))
            b_tile = group.load(b[0:tk, col0 : col0 + tn], shape=(tk, tn))
            store(group, c, row0, col0, step_fn(group, a_tile, b_tile, start(group)))
    elif windows == "constant":  # every workgroup reads the first tile row / column
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[0:tm, k0 : k0 + tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, 0:tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, row0, col0, acc_values)
    elif windows == "swapped":  # rows from group_id[1], columns from group_id[0]
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[1] * tm, group.group_id[0] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, row0, col0, acc_values)
    elif windows == "wide":  # the k window is wider than the k step
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + 2 * tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, row0, col0, acc_values)
    elif store_at == "shifted":  # the tile is stored one row lower than it was computed for
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, row0 + 1, col0, acc_values)
    elif store_at == "transposed":  # row and column origin exchanged in the store
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, col0, row0, acc_values)
    else:
        @kernel(**launch)
        def matmul(group, a: Buffer[M, K, in_dtype], b: Buffer[bd[0], bd[1], in_dtype],
                   c: Buffer[M, N, out_dtype]) -> None:
            row0, col0 = group.group_id[0] * tm, group.group_id[1] * tn
            acc_values = start(group)
            for k0 in range(0, a.shape[1], step):
                a_tile = group.load(a[row0 : row0 + tm, k0 : k0 + tk], shape=(tm, tk))
                b_tile = group.load(b[k0 : k0 + tk, col0 : col0 + tn], shape=(tk, tn))
                acc_values = step_fn(group, a_tile, b_tile, acc_values)
            store(group, c, row0, col0, acc_values)

    return matmul


# ---------------------------------------------------------------- compile() arguments ----


def test_compile_rejects_non_kernels_and_bad_symbols() -> None:
    with pytest.raises(TypeError, match="@kernel-decorated"):
        hc.compile(lambda group: None)
    kern = tiled_wmma_matmul_for("float16")
    with pytest.raises(TypeError, match="symbols must be a Mapping"):
        hc.compile(kern, [("M", 1)])
    with pytest.raises(TypeError, match="must bind to an int"):
        hc.compile(kern, {"M": 1.5})
    with pytest.raises(TypeError, match="must bind to an int"):
        hc.compile(kern, {"M": True})
    with pytest.raises(ValueError, match="bound twice with conflicting"):
        hc.compile(kern, {"M": 1, sym.M: 2})
    with pytest.raises(TypeError, match="cannot interpret"):
        hc.compile(kern, {3: 1})
    with pytest.raises(ValueError, match="unknown hc.compile target"):
        hc.compile(kern, target="amdgpu-gfx11")

    @kernel(work_shape=(M,), literals={M})
    def with_literals(group) -> None:
        pass

    with pytest.raises(ValueError, match="'N' is not a declared literal symbol"):
        hc.compile(with_literals, {"N": 1})
    assert hc.compile(with_literals, {"M": 4, sym.M: 4}).bindings == {"M": 4}


def test_handle_fields_and_repr() -> None:
    kern = tiled_wmma_matmul_for("float16")
    plain = hc.compile(kern, {"K": 64})
    assert plain.kernel is kern and plain.bindings == {"K": 64}
    assert plain.front_ir is None and plain.hc_ir is None and plain.hc_ir_text is None
    assert any("MLIR" in d for d in plain.pipeline_diagnostics)
    assert repr(plain) == "CompiledKernel(tiled_wmma_matmul_float16, {K=64}, stage=hc_front)"
    with pytest.raises(NotImplementedError, match="without a target"):
        plain(None, None, None)
    with pytest.raises(Exception):
        plain.target = "x"  # frozen
    handle = hc.compile(kern, target=NVIDIA_SM100A, schedule="module {}")
    assert handle.schedule == "module {}" and handle.target in known_targets()
    assert repr(handle).endswith("stage=nvidia-sm100a)")


# ---------------------------------------------------------------- recognition -----------


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_example_kernel_is_recognised(dtype: str) -> None:
    plan = compiled_for(dtype).plan
    assert plan is not None
    assert (plan.a_param, plan.b_param, plan.c_param) == ("a", "b", "c")
    assert (plan.m_dim, plan.n_dim, plan.k_dim) == ("M", "N", "K")
    assert plan.input_dtype == dtype and plan.output_dtype == "float32"
    assert plan.tile == (16, 16, 16) and plan.wave_size == 32 and plan.accumulators_per_lane == 8
    assert plan.intrinsic_name == "wmma_16x16x16" and plan.has_target_lowering
    assert plan.intrinsic_const_attrs == ("arch", "wave_size")


def test_lowering_hook_is_called_and_steers_the_variant() -> None:
    plan = compiled_for("float16").plan
    assert plan.lowering["variant"] == "auto" and plan.lowering["input_dtype"] == "float16"
    assert "tcgen05.mma" in plan.lowering["instruction"] and (256, 256, 128) in plan.lowering["cta_tiles"]

    def with_hook(hook):
        kern = _family()
        mma = next(fn for fn in __import__("hc._pipeline", fromlist=["x"])._reachable_callables(kern)
                   if hasattr(fn, "__hc_intrinsic__"))
        mma.lower(target=NVIDIA_SM100A)(hook)
        return hc.compile(kern, target=NVIDIA_SM100A)

    forced = with_hook(lambda ctx, *a, **k: {"variant": "dense", "why": f"{ctx.tile} on {ctx.target}"})
    assert forced.plan.lowering == {"variant": "dense", "why": "(16, 16, 16) on nvidia-sm100a"}
    assert with_hook(lambda ctx, *a, **k: None).plan.lowering is None
    bad = with_hook(lambda ctx, *a, **k: {"variant": "fastest"})
    assert bad.plan is None and any("variant must be one of" in d for d in bad.pipeline_diagnostics)
    broken = with_hook(lambda ctx, *a, **k: 1 / 0)
    assert broken.plan is None and any("raised ZeroDivisionError" in d for d in broken.pipeline_diagnostics)
    other = _family()
    assert hc.compile(other, target=NVIDIA_SM100A).plan.lowering is None  # no hook registered


def test_transposed_b_member_is_recognised() -> None:
    handle = compiled_for("float16", None, True)
    plan = handle.plan
    assert plan is not None and plan.b_transposed and plan.intrinsic_name == "wmma_16x16x16"
    assert (plan.m_dim, plan.n_dim, plan.k_dim) == ("M", "N", "K") and plan.tile == (16, 16, 16)
    launch = handle.prepare(np.zeros((17, 18), np.float16), np.zeros((19, 18), np.float16),
                            np.zeros((17, 19), np.float32))
    assert launch.symbols == {"M": 17, "K": 18, "N": 19} and launch.work_shape == (64, 2)
    with pytest.raises(hc.LaunchError, match="conflicting binding for K: 18 from 'a.shape\\[1\\]' vs 19 from 'b.shape\\[1\\]'"):
        handle(np.zeros((17, 18), np.float16), np.zeros((18, 19), np.float16), np.zeros((17, 19), np.float32))
    assert not compiled_for("float16").plan.b_transposed


def test_accumulating_and_fused_members_are_recognised() -> None:
    acc = compiled_for("float16", None, False, "accumulate").plan
    assert acc is not None and acc.accumulate and acc.epilogue == () and acc.bias_param is None
    fused_handle = compiled_for("bfloat16", None, False, "fused")
    fused = fused_handle.plan
    assert fused is not None and not fused.accumulate and fused.bias_param == "bias"
    assert fused.epilogue == (("scale", 0.125), ("bias",), ("max", 0.0))
    plain = compiled_for("float16").plan
    assert not plain.accumulate and plain.epilogue == () and plain.bias_param is None
    bf16 = np_bf16()
    launch = fused_handle.prepare(np.zeros((33, 40), bf16), np.zeros((40, 17), bf16), np.zeros((33, 17), np.float32),
                                  np.zeros((17,), np.float32))
    assert launch.symbols == {"M": 33, "K": 40, "N": 17}
    with pytest.raises(hc.LaunchError, match="conflicting binding for N: 17 from .* vs 16 from 'bias.shape\\[0\\]'"):
        fused_handle(np.zeros((33, 40), bf16), np.zeros((40, 17), bf16), np.zeros((33, 17), np.float32),
                     np.zeros((16,), np.float32))
    with pytest.raises(hc.LaunchError, match="bias dtype expected float32, got float64"):
        fused_handle(np.zeros((33, 40), bf16), np.zeros((40, 17), bf16), np.zeros((33, 17), np.float32),
                     np.zeros((17,), np.float64))


_VARIANT_SOURCE = """
import numpy as np
from hc import Buffer, WorkGroup, WorkItem, idx_type, kernel, sym, tensor_type, undef_type, vector_type
from hc.symbols import ceil_div

M, N, K = sym.M, sym.N, sym.K
SIX = 6.0

@kernel.intrinsic(
    scope=WorkItem, effects="pure", const_attrs={{"wave_size", "arch"}},
    operand_types=(undef_type(), tensor_type((16, 16), np.float16), tensor_type((16, 16), np.float16),
                   vector_type((16,), np.float16), vector_type((16,), np.float16),
                   vector_type((8,), np.float32), idx_type()),
    result_types=(vector_type((8,), np.float32),))
def mma(group, a_tile, b_tile, a_frag, b_frag, acc_frag, *, lane, wave_size, arch):
    a_vals = a_tile.with_inactive(value=np.float16(0))
    b_vals = b_tile.with_inactive(value=np.float16(0))
    out = np.empty((8,), dtype=np.float32)
    for slot in range(8):
        total = np.float32(acc_frag[slot])
        for kk in range(16):
            total += np.float32(a_vals[lane // 16 + 2 * slot, kk]) * np.float32(b_vals[kk, lane % 16])
        out[slot] = total
    return group.vload(out, shape=(8,))

@kernel.func(scope=WorkGroup)
def zeros(group):
    @group.workitems
    def per_lane(wi):
        return group.vzeros(shape=(8,), dtype=np.float32)
    return per_lane()

@kernel.func(scope=WorkGroup)
def step_fn(group, a_tile, b_tile, acc):
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        return mma(group, a_tile, b_tile, a_tile[lane % 16, :].vec(), b_tile[:, lane % 16].vec(),
                   acc[:, lane, 0], lane=lane, wave_size=32, arch="x")
    return per_lane()

@kernel.func(scope=WorkGroup)
def from_c(group, c, row0, col0):
    c_tile = group.load(c[row0 : row0 + 16, col0 : col0 + 16], shape=(16, 16))
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        return c_tile[lane // 16 :: 2, lane % 16].vec().with_inactive(value=np.float32(0))
    return per_lane()

@kernel.func(scope=WorkGroup)
def plus_bias(group, bias, col0, acc):
    bias_tile = group.load(bias[col0 : col0 + 16], shape=(16,))
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        return acc[:, lane, 0] + bias_tile[lane % 16 : lane % 16 + 1].vec().with_inactive(value=np.float32(0))
    return per_lane()

@kernel.func(scope=WorkGroup)
def minus_bias(group, bias, col0, acc):
    bias_tile = group.load(bias[col0 : col0 + 16], shape=(16,))
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        return acc[:, lane, 0] - bias_tile[lane % 16 : lane % 16 + 1].vec().with_inactive(value=np.float32(0))
    return per_lane()

@kernel.func(scope=WorkGroup)
def store(group, c, row0, col0, acc):
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        col = col0 + lane % 16
        group.store(c[row0 + lane // 16 : row0 + 16 : 2, col : col + 1], acc[:, lane, :])
    per_lane()

@kernel.func(scope=WorkGroup)
def store_some(group, c, row0, col0, acc):
    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        col = col0 + lane % 16
        if lane != 7:
            group.store(c[row0 + lane // 16 : row0 + 16 : 2, col : col + 1], acc[:, lane, :])
    per_lane()

@kernel(work_shape=(ceil_div(M, 16) * 32, ceil_div(N, 16)), group_shape=(32, 1), subgroup_size=32)
def matmul(group, a: Buffer[M, K, np.float16], b: Buffer[K, N, np.float16], c: Buffer[M, N, np.float32]{extra_param}) -> None:
    row0 = group.group_id[0] * 16
    col0 = 16 * group.group_id[1]
    acc = {init}
    for k0 in range(0, a.shape[1], 16):
        a_tile = group.load(a[row0 : row0 + 16, k0 : k0 + 16], shape=(16, 16))
        b_tile = group.load(b[k0 : k0 + 16, col0 : col0 + 16], shape=(16, 16))
        acc = step_fn(group, a_tile, b_tile, acc){in_loop}
{after}
    {store}(group, c, row0, col0, acc)
{tail}
"""


def _variant(tmp_path, name, *, init="zeros(group)", after=(), extra_param="", tail="", in_loop="", store="store"):
    import importlib.util

    text = _VARIANT_SOURCE.format(init=init, after="\n".join("    " + line for line in after),
                                  extra_param=extra_param, tail="    " + tail if tail else "", store=store,
                                  in_loop=("\n        " + in_loop) if in_loop else "")
    path = tmp_path / f"{name}.py"
    path.write_text(text, encoding="utf-8")
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.matmul


def test_statements_around_the_k_loop(tmp_path) -> None:
    """What the recogniser reads before the k-loop (accumulators loaded from c) and between the
    loop and the store (element-wise statements in their spellings)."""
    plan, why = recognise_tiled_matmul(_variant(tmp_path, "v_acc", init="from_c(group, c, row0, col0)"))
    assert plan is not None and plan.accumulate and plan.epilogue == (), why
    plan, why = recognise_tiled_matmul(_variant(
        tmp_path, "v_ops", after=["acc = 2 * acc", "acc = acc - np.float32(1.5)", "acc = acc.astype(np.float32)",
                                  "acc = np.minimum(SIX, acc)", "acc = np.maximum(acc, -0.5)"]))
    assert plan is not None and not plan.accumulate, why
    assert plan.epilogue == (("scale", 2.0), ("add", -1.5), ("min", 6.0), ("max", -0.5))
    plan, why = recognise_tiled_matmul(_variant(
        tmp_path, "v_bias", init="from_c(group, c, row0, col0)", extra_param=", bias: Buffer[N, np.float32]",
        after=["acc = plus_bias(group, bias, col0, acc)", "acc = acc * 0.1"]))
    assert plan is not None and plan.accumulate and plan.bias_param == "bias", why
    assert plan.epilogue == (("bias",), ("scale", float(np.float32(0.1))))

    def rejected(name, message, **kwargs):
        plan, why = recognise_tiled_matmul(_variant(tmp_path, name, **kwargs))
        assert plan is None and any(message in line for line in why), why

    rejected("r_div", "is not an element-wise statement this target folds", after=["acc = acc / 2"])
    rejected("r_square", "is not an element-wise statement this target folds", after=["acc = acc * acc"])
    rejected("r_exp", "is not an element-wise statement this target folds", after=["acc = np.exp(acc)"])
    rejected("r_other", "is not an element-wise statement this target folds", after=["other = acc * 2"])
    rejected("r_many", "at most 4 element-wise statements", after=["acc = acc + 1"] * 5)
    rejected("r_after", "after the store", tail="acc = acc * 2")
    rejected("r_unused", "must be added to `acc` exactly once", extra_param=", bias: Buffer[N, np.float32]")
    rejected("r_dtype", "must be Buffer[N, float32]", extra_param=", bias: Buffer[N, np.float16]",
             after=["acc = plus_bias(group, bias, col0, acc)"])
    rejected("r_extent", "must be Buffer[N, float32]", extra_param=", bias: Buffer[M, np.float32]",
             after=["acc = plus_bias(group, bias, col0, acc)"])
    rejected("r_early", "is neither a tile-origin assignment", init="zeros(group)\n    peek = from_c(group, c, row0, col0)")
    # What the statements do, not only how they look:
    rejected("r_literal", "the accumulators must be initialised once, by a call", init="0")
    rejected("r_loop_extra", "in the k-loop is not one of", in_loop="acc = acc * 2")
    rejected("r_loop_if", "in the k-loop is not one of", in_loop="if k0 > 16: acc = zeros(group)")
    rejected("r_bias_sign", "that are not a @ b + bias", extra_param=", bias: Buffer[N, np.float32]",
             after=["acc = minus_bias(group, bias, col0, acc)"])
    rejected("r_bias_origin", "that are not a @ b + bias",
             extra_param=", bias: Buffer[N, np.float32]", after=["acc = plus_bias(group, bias, row0, acc)"])
    rejected("r_branchy_store", "helpers around the intrinsic must be straight-line code", store="store_some")
    rejected("r_acc_origin", "or column origin", init="from_c(group, c, row0, col0 + 16)")


def test_narrow_member_and_astype_placement(tmp_path) -> None:
    narrow = compiled_for("bfloat16", None, False, "narrow")
    assert narrow.plan is not None and narrow.plan.output_dtype == "bfloat16" and narrow.plan.epilogue == ()
    bf16 = np_bf16()
    with pytest.raises(hc.LaunchError, match="c dtype expected bfloat16, got float32"):
        narrow(np.zeros((33, 40), bf16), np.zeros((40, 17), bf16), np.zeros((33, 17), np.float32))
    half_c = ", c: Buffer[M, N, np.float32]"
    source = _VARIANT_SOURCE.replace(half_c, ", c: Buffer[M, N, np.float16]")
    assert source != _VARIANT_SOURCE

    def variant(name, **kwargs):
        import importlib.util

        text = source.format(init=kwargs.get("init", "zeros(group)"), extra_param="", tail="", store="store", in_loop="",
                             after="\n".join("    " + line for line in kwargs.get("after", ())))
        path = tmp_path / f"{name}.py"
        path.write_text(text, encoding="utf-8")
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return recognise_tiled_matmul(module.matmul)

    plan, why = variant("n_implicit")  # the store itself narrows, as in the simulator
    assert plan is not None and plan.output_dtype == "float16", why
    plan, why = variant("n_ops", after=["acc = acc * 0.5", "acc = acc.astype(np.float32)", "acc = acc.astype(np.float16)"])
    assert plan is not None and plan.epilogue == (("scale", 0.5),), why
    plan, why = variant("n_late", after=["acc = acc.astype(np.float16)", "acc = acc * 0.5"])
    assert plan is None and any("runs on the 16-bit values" in line for line in why), why
    plan, why = variant("n_other", after=["acc = acc.astype(np.float64)"])
    assert plan is None and any("is not an element-wise statement" in line for line in why), why
    plan, why = variant("n_acc", init="from_c(group, c, row0, col0)")
    assert plan is None and any("needs a float32 `c`" in line for line in why), why


def np_bf16():
    import ml_dtypes

    return ml_dtypes.bfloat16


def test_family_members_are_recognised() -> None:
    for kwargs in ({}, {"in_dtype": __import__("ml_dtypes").bfloat16}, {"tile": (32, 16, 16), "acc": 16},
                   {"tile": (16, 16, 32)}, {"wave": 64, "acc": 4}):
        plan, diagnostics = recognise_tiled_matmul(_family(**kwargs))
        assert plan is not None, diagnostics
        assert plan.tile == kwargs.get("tile", (16, 16, 16))


@pytest.mark.parametrize(
    ("kwargs", "message"),
    [
        ({"in_dtype": np.float32}, "are not a\\[M,K\\], b\\[K,N\\]"),
        ({"out_dtype": np.float64}, "c\\[M,N\\] of one of \\['float32', 'float16', 'bfloat16'\\]"),
        ({"b_dims": (N, K)}, "axis 1 of the `b` window must advance with the k-loop variable"),
        ({"effects": "write"}, "expected 'pure'"),
        ({"acc": 4}, "accumulator values per lane"),
        ({"k_step": 8}, "k-loop must be"),
        ({"loop": False}, "exactly one k-loop"),
        ({"work_shape": (ceil_div(M, 16) * 32, ceil_div(N, 32))}, "work_shape evaluates to"),
        ({"work_shape": (M, N, K)}, "work_shape must be a pair"),
        # Kernels with the right shape that compute something else: the reference simulator would run
        # them as written, so launching them as C = A.B would give different results.
        ({"windows": "constant"}, "axis 0 of the `a` window must be the tile's rows .* \\(found `0:tm`\\)"),
        ({"windows": "constant"}, "axis 1 of the `b` window must be the tile's columns"),
        ({"windows": "swapped"}, "axis 0 of the `a` window must be the tile's rows .* o = group.group_id\\[0\\] \\* 16"),
        ({"windows": "wide"}, "axis 1 of the `a` window must advance with the k-loop variable as `k0 : k0 \\+ 16`"),
        ({"store_at": "shifted"}, "argument `row0 \\+ 1` of the store .* it is 16\\*group_id\\[0\\] \\+ 1"),
        ({"store_at": "transposed"}, "writes outside its tile of `c`"),
        ({"init": "ones"}, "does not start the accumulators at zero"),
        ({"mma_body": "identity"}, "leaves values in its tile of `c` that are not a @ b"),
    ],
)
def test_other_kernels_are_refused_with_a_reason(kwargs: dict, message: str) -> None:
    kern = _family(**kwargs)
    handle = hc.compile(kern, target=NVIDIA_SM100A)
    assert handle.plan is None
    assert any(__import__("re").search(message, d) for d in handle.pipeline_diagnostics), handle.pipeline_diagnostics
    assert "unsupported" in repr(handle)
    with pytest.raises(NotImplementedError, match="cannot launch"):
        handle(np.zeros((1, 1), np.float16), np.zeros((1, 1), np.float16), np.zeros((1, 1), np.float32))


def test_kernel_without_intrinsic_is_refused() -> None:
    @kernel(work_shape=(ceil_div(M, 16) * 32, ceil_div(N, 16)), group_shape=(32, 1), subgroup_size=32)
    def plain(group, a: Buffer[M, K, np.float16], b: Buffer[K, N, np.float16], c: Buffer[M, N, np.float32]) -> None:
        pass

    plan, diagnostics = recognise_tiled_matmul(plain)
    assert plan is None and "no @kernel.intrinsic is reachable" in diagnostics[0]


# ---------------------------------------------------------------- launch binding --------


def _buffers(m: int, n: int, k: int, dtype=np.float16):
    return np.zeros((m, k), dtype), np.zeros((k, n), dtype), np.zeros((m, n), np.float32)


def test_prepare_binds_symbols_and_geometry() -> None:
    handle = compiled_for("float16")
    launch = handle.prepare(*_buffers(17, 19, 18))
    assert launch.symbols == {"M": 17, "K": 18, "N": 19}
    assert launch.work_shape == (64, 2) and launch.group_shape == (32, 1) and launch.subgroup_size == 32
    assert launch.group_counts == (2, 2) and not launch.is_empty
    a, b, c = _buffers(4, 5, 6)
    assert handle.prepare(a, c=c, b=b).symbols == {"M": 4, "K": 6, "N": 5}


def test_launch_errors_use_the_simulator_messages() -> None:
    handle = compiled_for("float16")
    a, b, c = _buffers(16, 16, 16)
    cases = [
        ((a.tolist(), b, c), "a must be a numpy.ndarray buffer"),
        ((a[0], b, c), "a rank does not match its Buffer annotation"),
        ((a, b.astype(np.float32), c), "b dtype expected float16, got float32"),
        ((a, b, c.astype(np.float64)), "c dtype expected float32, got float64"),
        ((a, np.zeros((17, 16), np.float16), c), "conflicting binding for K: 16 from 'a.shape\\[1\\]' vs 17 from 'b.shape\\[0\\]'"),
        ((a, b, np.zeros((16, 15), np.float32)), "conflicting binding for N"),
        ((a, b), "missing a required argument: 'c'"),
    ]
    for args, message in cases:
        with pytest.raises(hc.LaunchError, match=message):
            handle(*args)
    assert issubclass(hc.LaunchError, hc.SimulatorError)


def test_compile_time_symbols_constrain_every_call() -> None:
    handle = hc.compile(tiled_wmma_matmul_for("float16"), {"K": 32}, target=NVIDIA_SM100A)
    assert handle.prepare(*_buffers(8, 8, 32)).symbols["K"] == 32
    with pytest.raises(hc.LaunchError, match="conflicting binding for K: 32 from 'hc.compile\\(symbols=...\\)' vs 16"):
        handle(*_buffers(8, 8, 16))


def test_zero_sized_work_is_a_no_op_without_a_device() -> None:
    handle = compiled_for("float16")
    for shape in ((0, 5, 7), (5, 0, 7)):
        a, b, c = _buffers(*shape)
        assert handle.prepare(a, b, c).is_empty
        assert handle(a, b, c) is None  # returns before any CUDA library is touched


@pytest.mark.skipif(not REFERENCE.exists(), reason="the reference checkout is not on this machine")
def test_the_reference_kernel_object_is_accepted_unchanged() -> None:
    """The decorated kernel of the reference's own example (made with the reference's `hc`)
    compiles for the NVIDIA target of this package: the drop-in is by duck typing."""
    script = r"""
import importlib.util, sys
import numpy as np
from examples.amdgpu_gfx11_wmma_matmul import tiled_gfx11_wmma_matmul
spec = importlib.util.spec_from_file_location("hc_b200", sys.argv[1] + "/__init__.py", submodule_search_locations=[sys.argv[1]])
ours = importlib.util.module_from_spec(spec); sys.modules["hc_b200"] = ours; spec.loader.exec_module(ours)
handle = ours.compile(tiled_gfx11_wmma_matmul, target="nvidia-sm100a")
plan = handle.plan
assert plan is not None, handle.pipeline_diagnostics
assert (plan.tile, plan.wave_size, plan.input_dtype, plan.intrinsic_name) == ((16, 16, 16), 32, "float16", "wmma_gfx11")
launch = handle.prepare(np.zeros((17, 18), np.float16), np.zeros((18, 19), np.float16), np.zeros((17, 19), np.float32))
assert launch.symbols == {"M": 17, "K": 18, "N": 19} and launch.work_shape == (64, 2)
try:
    handle.prepare(np.zeros((17, 18), np.float16), np.zeros((17, 19), np.float16), np.zeros((17, 19), np.float32))
except ours.LaunchError as exc:
    assert "conflicting binding for K" in str(exc)
else:
    raise AssertionError("conflict not detected")
print("ok")
"""
    env = dict(os.environ)
    env["HC_IXSIMPL_VENDOR_DIR"] = str(REPO / "oracle" / "standins" / "ixsimpl_vendor")
    env["PYTHONPATH"] = os.pathsep.join([str(REFERENCE), str(REPO / "oracle" / "standins")])
    result = subprocess.run([sys.executable, "-c", script, str(REPO / "5_b200" / "hc")], env=env,
                            capture_output=True, text=True, timeout=120, cwd=str(REPO / "tests"))
    assert result.returncode == 0, result.stderr
    assert result.stdout.strip() == "ok"


def test_simulator_launch_entry_point_runs_the_target() -> None:
    """`hc.simulator.launch(fn, *args)`, the reference's launch call, compiles for the NVIDIA target and
    launches: same binding errors, zero-sized work is a no-op, an unrecognised kernel is refused (there
    is no simulator to fall back to)."""
    import hc.simulator as sim

    kern = tiled_wmma_matmul_for("float16")
    handle = sim.compiled(kern)
    assert handle.plan is not None and handle.target == NVIDIA_SM100A and sim.compiled(kern) is handle
    assert sim.run is sim.launch
    a, b, c = _buffers(0, 8, 16)
    assert sim.launch(kern, a, b, c) is None  # zero-sized work: no CUDA library is touched
    with pytest.raises(sim.LaunchError, match="conflicting binding for K"):
        sim.launch(kern, np.zeros((4, 4), np.float16), np.zeros((5, 4), np.float16), np.zeros((4, 4), np.float32))
    with pytest.raises(sim.LaunchError, match="expects a function decorated with @kernel"):
        sim.launch(lambda group: None)
    with pytest.raises(sim.LaunchError, match="takes no simulator target"):
        sim.launch(kern, a, b, c, target=object())
    with pytest.raises(NotImplementedError, match="cannot launch"):
        sim.launch(_family(windows="constant"), *_buffers(16, 16, 16))


@pytest.mark.skipif(not REFERENCE.exists(), reason="the reference checkout is not on this machine")
def test_the_reference_example_module_runs_against_this_package() -> None:
    """The reference's example file, imported as it is with this package as `hc`: its own entry point
    `simulate_gfx11_wmma_matmul` reaches the GPU launch through `hc.simulator.launch` (checked here as
    far as a machine without a GPU goes: compilation, binding, the zero-sized launch)."""
    import importlib.util

    import hc.simulator as sim

    spec = importlib.util.spec_from_file_location("reference_example_under_b200",
                                                  REFERENCE / "examples" / "amdgpu_gfx11_wmma_matmul.py")
    example = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = example
    spec.loader.exec_module(example)
    assert example.sim is sim
    handle = sim.compiled(example.tiled_gfx11_wmma_matmul)
    assert handle.plan is not None and handle.plan.intrinsic_name == "wmma_gfx11", handle.pipeline_diagnostics
    out = example.simulate_gfx11_wmma_matmul(np.zeros((0, 16), np.float16), np.zeros((16, 8), np.float16))
    assert out.shape == (0, 8)
    with pytest.raises(ValueError, match="must match"):
        example.simulate_gfx11_wmma_matmul(np.zeros((4, 4), np.float16), np.zeros((5, 4), np.float16))
