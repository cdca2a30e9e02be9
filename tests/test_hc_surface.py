"""The hc definition surface: decorators, Buffer annotations, type contracts, symbols.

Mirrors the reference's tests/test_intrinsic_contracts.py, tests/test_public_api.py and the
symbol-binding parts of tests/test_simulator.py for the pieces the matmul path uses.
"""

from __future__ import annotations

import numpy as np
import pytest

import hc
from hc import Buffer, WorkItem, idx_type, kernel, sym, tensor_type, undef_type, vector_type
from hc._intrinsic_contracts import serialize_intrinsic_type_spec, validate_intrinsic_type_contract_record
from hc.symbols import Bindings, SymbolConflictError, UnboundSymbolError, ceil_div


def test_type_contract_schema_serializes_specs() -> None:
    assert serialize_intrinsic_type_spec(tensor_type((4, "N"), np.float32)) == {
        "kind": "tensor", "shape": ("4", "N"), "dtype": "float32"}
    assert serialize_intrinsic_type_spec(vector_type((8,), np.float16)) == {
        "kind": "vector", "shape": ("8",), "dtype": "float16"}
    assert serialize_intrinsic_type_spec(idx_type("lane")) == {"kind": "idx", "expr": "lane"}
    assert serialize_intrinsic_type_spec(undef_type()) == {"kind": "undef"}
    assert serialize_intrinsic_type_spec(None) == {"kind": "undef"}


@pytest.mark.parametrize(
    ("record", "message"),
    [
        ({}, "missing string kind"),
        ({"kind": "buffer"}, "unsupported kind"),
        ({"kind": "tensor", "shape": ("4",)}, "missing string dtype"),
        ({"kind": "vector", "dtype": "float32"}, "missing string sequence shape"),
        ({"kind": "tensor", "shape": ("4",), "dtype": "float32", "expr": "M"}, "unsupported key"),
        ({"kind": "idx", "expr": 7}, "non-string expr"),
        ({"kind": "undef", "shape": ()}, "unsupported key"),
    ],
)
def test_type_contract_schema_rejects_invalid_records(record: dict, message: str) -> None:
    with pytest.raises(RuntimeError, match=message):
        validate_intrinsic_type_contract_record(record)


def test_bfloat16_is_a_dtype_name() -> None:
    import ml_dtypes

    assert tensor_type((16, 16), ml_dtypes.bfloat16).dtype == "bfloat16"
    assert Buffer[sym.M, sym.K, ml_dtypes.bfloat16].dtype == "bfloat16"


def test_buffer_annotation_forms() -> None:
    spec = Buffer[sym.M, sym.K, np.float16]
    assert spec.dimensions == (sym.M, sym.K) and spec.dtype == "float16"
    assert repr(spec) == "Buffer[M, K, float16]"
    assert Buffer[sym.M, sym.K].dtype is None
    assert Buffer[np.float16].dimensions == (np.float16,)  # a lone item is an extent, not a dtype
    assert Buffer[4, np.dtype("float32")].dtype == "float32"


def test_decorators_only_record_metadata() -> None:
    @kernel(work_shape=(sym.M,), group_shape=(32,), subgroup_size=32, literals={sym.M})
    def k(group, x: Buffer[sym.M, np.float32]) -> None:
        raise AssertionError("never executed at decoration time")

    assert k.__hc_kernel__.work_shape == (sym.M,)
    assert k.__hc_kernel__.literals == frozenset({sym.M})

    @kernel
    def bare(group) -> None:
        pass

    assert bare.__hc_kernel__.work_shape is None

    @kernel.func(scope=hc.WorkGroup)
    def helper(group):
        return 1

    assert helper.__hc_func__.scope is hc.WorkGroup and helper(None) == 1


def test_intrinsic_hooks_register() -> None:
    @kernel.intrinsic(scope=WorkItem, effects="pure", const_attrs={"arch"},
                      operand_types=(undef_type(),), result_types=vector_type((8,), np.float32))
    def op(group, *, arch):
        return 0

    meta = op.__hc_intrinsic__
    assert meta.scope is WorkItem and meta.effects == "pure" and meta.const_attrs == frozenset({"arch"})
    assert meta.result_types == (vector_type((8,), np.float32),)
    assert op.__hc_has_fallback__ is True and op.__hc_lowerings__ == {}

    @op.lower(target="nvidia-sm100a")
    def lowered(*args, **kwargs):
        return "umma"

    @op.verify
    def verified(sig, target):
        return None

    assert op.__hc_lowerings__ == {"nvidia-sm100a": lowered} and op.__hc_verify__ is verified

    @kernel.intrinsic(scope=WorkItem)
    def device_only(group):
        """Declared only."""

    assert device_only.__hc_has_fallback__ is False


def test_current_group_stub() -> None:
    group = hc.CurrentGroup(shape=(32, 2))
    assert group.size == 64
    with pytest.raises(NotImplementedError, match="runtime backends"):
        group.load()
    with pytest.raises(NotImplementedError):
        hc.WorkItem().local_id()


def test_symbols_evaluate_launch_shapes() -> None:
    m, n = sym.M, sym.N
    assert sym.M is sym["M"]
    shape = (ceil_div(m, 16) * 32, ceil_div(n, 16))
    assert [e.eval({"M": 17, "N": 19}) for e in shape] == [64, 2]
    assert [e.eval({m: 4095, n: 3073}) for e in shape] == [8192, 193]
    assert (m // 3 + m % 3 - 1).eval({"M": 10}) == 3
    assert {s.name for s in (m * n + 1).free_symbols()} == {"M", "N"}
    with pytest.raises(UnboundSymbolError, match="missing bindings for symbols: N"):
        shape[1].eval({"M": 1})
    with pytest.raises(TypeError):
        bool(m)


def test_bindings_detect_conflicts() -> None:
    bindings = Bindings()
    bindings.bind(sym.K, 18, source="a.shape[1]")
    with pytest.raises(SymbolConflictError, match="conflicting binding for K: 18 from 'a.shape\\[1\\]' vs 17"):
        bindings.bind(sym.K, 17, source="b.shape[0]")
    bindings.bind(sym.K, 18, source="c.shape[0]")  # agreeing re-binds are fine
    assert bindings.freeze().eval(sym.K * 2) == 36


def test_lazy_public_names() -> None:
    assert hc.sym is sym
    assert hc.symbols.ceil_div is ceil_div
    assert "compile" in dir(hc) and "cuda" in dir(hc)
    with pytest.raises(AttributeError):
        hc.no_such_name
