"""Serialised form of an intrinsic's operand/result type contract.

Same record schema as the reference (hc/_intrinsic_contracts.py:32-100; golden values in
its tests/test_intrinsic_contracts.py:17-32): a dict with a `kind` of "undef", "idx",
"tensor" or "vector"; shaped kinds carry `shape` (tuple of strings) and `dtype` (NumPy
name); "idx" may carry `expr` (string). The NVIDIA target validates the WMMA intrinsic of a
kernel against these records rather than against Python objects, so that contracts written
with either `hc` package compare equal.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence

TypeContractRecord = dict[str, object]

_FIELDS = {
    "undef": {"kind"},
    "idx": {"kind", "expr"},
    "tensor": {"kind", "shape", "dtype"},
    "vector": {"kind", "shape", "dtype"},
}


def serialize_intrinsic_type_spec(value: object) -> TypeContractRecord:
    """Type spec object -> record. Accepts specs of this package or duck-typed equivalents."""
    kind = type(value).__name__
    if value is None or kind == "UndefTypeSpec":
        return {"kind": "undef"}
    if kind in ("TensorTypeSpec", "VectorTypeSpec"):
        record: TypeContractRecord = {
            "kind": "tensor" if kind == "TensorTypeSpec" else "vector",
            "shape": tuple(str(extent) for extent in value.dimensions),  # type: ignore[attr-defined]
            "dtype": value.dtype,  # type: ignore[attr-defined]
        }
        return validate_intrinsic_type_contract_record(record)
    if kind == "IdxTypeSpec":
        record = {"kind": "idx"}
        if value.expr is not None:  # type: ignore[attr-defined]
            record["expr"] = str(value.expr)  # type: ignore[attr-defined]
        return validate_intrinsic_type_contract_record(record)
    raise RuntimeError(f"unsupported HC intrinsic type spec: {value!r}")


def validate_intrinsic_type_contract_record(value: Mapping[str, object]) -> TypeContractRecord:
    """Checks a record against the schema and returns a normalised copy."""
    kind = value.get("kind")
    if not isinstance(kind, str):
        raise RuntimeError(f"type contract record missing string kind: {value!r}")
    if kind not in _FIELDS:
        raise RuntimeError(f"type contract record has unsupported kind {kind!r}")
    unknown = sorted(repr(key) for key in set(value) - _FIELDS[kind])
    if unknown:
        raise RuntimeError(
            f"type contract record kind {kind!r} has unsupported key(s): {', '.join(unknown)}"
        )
    if kind in ("tensor", "vector"):
        shape = value.get("shape")
        if isinstance(shape, (str, bytes)) or not isinstance(shape, Sequence):
            raise RuntimeError(f"type contract record kind {kind!r} missing string sequence shape")
        if not all(isinstance(extent, str) for extent in shape):
            raise RuntimeError(f"type contract record kind {kind!r} has non-string shape entry")
        dtype = value.get("dtype")
        if not isinstance(dtype, str):
            raise RuntimeError(f"type contract record kind {kind!r} missing string dtype")
        return {"kind": kind, "shape": tuple(shape), "dtype": dtype}
    if kind == "idx":
        expr = value.get("expr")
        if expr is None:
            return {"kind": kind}
        if not isinstance(expr, str):
            raise RuntimeError("type contract record kind 'idx' has non-string expr")
        return {"kind": kind, "expr": expr}
    return {"kind": kind}
