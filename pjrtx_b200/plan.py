"""Executable-plan builder: the host-side mirror of the reference's compiler IR.

A `PlanBuilder` records values and instructions with the vocabulary of
`ir.ExecutablePlan` (reference: src/compiler/executable_plan.zig:9-147,
src/compiler/operation.zig:84-168) and hands them to the C ABI
(`pjrtx_b200_plan_*`). It plays the role the StableHLO importer plays in the
reference (src/compiler/stablehlo_operation_import.zig:22-456): one method per
StableHLO op, result shapes inferred the way StableHLO defines them.

The recorded plan is plain Python data (`values`, `instructions`), so the CPU
oracle can interpret exactly the same program without touching the library.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

try:  # bf16 host arrays
    import ml_dtypes

    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    ml_dtypes = None
    BF16 = None

# Element-type codes of the C ABI (include/pjrtx_b200.h).
U8, F32, PRED, S32, U32, S8, F16, BF16_CODE, C64, U16, U64, S64, S16, F64 = range(1, 15)

DTYPE_NAMES = {
    U8: "u8", F32: "f32", PRED: "pred", S32: "s32", U32: "u32", S8: "s8", F16: "f16",
    BF16_CODE: "bf16", C64: "c64", U16: "u16", U64: "u64", S64: "s64", S16: "s16", F64: "f64",
}
_NP = {
    U8: np.dtype(np.uint8), F32: np.dtype(np.float32), PRED: np.dtype(np.bool_), S32: np.dtype(np.int32),
    U32: np.dtype(np.uint32), S8: np.dtype(np.int8), F16: np.dtype(np.float16), U16: np.dtype(np.uint16),
    U64: np.dtype(np.uint64), S64: np.dtype(np.int64), S16: np.dtype(np.int16), F64: np.dtype(np.float64),
    C64: np.dtype(np.complex64),
}
if BF16 is not None:
    _NP[BF16_CODE] = BF16


def np_dtype(code: int) -> np.dtype:
    return _NP[code]


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    for code, npdt in _NP.items():
        if npdt == dt:
            return code
    raise TypeError(f"unsupported dtype {dt}")


ROLE_PARAMETER, ROLE_CONSTANT, ROLE_RESULT, ROLE_OUTPUT = 0, 1, 2, 3
REPLICATED, PARTITIONED, MANUAL = 0, 1, 2
EQ, NE, GE, GT, LE, LT = range(6)


@dataclasses.dataclass
class ValueDesc:
    id: int
    role: int
    dtype: int
    dims: Tuple[int, ...]


@dataclasses.dataclass
class Instr:
    kind: str
    inputs: List[int]
    outputs: List[int]
    attrs: Dict[str, List[int]]
    literal: Optional[bytes] = None
    target: Optional[str] = None


class Val:
    """A value of the plan being built; arithmetic operators emit instructions."""

    __slots__ = ("b", "id")

    def __init__(self, b: "PlanBuilder", vid: int):
        self.b = b
        self.id = vid

    @property
    def dtype(self) -> int:
        return self.b.values[self.id].dtype

    @property
    def dims(self) -> Tuple[int, ...]:
        return self.b.values[self.id].dims

    def __add__(self, o): return self.b.binary("add", self, o)
    def __sub__(self, o): return self.b.binary("subtract", self, o)
    def __mul__(self, o): return self.b.binary("multiply", self, o)
    def __truediv__(self, o): return self.b.binary("divide", self, o)
    def __neg__(self): return self.b.unary("negate", self)


BINARY = {
    "add", "subtract", "multiply", "divide", "maximum", "minimum", "power", "atan2", "remainder", "and_", "or_",
    "xor_", "shift_left", "shift_right_arithmetic", "shift_right_logical",
}
UNARY = {
    "negate", "exp", "expm1", "tanh", "sqrt", "rsqrt", "abs", "cbrt", "ceil", "floor", "log", "log1p", "logistic",
    "sine", "cosine", "not_", "sign", "round_nearest_afz", "round_nearest_even", "popcnt", "count_leading_zeros",
    "copy_arg0",
}
REDUCE = {"reduce_sum", "reduce_max", "reduce_min", "reduce_and", "reduce_or"}


class PlanBuilder:
    def __init__(self, num_replicas: int = 1, num_partitions: int = 1, device_assignment: Optional[Sequence[int]] = None):
        self.num_replicas = num_replicas
        self.num_partitions = num_partitions
        self.device_assignment = list(device_assignment) if device_assignment is not None else list(
            range(num_replicas * num_partitions))
        self.values: List[ValueDesc] = []
        self.instructions: List[Instr] = []
        self.parameter_ids: List[int] = []
        self.parameter_shardings: List[Tuple[int, str, int]] = []
        self.output_ids: List[int] = []
        self.output_shardings: List[Tuple[int, str, int]] = []
        self.donated: List[int] = []
        self.aliases: List[Tuple[int, int]] = []  # (output index, parameter index)

    # ---- values -----------------------------------------------------------
    def _value(self, role: int, dtype: int, dims: Sequence[int]) -> Val:
        vid = len(self.values)
        self.values.append(ValueDesc(vid, role, dtype, tuple(int(d) for d in dims)))
        return Val(self, vid)

    def _emit(self, kind, inputs, dtype, dims, attrs=None, literal=None, target=None, extra_outputs=()) -> Val:
        out = self._value(ROLE_RESULT, dtype, dims)
        outs = [out.id]
        for dt, dm in extra_outputs:
            outs.append(self._value(ROLE_RESULT, dt, dm).id)
        self.instructions.append(
            Instr(kind, [v.id for v in inputs], outs, {k: [int(x) for x in v] for k, v in (attrs or {}).items()}, literal,
                  target))
        return out

    def parameter(self, dtype: int, dims: Sequence[int], sharding: int = REPLICATED, split_dim: int = -1,
                  mesh: str = "") -> Val:
        v = self._value(ROLE_PARAMETER, dtype, dims)
        self.parameter_ids.append(v.id)
        self.parameter_shardings.append((sharding, mesh, split_dim))
        return v

    def constant(self, array, dtype: Optional[int] = None) -> Val:
        if dtype is not None:
            arr = np.asarray(array).astype(np_dtype(dtype))
        else:
            arr = np.asarray(array)
            dtype = dtype_code(arr.dtype)
        shape = arr.shape
        arr = np.ascontiguousarray(arr)  # promotes rank 0 to rank 1; the plan keeps the original shape
        v = self._value(ROLE_CONSTANT, dtype, shape)
        self.instructions.append(Instr("constant", [], [v.id], {}, arr.tobytes(), None))
        return v

    def scalar_like(self, x: Val, value) -> Val:
        """Rank-0 constant of x's type broadcast to x's shape (how JAX lowers `x * 0.5`)."""
        c = self.constant(np.asarray(value), x.dtype)
        return self.broadcast_in_dim(c, x.dims, []) if len(x.dims) else c

    # ---- elementwise --------------------------------------------------------
    def _coerce(self, a, b):
        if not isinstance(b, Val):
            b = self.scalar_like(a, b)
        if not isinstance(a, Val):
            a = self.scalar_like(b, a)
        return a, b

    def binary(self, kind: str, a, b) -> Val:
        a, b = self._coerce(a, b)
        assert kind in BINARY, kind
        assert a.dims == b.dims and a.dtype == b.dtype, (kind, a.dims, b.dims, a.dtype, b.dtype)
        return self._emit(kind, [a, b], a.dtype, a.dims)

    def unary(self, kind: str, a: Val) -> Val:
        assert kind in UNARY, kind
        return self._emit(kind, [a], a.dtype, a.dims)

    def is_finite(self, a: Val) -> Val:
        return self._emit("is_finite", [a], PRED, a.dims)

    def convert(self, a: Val, dtype: int) -> Val:
        return self._emit("convert", [a], dtype, a.dims)

    def bitcast_convert(self, a: Val, dtype: int) -> Val:
        return self._emit("bitcast_convert", [a], dtype, a.dims)

    def compare(self, a, b, direction: int) -> Val:
        a, b = self._coerce(a, b)
        assert a.dims == b.dims and a.dtype == b.dtype
        return self._emit("compare", [a, b], PRED, a.dims, {"compare_direction": [direction]})

    def select(self, pred: Val, on_true, on_false) -> Val:
        on_true, on_false = self._coerce(on_true, on_false)
        assert on_true.dims == on_false.dims and on_true.dtype == on_false.dtype
        return self._emit("select", [pred, on_true, on_false], on_true.dtype, on_true.dims)

    def clamp(self, lo: Val, x: Val, hi: Val) -> Val:
        return self._emit("clamp", [lo, x, hi], x.dtype, x.dims)

    # ---- views / structural -------------------------------------------------
    def reshape(self, a: Val, dims: Sequence[int]) -> Val:
        assert int(np.prod(a.dims, dtype=np.int64)) == int(np.prod(dims, dtype=np.int64)), (a.dims, dims)
        return self._emit("reshape", [a], a.dtype, dims, {"dims": dims})

    def transpose(self, a: Val, perm: Sequence[int]) -> Val:
        dims = [a.dims[p] for p in perm]
        return self._emit("transpose", [a], a.dtype, dims, {"permutation": perm, "dims": dims})

    def broadcast_in_dim(self, a: Val, dims: Sequence[int], broadcast_dimensions: Sequence[int]) -> Val:
        assert len(broadcast_dimensions) == len(a.dims)
        for k, d in enumerate(broadcast_dimensions):
            assert a.dims[k] in (1, dims[d]), (a.dims, dims, broadcast_dimensions)
        return self._emit("broadcast_in_dim", [a], a.dtype, dims, {"broadcast_dimensions": broadcast_dimensions, "dims": dims})

    def slice(self, a: Val, start: Sequence[int], limit: Sequence[int], strides: Optional[Sequence[int]] = None) -> Val:
        strides = list(strides) if strides is not None else [1] * len(start)
        dims = [max(0, -(-(l - s) // st)) for s, l, st in zip(start, limit, strides)]
        return self._emit("slice", [a], a.dtype, dims,
                          {"start_indices": start, "limit_indices": limit, "strides": strides, "dims": dims})

    def reverse(self, a: Val, dimensions: Sequence[int]) -> Val:
        return self._emit("reverse", [a], a.dtype, a.dims, {"dimensions": dimensions, "dims": a.dims})

    def concatenate(self, parts: Sequence[Val], dimension: int) -> Val:
        dims = list(parts[0].dims)
        dims[dimension] = sum(p.dims[dimension] for p in parts)
        return self._emit("concatenate", list(parts), parts[0].dtype, dims, {"dimension": [dimension], "dims": dims})

    def pad(self, a: Val, padding_value: Val, low: Sequence[int], high: Sequence[int],
            interior: Optional[Sequence[int]] = None) -> Val:
        """stablehlo.pad: edge padding (negative = cropping) and interior padding with a scalar value."""
        interior = list(interior) if interior is not None else [0] * len(a.dims)
        dims = []
        for d, lo, hi, gap in zip(a.dims, low, high, interior):
            span = 0 if d == 0 else (d - 1) * (gap + 1) + 1
            dims.append(max(0, lo + span + hi))
        return self._emit("pad", [a, padding_value], a.dtype, dims,
                          {"edge_padding_low": list(low), "edge_padding_high": list(high), "interior_padding": interior})

    def iota(self, dtype: int, dims: Sequence[int], iota_dimension: int) -> Val:
        return self._emit("iota", [], dtype, dims, {"iota_dimension": [iota_dimension], "dims": dims})

    def dynamic_slice(self, a: Val, starts: Sequence[Val], slice_sizes: Sequence[int]) -> Val:
        assert len(starts) == len(a.dims)
        return self._emit("dynamic_slice", [a, *starts], a.dtype, slice_sizes, {"slice_sizes": slice_sizes, "dims": slice_sizes})

    def dynamic_update_slice(self, a: Val, update: Val, starts: Sequence[Val]) -> Val:
        assert len(starts) == len(a.dims) and update.dtype == a.dtype
        return self._emit("dynamic_update_slice", [a, update, *starts], a.dtype, a.dims, {"dims": a.dims})

    def gather_rows(self, table: Val, ids: Val) -> Val:
        """Embedding lookup `table[ids]` as the StableHLO gather JAX emits for `jnp.take(table, ids, axis=0)`."""
        batch_rank = len(ids.dims)
        dims = list(ids.dims) + list(table.dims[1:])
        return self._emit("gather", [table, ids], table.dtype, dims, {
            "offset_dims": list(range(batch_rank, batch_rank + len(table.dims) - 1)),
            "collapsed_slice_dims": [0], "start_index_map": [0], "index_vector_dim": [batch_rank],
            "slice_sizes": [1] + list(table.dims[1:]), "dims": dims,
        })

    # ---- contractions / reductions -------------------------------------------
    def dot_general(self, a: Val, b: Val, lhs_contract: Sequence[int], rhs_contract: Sequence[int],
                    lhs_batch: Sequence[int] = (), rhs_batch: Sequence[int] = ()) -> Val:
        dims = [a.dims[d] for d in lhs_batch]
        dims += [a.dims[d] for d in range(len(a.dims)) if d not in lhs_batch and d not in lhs_contract]
        dims += [b.dims[d] for d in range(len(b.dims)) if d not in rhs_batch and d not in rhs_contract]
        return self._emit("dot_general", [a, b], a.dtype, dims, {
            "lhs_batch_dimensions": lhs_batch, "rhs_batch_dimensions": rhs_batch,
            "lhs_contracting_dimensions": lhs_contract, "rhs_contracting_dimensions": rhs_contract, "dims": dims})

    def matmul(self, a: Val, b: Val) -> Val:
        return self.dot_general(a, b, [len(a.dims) - 1], [0])

    def reduce(self, kind: str, a: Val, dimensions: Sequence[int]) -> Val:
        assert kind in REDUCE
        dims = [d for k, d in enumerate(a.dims) if k not in dimensions]
        return self._emit(kind, [a], a.dtype, dims, {"reduce_dimensions": dimensions, "dims": dims})

    def reduce_max_with_indices(self, values: Val, indices: Val, dimensions: Sequence[int]) -> Tuple[Val, Val]:
        """Two-operand reduce whose body is compare+select: max value and the smallest index holding it
        (reference: src/compiler/stablehlo_operation_attrs.zig:222-246, src/backend/mlx_metal/api.cc:4046-4170)."""
        dims = [d for k, d in enumerate(values.dims) if k not in dimensions]
        out = self._emit("reduce_max", [values, indices], values.dtype, dims, {"reduce_dimensions": dimensions, "dims": dims},
                         extra_outputs=[(indices.dtype, dims)])
        return out, Val(self, out.id + 1)

    def argmax(self, a: Val, axis: int, index_dtype: int = S32) -> Tuple[Val, Val]:
        idx = self.iota(index_dtype, a.dims, axis)
        return self.reduce_max_with_indices(a, idx, [axis])

    # ---- calls / collectives -------------------------------------------------
    def custom_call(self, target: str, inputs: Sequence[Val], dtype: int, dims: Sequence[int]) -> Val:
        return self._emit("custom_call", list(inputs), dtype, dims, {"dims": dims}, target=target)

    def all_reduce(self, a: Val) -> Val:
        return self._emit("all_reduce", [a], a.dtype, a.dims, {"dims": a.dims})

    # ---- outputs --------------------------------------------------------------
    def set_outputs(self, outputs: Sequence[Val], donate: Optional[Dict[int, int]] = None,
                    shardings: Optional[Sequence[Tuple[int, str, int]]] = None) -> None:
        """`donate` maps output position -> parameter position whose storage the output may take."""
        self.output_ids = [v.id for v in outputs]
        self.output_shardings = list(shardings) if shardings is not None else [(REPLICATED, "", -1)] * len(outputs)
        self.aliases = sorted((donate or {}).items())
        self.donated = sorted({p for _, p in self.aliases})

    @classmethod
    def from_description(cls, d: dict) -> "PlanBuilder":
        """Rebuilds a builder from `pjrtx_b200_plan_describe` JSON."""
        b = cls(d["num_replicas"], d["num_partitions"])
        for i, v in enumerate(d["values"]):
            b.values.append(ValueDesc(i, v["role"], v["dtype"], tuple(v["dims"])))
            if v["role"] == ROLE_PARAMETER:
                b.parameter_ids.append(i)
        for ins in d["instructions"]:
            kind = ins["kind"]
            lit = bytes.fromhex(ins["literal"]) if "literal" in ins else None
            b.instructions.append(Instr(kind, list(ins["inputs"]), list(ins["outputs"]), {k: list(v) for k, v in ins["attrs"].items()},
                                        lit, ins.get("target")))
        b.parameter_shardings = [(s["kind"], s["mesh"], s["split_dim"]) for s in d["parameter_shardings"]]
        b.output_ids = list(d["outputs"])
        b.output_shardings = [(s["kind"], s["mesh"], s["split_dim"]) for s in d["output_shardings"]]
        b.donated = list(d["donated"])
        b.aliases = [tuple(a) for a in d["aliases"]]
        return b

    # ---- lowering to the C ABI --------------------------------------------------
    def build(self, lib) -> "ctypes.c_void_p":
        """Creates the C plan object; the caller owns it (pjrtx_b200_plan_destroy)."""
        import ctypes

        from .backend import Attribute

        assign = (ctypes.c_int32 * len(self.device_assignment))(*self.device_assignment)
        plan = lib.pjrtx_b200_plan_create(self.num_replicas, self.num_partitions, assign, len(self.device_assignment))
        if not plan:
            raise RuntimeError("plan_create failed")
        for v in self.values:
            dims = (ctypes.c_int64 * len(v.dims))(*v.dims)
            vid = lib.pjrtx_b200_plan_add_value(plan, v.role, v.dtype, dims, len(v.dims))
            assert vid == v.id
        for ins in self.instructions:
            ins_in = (ctypes.c_uint32 * len(ins.inputs))(*ins.inputs)
            ins_out = (ctypes.c_uint32 * len(ins.outputs))(*ins.outputs)
            keep = []
            attrs = (Attribute * len(ins.attrs))()
            for k, (name, vals) in enumerate(ins.attrs.items()):
                arr = (ctypes.c_int64 * len(vals))(*vals)
                keep.append(arr)
                attrs[k].name = name.encode()
                attrs[k].values = ctypes.cast(arr, ctypes.POINTER(ctypes.c_int64))
                attrs[k].count = len(vals)
            lit = ins.literal
            ok = lib.pjrtx_b200_plan_add_instruction(
                plan, ins.kind.encode(), ins_in, len(ins.inputs), ins_out, len(ins.outputs), attrs, len(ins.attrs), lit,
                len(lit) if lit else 0, ins.target.encode() if ins.target else None)
            if not ok:
                msg = lib.pjrtx_b200_last_error().decode()
                lib.pjrtx_b200_plan_destroy(plan)
                raise RuntimeError(msg)
        outs = (ctypes.c_uint32 * len(self.output_ids))(*self.output_ids)
        lib.pjrtx_b200_plan_set_outputs(plan, outs, len(self.output_ids))
        for k, (kind, mesh, split) in enumerate(self.parameter_shardings):
            lib.pjrtx_b200_plan_set_parameter_sharding(plan, k, kind, mesh.encode(), split)
        for k, (kind, mesh, split) in enumerate(self.output_shardings):
            lib.pjrtx_b200_plan_set_output_sharding(plan, k, kind, mesh.encode(), split)
        don = (ctypes.c_uint32 * len(self.donated))(*self.donated)
        ao = (ctypes.c_uint32 * len(self.aliases))(*[o for o, _ in self.aliases])
        ap = (ctypes.c_uint32 * len(self.aliases))(*[p for _, p in self.aliases])
        lib.pjrtx_b200_plan_set_donation(plan, don, len(self.donated), ao, ap, len(self.aliases))
        return plan
