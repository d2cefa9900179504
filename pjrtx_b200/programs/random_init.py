"""Seeded random tensors produced on the device by an ordinary executable plan.

Benchmarks need tens of gigabytes of random-init weights; generating them on the host would dominate the run.
The generator is a counter-based hash written with plan ops only (iota, integer multiply / xor / shift, convert,
log, sqrt, cosine), so the backend itself materialises the tensors and the CPU oracle can reproduce them.

Element (r, c) of a tensor whose full width is `full_cols` uses counter `(row_offset + r) * full_cols + col_offset + c`
mixed with a per-tensor seed; a tensor-parallel shard therefore holds exactly its slice of the full tensor.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

from .. import plan as P
from ..plan import PlanBuilder, Val

_M1, _M2 = 0x85EBCA6B, 0xC2B2AE35  # murmur3 finaliser multipliers


def _mix(b: PlanBuilder, h: Val) -> Val:
    u = lambda v: b.scalar_like(h, np.uint32(v))
    h = b.binary("xor_", h, b.binary("shift_right_logical", h, u(16)))
    h = h * u(_M1)
    h = b.binary("xor_", h, b.binary("shift_right_logical", h, u(13)))
    h = h * u(_M2)
    return b.binary("xor_", h, b.binary("shift_right_logical", h, u(16)))


def _counter(b: PlanBuilder, rows: int, cols: int, full_cols: int, row_offset: int, col_offset: int, seed: Val) -> Val:
    r = b.iota(P.U32, [rows, cols], 0)
    c = b.iota(P.U32, [rows, cols], 1)
    ctr = (r + np.uint32(row_offset)) * np.uint32(full_cols & 0xFFFFFFFF) + (c + np.uint32(col_offset))
    return b.binary("xor_", ctr, b.broadcast_in_dim(seed, [rows, cols], []))


def build_normal(rows: int, cols: int, dtype: int, std: float, mean: float = 0.0, full_cols: int = 0, row_offset: int = 0,
                 col_offset: int = 0) -> PlanBuilder:
    """(seed: u32[]) -> [rows, cols] of N(mean, std) in `dtype` (Box-Muller on two hashed uniforms)."""
    b = PlanBuilder()
    seed = b.parameter(P.U32, [])
    ctr = _counter(b, rows, cols, full_cols or cols, row_offset, col_offset, seed)
    h1 = _mix(b, ctr)
    h2 = _mix(b, b.binary("xor_", h1, b.scalar_like(h1, np.uint32(0x9E3779B9))))
    inv = np.float32(1.0 / (1 << 24))
    u1 = (b.convert(b.binary("shift_right_logical", h1, b.scalar_like(h1, np.uint32(8))), P.F32) + np.float32(1.0)) * inv
    u2 = b.convert(b.binary("shift_right_logical", h2, b.scalar_like(h2, np.uint32(8))), P.F32) * inv
    radius = b.unary("sqrt", b.unary("log", u1) * np.float32(-2.0))
    z = radius * b.unary("cosine", u2 * np.float32(2.0 * np.pi))
    out = z * np.float32(std)
    if mean:
        out = out + np.float32(mean)
    b.set_outputs([b.convert(out, dtype) if dtype != P.F32 else out])
    return b


def build_uniform_int8(rows: int, cols: int, full_cols: int = 0, row_offset: int = 0, col_offset: int = 0) -> PlanBuilder:
    """(seed: u32[]) -> s8 [rows, cols] uniform in {-127..127}."""
    b = PlanBuilder()
    seed = b.parameter(P.U32, [])
    h = _mix(b, _counter(b, rows, cols, full_cols or cols, row_offset, col_offset, seed))
    v = b.binary("remainder", b.binary("shift_right_logical", h, b.scalar_like(h, np.uint32(8))), b.scalar_like(h, np.uint32(255)))
    b.set_outputs([b.convert(b.convert(v, P.S32) - np.int32(127), P.S8)])
    return b


def build_uniform(rows: int, cols: int, dtype: int, lo: float, hi: float, full_cols: int = 0, row_offset: int = 0,
                  col_offset: int = 0) -> PlanBuilder:
    b = PlanBuilder()
    seed = b.parameter(P.U32, [])
    h = _mix(b, _counter(b, rows, cols, full_cols or cols, row_offset, col_offset, seed))
    u = b.convert(b.binary("shift_right_logical", h, b.scalar_like(h, np.uint32(8))), P.F32) * np.float32(1.0 / (1 << 24))
    out = u * np.float32(hi - lo) + np.float32(lo)
    b.set_outputs([b.convert(out, dtype) if dtype != P.F32 else out])
    return b


def tensor_seed(seed: int, index: int) -> np.ndarray:
    return np.array((seed * 0x9E3779B1 + index * 0x85EBCA77 + 0x1234567) & 0xFFFFFFFF, np.uint32)
