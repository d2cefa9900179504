"""CPU oracle: a NumPy interpreter for executable plans. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module; the product path (pjrtx_b200/) never does.

What it restates. The reference has no CPU execution path; its own oracle is
`jax.jit(fn, backend="cpu")` (src/plugin/jax/jax_op_suite.py:98-109), and the
arithmetic of its device path lives in MLX (ml-explore/mlx 0.31.2, not in the
reference tree) behind the call sites of src/backend/mlx_metal/api.cc. This
interpreter therefore follows StableHLO op semantics the way XLA's CPU backend
evaluates them: every instruction is computed in float64 (floats) or the exact
integer type and rounded to the storage dtype at the op boundary, so bf16/f16
programs round once per op. Per-op anchors in the reference:
  elementwise       api.cc:1311-1499 (binary/unary tables), :1704-1723 (compare/select)
  convert           api.cc:907-935
  reduce            api.cc:3982-4044; generated kernel executable_metal_graph_reduction.zig:39-54
  max-with-index    api.cc:4046-4170 (max, then smallest index where value == max or both NaN)
  dot_general       api.cc:3349-3498; generated kernel metal_graph_dot.zig:50-63 (f32 accumulate)
  gather (take)     api.cc:2813-2859
  dynamic slices    api.cc:2552-2635 (start indices clamped)
  attention         api.cc:4929-5043 with mask api.cc:937-950 (key <= token + query), scale 1/sqrt(head_dim)

Parity status: pinned against every literal known-answer vector the reference's
tests hold for these ops (tests/test_oracle_golden.py lists them with file:line)
and against fixtures produced by the reference's own NumPy llama-like reference
(tests/golden/). Accumulation order inside MLX matmul/reduce is not pinned by
any reference test below its 1e-4 / 1e-2 / 2e-4 tolerances.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from pjrtx_b200 import plan as P


def _round_to(x: np.ndarray, code: int) -> np.ndarray:
    """Rounds a float64 / wide-int result to the storage dtype (one rounding per op)."""
    dt = P.np_dtype(code)
    if code in (P.F32, P.F16, P.BF16_CODE):
        with np.errstate(over="ignore", invalid="ignore"):
            if code == P.BF16_CODE:
                return np.asarray(x, dtype=np.float32).astype(dt)
            return np.asarray(x).astype(dt)
    if code == P.PRED:
        return np.asarray(x).astype(np.bool_)
    return np.asarray(x).astype(dt)


def _f64(x: np.ndarray) -> np.ndarray:
    return np.asarray(x).astype(np.float64)


def _is_float(code: int) -> bool:
    return code in (P.F32, P.F16, P.BF16_CODE)


def _float_to_int(x: np.ndarray, code: int) -> np.ndarray:
    dt = P.np_dtype(code)
    info = np.iinfo(dt)
    v = np.nan_to_num(_f64(x), nan=0.0, posinf=float(info.max), neginf=float(info.min))
    v = np.trunc(v)
    v = np.clip(v, float(info.min), float(info.max))
    # float(info.max) may round up; clip again in integer space
    out = np.where(v >= float(info.max), info.max, np.where(v <= float(info.min), info.min, v.astype(np.int64 if info.min < 0 else np.uint64)))
    return out.astype(dt)


def _binary(kind: str, a: np.ndarray, b: np.ndarray, code: int) -> np.ndarray:
    if _is_float(code):
        x, y = _f64(a), _f64(b)
        with np.errstate(all="ignore"):
            if kind == "add": r = x + y
            elif kind == "subtract": r = x - y
            elif kind == "multiply": r = x * y
            elif kind == "divide": r = x / y
            elif kind == "maximum": r = np.where(np.isnan(x) | np.isnan(y), np.nan, np.maximum(x, y))
            elif kind == "minimum": r = np.where(np.isnan(x) | np.isnan(y), np.nan, np.minimum(x, y))
            elif kind == "power": r = np.power(x, y)
            elif kind == "atan2": r = np.arctan2(x, y)
            elif kind == "remainder": r = np.fmod(x, y)
            else: raise NotImplementedError(kind)
        return _round_to(r, code)
    if code == P.PRED:
        if kind in ("and_", "multiply", "minimum"): return a & b
        if kind in ("or_", "add", "maximum"): return a | b
        if kind == "xor_": return a ^ b
        raise NotImplementedError(kind)
    dt = P.np_dtype(code)
    bits = dt.itemsize * 8
    with np.errstate(all="ignore"):
        if kind == "add": return (a + b).astype(dt)
        if kind == "subtract": return (a - b).astype(dt)
        if kind == "multiply": return (a * b).astype(dt)
        if kind == "maximum": return np.maximum(a, b)
        if kind == "minimum": return np.minimum(a, b)
        if kind == "and_": return a & b
        if kind == "or_": return a | b
        if kind == "xor_": return a ^ b
        if kind in ("divide", "remainder"):
            # C semantics: truncation toward zero; x/0 = -1 (all ones), x%0 = x.
            ai, bi = a.astype(object), b.astype(object)
            out = np.empty(a.shape, dtype=object)
            for idx in np.ndindex(a.shape):
                p, q = int(ai[idx]), int(bi[idx])
                if q == 0:
                    out[idx] = -1 if kind == "divide" else p
                else:
                    t = abs(p) // abs(q)
                    t = t if (p >= 0) == (q >= 0) else -t
                    out[idx] = t if kind == "divide" else p - t * q
            mask = (1 << bits) - 1
            return np.vectorize(lambda v: v & mask, otypes=[object])(out).astype(np.uint64).astype(
                np.dtype(f"uint{bits}")).view(dt) if a.size else a
        if kind in ("shift_left", "shift_right_logical", "shift_right_arithmetic"):
            sh = b.astype(np.int64)
            big = (sh >= bits) | (sh < 0)
            shc = np.where(big, 0, sh).astype(np.uint64)
            if kind == "shift_left":
                r = (a.astype(np.uint64) << shc).astype(np.dtype(f"uint{bits}")).view(dt) if dt.kind == "i" else (a.astype(np.uint64) << shc).astype(dt)
                return np.where(big, np.zeros_like(a), r).astype(dt)
            if kind == "shift_right_logical":
                u = a.view(np.dtype(f"uint{bits}")) if dt.kind == "i" else a
                r = (u.astype(np.uint64) >> shc).astype(np.dtype(f"uint{bits}"))
                r = r.view(dt) if dt.kind == "i" else r.astype(dt)
                return np.where(big, np.zeros_like(a), r).astype(dt)
            r = (a.astype(np.int64) >> shc.astype(np.int64)).astype(dt)
            fill = np.where(a < 0, -1, 0).astype(dt) if dt.kind == "i" else np.zeros_like(a)
            return np.where(big, fill, r).astype(dt)
        if kind == "power":
            out = np.empty(a.shape, dtype=object)
            for idx in np.ndindex(a.shape):
                p, q = int(a[idx]), int(b[idx])
                out[idx] = (1 if p == 1 else (-1 if q % 2 else 1) if p == -1 else 0) if q < 0 else pow(p, q, 1 << 64)
            mask = (1 << bits) - 1
            return np.vectorize(lambda v: v & mask, otypes=[object])(out).astype(np.uint64).astype(np.dtype(f"uint{bits}")).view(dt)
    raise NotImplementedError(kind)


def _unary(kind: str, a: np.ndarray, code: int) -> np.ndarray:
    if kind == "copy_arg0":
        return a
    if _is_float(code):
        x = _f64(a)
        with np.errstate(all="ignore"):
            if kind == "negate": r = -x
            elif kind == "exp": r = np.exp(x)
            elif kind == "expm1": r = np.expm1(x)
            elif kind == "tanh": r = np.tanh(x)
            elif kind == "sqrt": r = np.sqrt(x)
            elif kind == "rsqrt": r = 1.0 / np.sqrt(x)
            elif kind == "abs": r = np.abs(x)
            elif kind == "cbrt": r = np.cbrt(x)
            elif kind == "ceil": r = np.ceil(x)
            elif kind == "floor": r = np.floor(x)
            elif kind == "log": r = np.log(x)
            elif kind == "log1p": r = np.log1p(x)
            elif kind == "logistic": r = 1.0 / (1.0 + np.exp(-x))
            elif kind == "sine": r = np.sin(x)
            elif kind == "cosine": r = np.cos(x)
            elif kind == "sign": r = np.sign(x)
            elif kind == "round_nearest_even": r = np.rint(x)
            elif kind == "round_nearest_afz": r = np.sign(x) * np.floor(np.abs(x) + 0.5)
            else: raise NotImplementedError(kind)
        return _round_to(r, code)
    dt = P.np_dtype(code)
    if kind == "not_":
        return ~a if code != P.PRED else np.logical_not(a)
    if kind == "negate":
        with np.errstate(all="ignore"):
            return (0 - a).astype(dt)
    if kind == "abs":
        with np.errstate(all="ignore"):
            return np.abs(a).astype(dt)
    if kind == "sign":
        return np.sign(a).astype(dt)
    bits = dt.itemsize * 8
    if kind == "popcnt":
        u = a.view(np.dtype(f"uint{bits}")) if dt.kind == "i" else a
        return np.vectorize(lambda v: bin(int(v)).count("1"), otypes=[np.int64])(u).astype(dt) if a.size else a
    if kind == "count_leading_zeros":
        u = a.view(np.dtype(f"uint{bits}")) if dt.kind == "i" else a
        return np.vectorize(lambda v: bits - int(v).bit_length(), otypes=[np.int64])(u).astype(dt) if a.size else a
    raise NotImplementedError(kind)


def _argmax_pair(values: np.ndarray, indices: np.ndarray, dims: Sequence[int]):
    """max over `dims`; among equal maxima (NaN counts as the maximum) the smallest index operand wins."""
    keep = [d for d in range(values.ndim) if d not in dims]
    perm = keep + list(dims)
    v = np.transpose(values, perm).reshape([values.shape[d] for d in keep] + [-1])
    i = np.transpose(indices, perm).reshape(v.shape)
    vf = _f64(v) if v.dtype.kind == "f" or v.dtype.itemsize == 2 and v.dtype.kind == "V" else v
    vf = np.asarray(v).astype(np.float64) if np.asarray(v).dtype.kind not in "iu" else np.asarray(v)
    if vf.dtype.kind == "f":
        has_nan = np.isnan(vf).any(axis=-1, keepdims=True)
        mx = np.where(has_nan, np.nan, np.max(np.where(np.isnan(vf), -np.inf, vf), axis=-1, keepdims=True))
        hit = np.where(has_nan, np.isnan(vf), vf == mx)
    else:
        mx = np.max(vf, axis=-1, keepdims=True)
        hit = vf == mx
    big = np.iinfo(i.dtype).max
    idx = np.min(np.where(hit, i, big), axis=-1)
    val = np.squeeze(mx, axis=-1)
    return val, idx.astype(i.dtype)


def _dot_general(a, b, ins) -> np.ndarray:
    """float64 contraction: batch axes first, then lhs free axes, then rhs free axes (StableHLO's result order).
    Operands are brought to [batch..., M, K] x [batch..., K, N] and multiplied with the float64 BLAS."""
    lb, rb = list(ins.attrs.get("lhs_batch_dimensions", [])), list(ins.attrs.get("rhs_batch_dimensions", []))
    lc, rc = list(ins.attrs["lhs_contracting_dimensions"]), list(ins.attrs["rhs_contracting_dimensions"])
    lf = [d for d in range(a.ndim) if d not in lb and d not in lc]
    rf = [d for d in range(b.ndim) if d not in rb and d not in rc]
    batch_shape = [a.shape[d] for d in lb]
    m_shape, n_shape = [a.shape[d] for d in lf], [b.shape[d] for d in rf]
    k = int(np.prod([a.shape[d] for d in lc], dtype=np.int64))
    m, n = int(np.prod(m_shape, dtype=np.int64)), int(np.prod(n_shape, dtype=np.int64))
    at = np.transpose(_f64(a), lb + lf + lc).reshape(batch_shape + [m, k])
    bt = np.transpose(_f64(b), rb + rc + rf).reshape(batch_shape + [k, n])
    return np.matmul(at, bt).reshape(batch_shape + m_shape + n_shape)


def _sdpa(q, k, v, token) -> np.ndarray:
    has_batch = q.ndim == 4
    q4 = _f64(q) if has_batch else _f64(q)[None]
    k4 = _f64(k) if has_batch else _f64(k)[None]
    v4 = _f64(v) if has_batch else _f64(v)[None]
    B, Q, H, D = q4.shape
    S, G = k4.shape[1], k4.shape[2]
    rep = H // G
    out = np.zeros_like(q4)
    t = int(np.asarray(token).reshape(()))
    scale = 1.0 / np.sqrt(np.float32(D)).astype(np.float64)
    for qi in range(Q):
        limit = min(t + qi, S - 1)
        if limit < 0:
            continue
        for h in range(H):
            g = h // rep
            s = np.einsum("bd,bkd->bk", q4[:, qi, h], k4[:, : limit + 1, g]) * scale
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p = p / p.sum(axis=-1, keepdims=True)
            out[:, qi, h] = np.einsum("bk,bkd->bd", p, v4[:, : limit + 1, g])
    return out if has_batch else out[0]


def _dot_general_f32(a, b, ins, cache, key):
    """BLAS path for the timed CPU baseline: operands widened to f32 (the widened copy of a parameter is cached
    across calls, as a CPU backend would keep its weights), f32 accumulate, any layout via einsum."""
    lb, rb = ins.attrs.get("lhs_batch_dimensions", []), ins.attrs.get("rhs_batch_dimensions", [])
    lc, rc = ins.attrs["lhs_contracting_dimensions"], ins.attrs["rhs_contracting_dimensions"]
    bf = cache.get(key) if cache is not None and key is not None else None
    if bf is None:
        bf = np.asarray(b).astype(np.float32)
        if cache is not None and key is not None:
            cache[key] = bf
    af = np.asarray(a).astype(np.float32)
    if not lb and a.ndim == 2 and b.ndim == 2 and lc == [1] and rc == [0]:
        return af @ bf
    lf = [d for d in range(a.ndim) if d not in lb and d not in lc]
    rf = [d for d in range(b.ndim) if d not in rb and d not in rc]
    letters = iter("abcdefghijklmnopqrstuvwxyz")
    la, lbl, out = [None] * a.ndim, [None] * b.ndim, []
    for x, y in zip(lb, rb):
        c = next(letters); la[x] = c; lbl[y] = c; out.append(c)
    for x, y in zip(lc, rc):
        c = next(letters); la[x] = c; lbl[y] = c
    for x in lf:
        c = next(letters); la[x] = c; out.append(c)
    for y in rf:
        c = next(letters); lbl[y] = c; out.append(c)
    return np.einsum(f"{''.join(la)},{''.join(lbl)}->{''.join(out)}", af, bf, optimize=True)


def run_plan(builder: P.PlanBuilder, arguments: Sequence[np.ndarray], all_reduce=None, fast_dot: bool = False,
             weight_cache: Dict[int, np.ndarray] = None, all_gather=None) -> List[np.ndarray]:
    """Evaluates the recorded plan on host arrays and returns its outputs (storage dtypes).

    `fast_dot` switches contractions from float64 einsum to float32 BLAS (used only when the oracle is timed as the
    CPU baseline); `weight_cache` keeps widened copies of parameters between calls."""
    env: Dict[int, np.ndarray] = {}
    assert len(arguments) == len(builder.parameter_ids)
    # Intermediates are dropped after their last reader so that full-width programs fit in host memory.
    last_use: Dict[int, int] = {}
    for index, ins in enumerate(builder.instructions):
        for i in ins.inputs:
            last_use[i] = index
    keep = set(builder.output_ids)

    def release(index, ins):
        for i in ins.inputs:
            if last_use.get(i) == index and i not in keep:
                env.pop(i, None)

    for vid, arr in zip(builder.parameter_ids, arguments):
        desc = builder.values[vid]
        a = np.asarray(arr)
        assert tuple(a.shape) == desc.dims and a.dtype == P.np_dtype(desc.dtype), (vid, a.shape, desc.dims, a.dtype)
        env[vid] = a
    for index, ins in enumerate(builder.instructions):
        out_desc = builder.values[ins.outputs[0]]
        code, dims = out_desc.dtype, out_desc.dims
        x = [env[i] for i in ins.inputs]
        k = ins.kind
        if k == "constant":
            r = np.frombuffer(ins.literal, dtype=P.np_dtype(code)).reshape(dims).copy()
        elif k in P.BINARY:
            r = _binary(k, x[0], x[1], code)
        elif k in P.UNARY:
            r = _unary(k, x[0], code)
        elif k == "is_finite":
            r = np.isfinite(_f64(x[0]))
        elif k == "convert":
            src = builder.values[ins.inputs[0]].dtype
            if _is_float(code):
                r = _round_to(_f64(x[0]) if src != P.PRED else x[0].astype(np.float64), code)
            elif code == P.PRED:
                r = x[0] != 0
            elif _is_float(src):
                r = _float_to_int(x[0], code)
            else:
                r = x[0].astype(P.np_dtype(code))
        elif k == "bitcast_convert":
            r = np.ascontiguousarray(x[0]).view(P.np_dtype(code)).reshape(dims)
        elif k == "compare":
            d = ins.attrs["compare_direction"][0]
            a, b = (_f64(x[0]), _f64(x[1])) if _is_float(builder.values[ins.inputs[0]].dtype) else (x[0], x[1])
            with np.errstate(invalid="ignore"):
                r = [a == b, a != b, a >= b, a > b, a <= b, a < b][d]
        elif k == "select":
            r = np.where(x[0], x[1], x[2]).astype(P.np_dtype(code))
        elif k == "clamp":
            if _is_float(code):
                lo, v, hi = _f64(x[0]), _f64(x[1]), _f64(x[2])
                r = _round_to(np.where(np.isnan(v) | np.isnan(lo) | np.isnan(hi), np.nan, np.minimum(np.maximum(v, lo), hi)), code)
            else:
                r = np.minimum(np.maximum(x[1], x[0]), x[2]).astype(P.np_dtype(code))
        elif k == "reshape":
            r = x[0].reshape(dims)
        elif k == "transpose":
            r = np.transpose(x[0], ins.attrs["permutation"])
        elif k == "broadcast_in_dim":
            bd = ins.attrs["broadcast_dimensions"]
            shape = [1] * len(dims)
            for src_axis, dst_axis in enumerate(bd):
                shape[dst_axis] = x[0].shape[src_axis]
            r = np.broadcast_to(x[0].reshape(shape), dims)
        elif k == "slice":
            st, li, sr = ins.attrs["start_indices"], ins.attrs["limit_indices"], ins.attrs["strides"]
            r = x[0][tuple(slice(s, l, t) for s, l, t in zip(st, li, sr))]
        elif k == "reverse":
            r = np.flip(x[0], axis=tuple(ins.attrs["dimensions"]))
        elif k == "concatenate":
            r = np.concatenate(x, axis=ins.attrs["dimension"][0])
        elif k == "pad":
            # stablehlo.pad: interior padding first, then edge padding; negative edge padding removes elements.
            lo, hi = ins.attrs["edge_padding_low"], ins.attrs["edge_padding_high"]
            gaps = ins.attrs.get("interior_padding") or [0] * x[0].ndim
            src = x[0]
            spread_shape = [0 if n == 0 else (n - 1) * (g + 1) + 1 for n, g in zip(src.shape, gaps)]
            spread = np.full(spread_shape, np.asarray(x[1]).reshape(()), dtype=src.dtype)
            spread[tuple(slice(None, None, g + 1) for g in gaps)] = src
            r = np.full(dims, np.asarray(x[1]).reshape(()), dtype=src.dtype)
            dst_sel, src_sel = [], []
            for d, (l, h) in enumerate(zip(lo, hi)):
                s0 = max(0, -l)
                s1 = spread_shape[d] - max(0, -h)
                dst_sel.append(slice(max(0, l), max(0, l) + max(0, s1 - s0)))
                src_sel.append(slice(s0, max(s0, s1)))
            r[tuple(dst_sel)] = spread[tuple(src_sel)]
        elif k == "iota":
            d = ins.attrs["iota_dimension"][0]
            shape = [1] * len(dims)
            shape[d] = dims[d]
            base = np.arange(dims[d]).reshape(shape)
            r = _round_to(np.broadcast_to(base, dims).astype(np.float64), code) if _is_float(code) else np.broadcast_to(
                base, dims).astype(P.np_dtype(code))
        elif k == "dynamic_slice":
            sizes = ins.attrs["slice_sizes"]
            starts = [int(np.clip(int(np.asarray(s).reshape(())), 0, x[0].shape[d] - sizes[d])) for d, s in enumerate(x[1:])]
            r = x[0][tuple(slice(s, s + n) for s, n in zip(starts, sizes))]
        elif k == "dynamic_update_slice":
            upd = x[1]
            starts = [int(np.clip(int(np.asarray(s).reshape(())), 0, x[0].shape[d] - upd.shape[d])) for d, s in enumerate(x[2:])]
            r = x[0].copy()
            r[tuple(slice(s, s + n) for s, n in zip(starts, upd.shape))] = upd
        elif k == "gather":
            ids = np.clip(x[1].astype(np.int64).reshape(-1), 0, x[0].shape[0] - 1)
            r = x[0][ids].reshape(dims)
        elif k == "dot_general":
            if fast_dot:
                key = ins.inputs[1] if ins.inputs[1] in builder.parameter_ids else None
                r = _round_to(_dot_general_f32(x[0], x[1], ins, weight_cache, key), code)
            else:
                r = _round_to(_dot_general(x[0], x[1], ins), code)
        elif k in P.REDUCE and len(ins.outputs) == 1:
            axes = tuple(ins.attrs["reduce_dimensions"])
            src = builder.values[ins.inputs[0]].dtype
            if _is_float(src):
                v = _f64(x[0])
                with np.errstate(invalid="ignore"):
                    if k == "reduce_sum": r = v.sum(axis=axes)
                    elif k == "reduce_max": r = np.where(np.isnan(v).any(axis=axes), np.nan, np.max(np.where(np.isnan(v), -np.inf, v), axis=axes, initial=-np.inf))
                    else: r = np.where(np.isnan(v).any(axis=axes), np.nan, np.min(np.where(np.isnan(v), np.inf, v), axis=axes, initial=np.inf))
                r = _round_to(r, code)
            elif src == P.PRED:
                r = x[0].any(axis=axes) if k in ("reduce_or", "reduce_sum", "reduce_max") else x[0].all(axis=axes)
            else:
                dt = P.np_dtype(code)
                info = np.iinfo(dt)
                if k == "reduce_sum": r = x[0].sum(axis=axes, dtype=np.int64 if dt.kind == "i" else np.uint64).astype(dt)
                elif k == "reduce_max": r = x[0].max(axis=axes, initial=info.min)
                elif k == "reduce_min": r = x[0].min(axis=axes, initial=info.max)
                elif k == "reduce_and": r = np.bitwise_and.reduce(x[0], axis=axes) if len(axes) == 1 else np.bitwise_and.reduce(x[0].reshape(-1))
                else: r = np.bitwise_or.reduce(x[0], axis=axes) if len(axes) == 1 else np.bitwise_or.reduce(x[0].reshape(-1))
        elif k == "reduce_max" and len(ins.outputs) == 2:
            val, idx = _argmax_pair(x[0], x[1], ins.attrs["reduce_dimensions"])
            env[ins.outputs[0]] = _round_to(val, code).reshape(dims)
            env[ins.outputs[1]] = idx.reshape(dims)
            del x
            release(index, ins)
            continue
        elif k == "custom_call":
            if ins.target and ins.target.endswith("scaled_dot_product_attention"):
                r = _round_to(_sdpa(x[0], x[1], x[2], x[3]), code)
            elif ins.target and ins.target.endswith("custom_binary_add_f32"):
                r = _binary("add", x[0], x[1], code)
            elif ins.target == "annotate_device_placement":
                r = x[0]
            else:
                raise NotImplementedError(f"custom call {ins.target}")
        elif k == "optimization_barrier":
            r = x[0]
        elif k == "all_reduce":
            r = all_reduce(x[0], code) if all_reduce is not None else x[0]
        elif k == "all_gather":
            r = all_gather(x[0], code) if all_gather is not None else x[0][None]
        else:
            raise NotImplementedError(k)
        r = np.ascontiguousarray(np.asarray(r)).reshape(dims)
        if r.dtype != P.np_dtype(code):
            r = _round_to(r, code)
        env[ins.outputs[0]] = r
        del x
        release(index, ins)
    return [env[o] for o in builder.output_ids]
