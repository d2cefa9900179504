"""Programs shared by the CPU (oracle / planner) and GPU (parity) tests.

Each case returns (builder, arguments). Shapes and values follow the reference's own op suite
(src/plugin/jax/jax_op_suite.py:112-440) and its C++ known-answer tests
(src/backend/mlx_metal/api_test.cc); the literal expected values live in test_oracle_golden.py.
"""
import numpy as np

from pjrtx_b200 import PlanBuilder
from pjrtx_b200 import plan as P

F32_A = ((np.arange(12, dtype=np.float32).reshape(3, 4) - np.float32(3.0)) / np.float32(7.0))
F32_B = np.linspace(0.5, 1.7, 12, dtype=np.float32).reshape(3, 4)
F32_CUBE = (np.arange(24, dtype=np.float32).reshape(2, 3, 4) - np.float32(8.0)) / np.float32(5.0)
ARGMAX_VALUES = np.array([[1.0, 7.0, 7.0, 3.0], [-2.0, 5.0, 4.0, 5.0]], dtype=np.float32)


def _params(b, arrays):
    return [b.parameter(P.dtype_code(a.dtype), a.shape) for a in arrays]


def u8_chain(x=np.array([1, 2, 3, 4], np.uint8)):
    """(x + c) * c with c = {2,3,4,5} (src/backend/mlx_metal/execution_call.zig:147-211)."""
    b = PlanBuilder()
    px = b.parameter(P.U8, [4])
    c = b.constant(np.array([2, 3, 4, 5], np.uint8))
    b.set_outputs([(px + c) * c])
    return b, [x]


def dot_2x2(dtype):
    """{1,2,3,4} @ {5,6,7,8} (api_test.cc:624-687)."""
    b = PlanBuilder()
    lhs = np.array([[1, 2], [3, 4]], np.float32).astype(P.np_dtype(dtype))
    rhs = np.array([[5, 6], [7, 8]], np.float32).astype(P.np_dtype(dtype))
    pl, pr = _params(b, [lhs, rhs])
    b.set_outputs([b.convert(b.dot_general(pl, pr, [1], [0]), P.F32)])
    return b, [lhs, rhs]


def dot_rhs_transposed():
    """lhs[2,3] · rhs[4,3] contracting both last axes (api_test.cc:689-727)."""
    b = PlanBuilder()
    lhs = np.array([[1, 2, 3], [-1, 0.5, 4]], np.float32)
    rhs = np.array([[1, 0, 2], [-1, 3, 0.5], [2, -2, 1], [0.25, 0.5, -1]], np.float32)
    pl, pr = _params(b, [lhs, rhs])
    b.set_outputs([b.dot_general(pl, pr, [1], [1])])
    return b, [lhs, rhs]


def dot_batched():
    """[2,2,3] x [2,3,4] with batch axis 0 (api_test.cc:729-776)."""
    b = PlanBuilder()
    lhs = np.array([(i % 7) - 3 for i in range(12)], np.float32).reshape(2, 2, 3)
    rhs = (np.array([(i % 11) - 5 for i in range(24)], np.float32) / np.float32(3.0)).reshape(2, 3, 4)
    pl, pr = _params(b, [lhs, rhs])
    b.set_outputs([b.dot_general(pl, pr, [2], [1], [0], [0])])
    return b, [lhs, rhs]


def attention_scores_context(dtype=P.F32):
    """einsum bhqd,bkd->bhqk and bhqk,bkd->bhqd (jax_op_suite.py:345-346, api_test.cc:826-928)."""
    rng = np.random.default_rng(3)
    dt = P.np_dtype(dtype)
    q = rng.standard_normal((2, 3, 4, 5), dtype=np.float32).astype(dt)
    k = rng.standard_normal((2, 6, 5), dtype=np.float32).astype(dt)
    p = rng.standard_normal((2, 3, 4, 6), dtype=np.float32).astype(dt)
    b = PlanBuilder()
    pq, pk, pp = _params(b, [q, k, p])
    scores = b.dot_general(pq, pk, [3], [2], [0], [0])
    context = b.dot_general(pp, pk, [3], [1], [0], [0])
    b.set_outputs([scores, context])
    return b, [q, k, p]


def reduce_rows(dtype):
    """Row sum / max / min of [[1,2],[3,4]] -> {3,7},{2,4},{1,3} (api_test.cc:930-1014)."""
    b = PlanBuilder()
    x = np.array([[1, 2], [3, 4]], np.float32).astype(P.np_dtype(dtype))
    (px,) = _params(b, [x])
    outs = [b.convert(b.reduce(k, px, [1]), P.F32) for k in ("reduce_sum", "reduce_max", "reduce_min")]
    b.set_outputs(outs)
    return b, [x]


def argmax_ties(values=ARGMAX_VALUES):
    """Two-operand max reduce: values {7,5}, indices {1,1} (api_test.cc:1016-1055, jax_op_suite.py:125,258-269)."""
    b = PlanBuilder()
    (pv,) = _params(b, [values])
    val, idx = b.argmax(pv, 1)
    b.set_outputs([val, idx])
    return b, [values]


def sdpa_single():
    """1 query, 2 keys, token_index 0 -> {10, 0} (api_test.cc:271-310)."""
    b = PlanBuilder()
    q = np.array([1, 0], np.float32).reshape(1, 1, 2)
    k = np.array([1, 0, 0, 1], np.float32).reshape(2, 1, 2)
    v = np.array([10, 0, 0, 20], np.float32).reshape(2, 1, 2)
    t = np.array(0, np.uint32)
    pq, pk, pv, pt = _params(b, [q, k, v, t])
    b.set_outputs([b.custom_call("pjrtx.mlx_metal.scaled_dot_product_attention", [pq, pk, pv, pt], P.F32, q.shape)])
    return b, [q, k, v, t]


def sdpa_gqa():
    """4 query heads over 2 kv heads -> {10,0,10,0,20,0,20,0} (api_test.cc:312-353)."""
    b = PlanBuilder()
    q = np.array([1, 0] * 4, np.float32).reshape(1, 4, 2)
    k = np.array([1, 0, 0, 1, 1, 0, 0, 1], np.float32).reshape(2, 2, 2)
    v = np.array([10, 0, 20, 0, 0, 30, 0, 40], np.float32).reshape(2, 2, 2)
    t = np.array(0, np.uint32)
    pq, pk, pv, pt = _params(b, [q, k, v, t])
    b.set_outputs([b.custom_call("pjrtx.mlx_metal.scaled_dot_product_attention", [pq, pk, pv, pt], P.F32, q.shape)])
    return b, [q, k, v, t]


def sdpa_random(dtype=P.BF16_CODE, batch=2, q_len=3, heads=8, kv_len=40, kv_heads=2, head_dim=64, token=20):
    rng = np.random.default_rng(11)
    dt = P.np_dtype(dtype)
    q = rng.standard_normal((batch, q_len, heads, head_dim), dtype=np.float32).astype(dt)
    k = rng.standard_normal((batch, kv_len, kv_heads, head_dim), dtype=np.float32).astype(dt)
    v = rng.standard_normal((batch, kv_len, kv_heads, head_dim), dtype=np.float32).astype(dt)
    t = np.array(token, np.int32)
    b = PlanBuilder()
    pq, pk, pv, pt = _params(b, [q, k, v, t])
    b.set_outputs([b.custom_call("pjrtx.b200.scaled_dot_product_attention", [pq, pk, pv, pt], dtype, q.shape)])
    return b, [q, k, v, t]


def prefill_attention(dtype=P.BF16_CODE, batch=2, kv_heads=2, rep=4, seq=96, head_dim=64, seed=13):
    """Causal self-attention over whole sequences, written op by op the way the prefill program writes it:
    scores = dot_general(q [B,G,S,rep,hd], k [B,S,G,hd]) -> f32 -> * 1/sqrt(hd) -> select(key <= position, ., -inf)
    -> max / exp / sum / divide -> element type -> dot_general(., v)."""
    rng = np.random.default_rng(seed)
    dt = P.np_dtype(dtype)
    q = rng.standard_normal((batch, kv_heads, seq, rep, head_dim), dtype=np.float32).astype(dt)
    k = rng.standard_normal((batch, seq, kv_heads, head_dim), dtype=np.float32).astype(dt)
    v = rng.standard_normal((batch, seq, kv_heads, head_dim), dtype=np.float32).astype(dt)
    b = PlanBuilder()
    pq, pk, pv = _params(b, [q, k, v])
    sdims = [batch, kv_heads, seq, rep, seq]
    causal = b.compare(b.iota(P.S32, sdims, 4), b.iota(P.S32, sdims, 2), P.LE)
    sf = b.convert(b.dot_general(pq, pk, [4], [3], [0, 1], [0, 2]), P.F32)
    sf = sf * b.scalar_like(sf, np.float32(1.0 / np.sqrt(np.float32(head_dim))))
    sf = b.select(causal, sf, b.scalar_like(sf, np.float32(-np.inf)))
    m = b.reduce("reduce_max", sf, [4])
    e = b.unary("exp", sf - b.broadcast_in_dim(m, sdims, [0, 1, 2, 3]))
    z = b.reduce("reduce_sum", e, [4])
    probs = b.convert(e / b.broadcast_in_dim(z, sdims, [0, 1, 2, 3]), dtype)
    b.set_outputs([b.dot_general(probs, pv, [4], [1], [0, 1], [0, 2])])
    return b, [q, k, v]


# ---- op-suite style cases (jax_op_suite.py) ---------------------------------------------------------------

def elementwise_float_chain():
    """tanh((x + y) * rsqrt(max(y, floor))) - exp(x * tiny) (jax_op_suite.py:176-186)."""
    b = PlanBuilder()
    floor = np.full((3, 4), 0.75, np.float32)
    tiny = np.full((3, 4), 0.125, np.float32)
    px, py, pf, pt = _params(b, [F32_A, F32_B, floor, tiny])
    r = b.unary("tanh", (px + py) * b.unary("rsqrt", b.binary("maximum", py, pf))) - b.unary("exp", px * pt)
    b.set_outputs([r])
    return b, [F32_A, F32_B, floor, tiny]


def reshape_transpose_broadcast():
    b = PlanBuilder()
    (px,) = _params(b, [F32_A])
    r = b.transpose(b.broadcast_in_dim(b.reshape(px, [2, 6]), [2, 2, 6], [1, 2]), [1, 2, 0])
    b.set_outputs([r])
    return b, [F32_A]


def reduce_cases():
    b = PlanBuilder()
    pa, pc = _params(b, [F32_A, F32_CUBE])
    outs = [
        b.reshape(b.reduce("reduce_sum", pa * pa, [1]), [3, 1]),
        b.reduce("reduce_max", pc, [1]),
        b.reduce("reduce_min", pc, [1]),
        b.reduce("reduce_sum", pc, [0, 1, 2]),
        b.reduce("reduce_sum", pc, [0, 2]),
    ]
    b.set_outputs(outs)
    return b, [F32_A, F32_CUBE]


def float_unary_math():
    """sin + cos + log1p(abs) + logistic; floor + ceil + sign; power + remainder; cbrt; round (jax_op_suite.py:421-430)."""
    b = PlanBuilder()
    pa, pb = _params(b, [F32_A, F32_B])
    u = lambda k, x: b.unary(k, x)
    outs = [
        u("sine", pa) + u("cosine", pa) + u("log1p", u("abs", pa)) + u("logistic", pa),
        u("floor", pa) + u("ceil", pa) + u("sign", pa),
        b.binary("power", u("abs", pa) + 1.0, pb) + b.binary("remainder", pa, pb),
        u("cbrt", pa),
        u("round_nearest_afz", pa),
        u("round_nearest_even", pa * 3.5),
        u("expm1", pa), u("log", pb), u("sqrt", pb), u("negate", pa),
        b.binary("atan2", pa, pb), b.binary("divide", pa, pb), b.binary("minimum", pa, pb),
        b.is_finite(pa),
    ]
    b.set_outputs(outs)
    return b, [F32_A, F32_B]


def is_finite_case():
    b = PlanBuilder()
    x = np.array([0.0, np.inf, -np.inf, np.nan], np.float32)
    (px,) = _params(b, [x])
    b.set_outputs([b.is_finite(px), b.binary("maximum", px, b.scalar_like(px, 1.0)), b.binary("minimum", px, b.scalar_like(px, 1.0))])
    return b, [x]


def int_ops():
    b = PlanBuilder()
    a = np.array([[7, -3, 12, 100], [0, -128, 5, 64]], np.int32)
    c = np.array([[3, 5, -4, 7], [9, 2, 5, -8]], np.int32)
    sh = np.array([[1, 2, 3, 31], [0, 33, 4, 5]], np.int32)
    u = np.array([0x80000000, 0xFFFFFFFF, 12345, 1], np.uint32)
    pa, pc, ps, pu = _params(b, [a, c, sh, u])
    outs = [
        b.binary("xor_", b.binary("and_", pa, pc), b.binary("shift_left", pa, ps)),
        b.binary("shift_right_arithmetic", pa, ps),
        b.binary("shift_right_logical", pu, b.scalar_like(pu, np.uint32(1))),
        b.binary("divide", pa, pc), b.binary("remainder", pa, pc), b.binary("or_", pa, pc),
        b.unary("negate", pa), b.unary("abs", pa), b.unary("sign", pa), b.unary("not_", pa),
        b.unary("popcnt", pu), b.unary("count_leading_zeros", pu),
        b.binary("maximum", pa, pc), b.binary("minimum", pa, pc), b.binary("multiply", pa, pc),
        b.convert(pa, P.F32), b.convert(b.convert(pa, P.F32) * 0.5, P.S32), b.convert(pa, P.S8), b.convert(pu, P.U8),
        b.compare(pa, pc, P.LT), b.select(b.compare(pa, pc, P.GE), pa, pc),
        b.clamp(b.scalar_like(pa, np.int32(-5)), pa, b.scalar_like(pa, np.int32(10))),
    ]
    b.set_outputs(outs)
    return b, [a, c, sh, u]


def i8_negate_sub():
    """negate(a - b) on i8 (src/plugin/api_execute_*_test.zig)."""
    b = PlanBuilder()
    a = np.array([1, -2, 127, -128], np.int8)
    c = np.array([3, 4, -1, 1], np.int8)
    pa, pc = _params(b, [a, c])
    b.set_outputs([-(pa - pc)])
    return b, [a, c]


def predicate_logic():
    b = PlanBuilder()
    x = np.array([True, True, False, False])
    y = np.array([True, False, True, False])
    px, py = _params(b, [x, y])
    b.set_outputs([b.binary("or_", b.unary("not_", b.binary("and_", px, py)), b.binary("xor_", px, py))])
    return b, [x, y]


def structural_ops():
    """slice / concatenate / reverse / iota / dynamic_slice / dynamic_update_slice / gather / pad-free views."""
    b = PlanBuilder()
    cube = F32_CUBE
    table = (np.arange(40, dtype=np.float32).reshape(10, 4) / np.float32(3.0))
    ids = np.array([[3, 9], [0, 12]], np.int32)  # 12 is clamped to 9
    start = np.array(2, np.int32)
    upd = np.full((2, 1, 4), -1.5, np.float32)
    pc, pt, pi, ps, pu = _params(b, [cube, table, ids, start, upd])
    zero = b.constant(np.int32(0))
    outs = [
        b.slice(pc, [0, 1, 0], [2, 3, 4], [1, 1, 2]),
        b.concatenate([pc, pc * 2.0], 1),
        b.reverse(pc, [2]),
        b.iota(P.S32, [3, 5], 1),
        b.iota(P.F32, [3, 5], 0),
        b.dynamic_slice(pc, [zero, ps, zero], [2, 2, 4]),   # start 2 clamps to 1
        b.dynamic_update_slice(pc, pu, [zero, ps, zero]),
        b.gather_rows(pt, pi),
        b.transpose(pc, [2, 0, 1]),
        b.broadcast_in_dim(b.reduce("reduce_max", pc, [2]), [2, 3, 4], [0, 1]),
    ]
    b.set_outputs(outs)
    return b, [cube, table, ids, start, upd]


def pad_cases():
    """stablehlo.pad: edge padding, interior padding, cropping by negative edges, a padded value feeding more work
    (src/backend/mlx_metal/api.cc:2637 is the reference's pad; api.h:310-313 its arguments)."""
    b = PlanBuilder()
    cube = F32_CUBE
    row = np.array([1, 2, 3, 4, 5], np.int32)
    pc, pr = _params(b, [cube, row])
    fill = b.constant(np.float32(-7.5))
    ifill = b.constant(np.int32(9))
    edge = b.pad(pc, fill, [1, 0, 2], [0, 2, 1])
    outs = [
        edge,
        b.pad(pc, fill, [0, 1, 0], [1, 0, 0], [1, 0, 2]),
        b.pad(pr, ifill, [-1], [3], [1]),          # crops the first element, spreads the rest, pads the tail
        b.pad(pr, ifill, [2], [-2]),
        b.reduce("reduce_sum", edge * 2.0, [2]),
    ]
    b.set_outputs(outs)
    return b, [cube, row]


def matmul_small(dtype=P.F32):
    b = PlanBuilder()
    dt = P.np_dtype(dtype)
    lhs = (np.arange(8, dtype=np.float32).reshape(2, 4) / np.float32(5.0)).astype(dt)
    rhs = (np.arange(12, dtype=np.float32).reshape(4, 3) / np.float32(6.0)).astype(dt)
    pl, pr = _params(b, [lhs, rhs])
    b.set_outputs([b.matmul(pl, pr)])
    return b, [lhs, rhs]


def llama_like_block(x, norm_w, wq, wk, wv, wo, w1, w2, w3):
    """The reference's llama-like block with closed-over weights as constants
    (src/plugin/jax/jax_llama_like_inference.py:212-237 and :313-335)."""
    seq, dim = x.shape
    b = PlanBuilder()
    px = b.parameter(P.F32, x.shape)
    c = b.constant
    ss = b.reshape(b.reduce("reduce_sum", px * px, [1]), [seq, 1])
    denom = ss * 0.25 + 1.0e-5
    h = px * b.broadcast_in_dim(b.unary("rsqrt", denom), [seq, dim], [0, 1]) * b.broadcast_in_dim(c(norm_w), [seq, dim], [1])
    q, k, v = b.matmul(h, c(wq)), b.matmul(h, c(wk)), b.matmul(h, c(wv))
    scores = b.matmul(q, b.transpose(k, [1, 0])) * 0.5
    mx = b.reshape(b.reduce("reduce_max", scores, [1]), [seq, 1])
    wts = b.unary("exp", scores - b.broadcast_in_dim(mx, [seq, seq], [0, 1]))
    sm = b.reshape(b.reduce("reduce_sum", wts, [1]), [seq, 1])
    wts = wts / b.broadcast_in_dim(sm, [seq, seq], [0, 1])
    attn = b.matmul(b.matmul(wts, v), c(wo))
    gate = b.unary("tanh", b.matmul(h, c(w1)))
    mlp = b.matmul(gate * b.matmul(h, c(w3)), c(w2))
    b.set_outputs([px + attn + mlp])
    return b, [x]


def op_suite_config1(rows=4096, cols=4096, seed=0):
    """z = x*y + sin(x) - log1p(|y|); row sum, max, argmax (s32) of z."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, size=(rows, cols)).astype(np.float32)
    y = rng.uniform(-1, 1, size=(rows, cols)).astype(np.float32)
    b = PlanBuilder()
    px, py = _params(b, [x, y])
    z = px * py + b.unary("sine", px) - b.unary("log1p", b.unary("abs", py))
    _, idx = b.argmax(z, 1)
    b.set_outputs([b.reduce("reduce_sum", z, [1]), b.reduce("reduce_max", z, [1]), idx])
    return b, [x, y]


def matmul_config1(n=1024, dtype=P.F32, seed=1):
    rng = np.random.default_rng(seed)
    dt = P.np_dtype(dtype)
    a = rng.uniform(-1, 1, size=(n, n)).astype(np.float32).astype(dt)
    bm = rng.uniform(-1, 1, size=(n, n)).astype(np.float32).astype(dt)
    b = PlanBuilder()
    pa, pb = _params(b, [a, bm])
    b.set_outputs([b.matmul(pa, pb)])
    return b, [a, bm]
