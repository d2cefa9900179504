"""Pins the CPU oracle to every literal known-answer vector the reference's tests hold for the hot path."""
import os

import numpy as np
import pytest

from oracle import plan_interp
from pjrtx_b200 import plan as P
from tests import cases

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run(case):
    b, args = case
    return plan_interp.run_plan(b, args)


def test_u8_chain_first_and_second_run():
    # src/backend/mlx_metal/execution_call.zig:300-303 and :352-353
    assert run(cases.u8_chain())[0].tolist() == [6, 15, 28, 45]
    assert run(cases.u8_chain(np.array([2, 4, 6, 8], np.uint8)))[0].tolist() == [8, 21, 40, 65]


@pytest.mark.parametrize("dtype", [P.F16, P.BF16_CODE, P.F32])
def test_dot_2x2(dtype):
    # src/backend/mlx_metal/api_test.cc:624-687
    assert run(cases.dot_2x2(dtype))[0].reshape(-1).tolist() == [19.0, 22.0, 43.0, 50.0]


def test_dot_rhs_transposed_and_batched_match_triple_loop():
    # api_test.cc:689-776 recompute with a triple loop; same here
    b, (lhs, rhs) = cases.dot_rhs_transposed()
    want = np.array([[sum(lhs[m, k] * rhs[n, k] for k in range(3)) for n in range(4)] for m in range(2)], np.float32)
    np.testing.assert_allclose(plan_interp.run_plan(b, [lhs, rhs])[0], want, rtol=1e-6)
    b, (lhs, rhs) = cases.dot_batched()
    want = np.einsum("bmk,bkn->bmn", lhs.astype(np.float64), rhs.astype(np.float64)).astype(np.float32)
    np.testing.assert_allclose(plan_interp.run_plan(b, [lhs, rhs])[0], want, rtol=1e-6)


def test_attention_scores_and_context_match_triple_loop():
    # api_test.cc:826-928
    b, (q, k, p) = cases.attention_scores_context()
    scores, context = plan_interp.run_plan(b, [q, k, p])
    np.testing.assert_allclose(scores, np.einsum("bhqd,bkd->bhqk", q.astype(np.float64), k.astype(np.float64)), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(context, np.einsum("bhqk,bkd->bhqd", p.astype(np.float64), k.astype(np.float64)), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [P.F16, P.BF16_CODE])
def test_reduce_rows(dtype):
    # api_test.cc:930-1014
    s, mx, mn = run(cases.reduce_rows(dtype))
    assert s.tolist() == [3.0, 7.0] and mx.tolist() == [2.0, 4.0] and mn.tolist() == [1.0, 3.0]


def test_argmax_ties_pick_smallest_index():
    # api_test.cc:1016-1055; jax_op_suite.py:125 and :258-269
    val, idx = run(cases.argmax_ties())
    assert val.tolist() == [7.0, 5.0] and idx.tolist() == [1, 1] and idx.dtype == np.int32


def test_argmax_nan_counts_as_maximum():
    # api.cc:4102-4130: index where value == max or both are NaN
    v = np.array([[1.0, np.nan, 7.0, np.nan]], np.float32)
    val, idx = run(cases.argmax_ties(v))
    assert np.isnan(val[0]) and idx.tolist() == [1]


def test_sdpa_known_answers():
    # api_test.cc:271-353 (near_relaxed = 1e-2)
    np.testing.assert_allclose(run(cases.sdpa_single())[0].reshape(-1), [10.0, 0.0], atol=1e-2)
    np.testing.assert_allclose(run(cases.sdpa_gqa())[0].reshape(-1), [10, 0, 10, 0, 20, 0, 20, 0], atol=1e-2)


@pytest.mark.parametrize("name", ["tiny", "medium"])
def test_llama_like_block_matches_reference_numpy(name):
    # vectors produced by the reference's own np_reference (tests/golden/make_llama_like_golden.py); its tolerance
    # is rtol = atol = 2e-4 (jax_llama_like_inference.py:246-252)
    data = np.load(os.path.join(GOLDEN, f"llama_like_{name}.npz"))
    keys = ("x", "norm_w", "wq", "wk", "wv", "wo", "w1", "w2", "w3")
    b, args = cases.llama_like_block(*[data[k] for k in keys])
    got = plan_interp.run_plan(b, args)[0]
    np.testing.assert_allclose(got, data["expected"], rtol=2e-4, atol=2e-4)


def test_i8_negate_sub_wraps():
    assert run(cases.i8_negate_sub())[0].tolist() == [2, 6, -128, -127]


def test_structural_ops_clamp_indices():
    outs = run(cases.structural_ops())
    cube = cases.F32_CUBE
    np.testing.assert_array_equal(outs[5], cube[:, 1:3, :])        # dynamic_slice start 2 clamped to 1
    want = cube.copy(); want[:, 2:3, :] = -1.5
    np.testing.assert_array_equal(outs[6], want)
    table = np.arange(40, dtype=np.float32).reshape(10, 4) / np.float32(3.0)
    np.testing.assert_array_equal(outs[7], table[[[3, 9], [0, 9]]])  # id 12 clamped to 9


def test_pad_matches_numpy():
    """stablehlo.pad in the oracle against numpy.pad / explicit spreading (edge, interior and negative edge padding)."""
    b, (cube, row) = cases.pad_cases()
    outs = plan_interp.run_plan(b, [cube, row])
    edge = np.pad(cube, [(1, 0), (0, 2), (2, 1)], constant_values=np.float32(-7.5))
    assert np.array_equal(outs[0], edge)
    spread = np.full((2 * cube.shape[0] - 1, cube.shape[1], 3 * (cube.shape[2] - 1) + 1), np.float32(-7.5))
    spread[::2, :, ::3] = cube
    assert np.array_equal(outs[1], np.pad(spread, [(0, 1), (1, 0), (0, 0)], constant_values=np.float32(-7.5)))
    assert outs[2].tolist() == [9, 2, 9, 3, 9, 4, 9, 5, 9, 9, 9]
    assert outs[3].tolist() == [9, 9, 1, 2, 3]
    assert np.allclose(outs[4], (edge * 2.0).sum(axis=2))
