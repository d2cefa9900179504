"""GPU parity: every case runs through the C ABI on a B200 and is compared with the CPU oracle.

Bar: integer / predicate / index results bit-exact; f32 rel 1e-5; f16 / bf16 rel 2e-2 (atol = rtol * max|want|).
"""
import os

import numpy as np
import pytest

from pjrtx_b200 import PlanBuilder
from pjrtx_b200 import backend as be_mod
from pjrtx_b200 import plan as P
from tests import cases
from tests.util import assert_close, assert_outputs, run_backend, run_oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")

CASES = ["dot_rhs_transposed", "dot_batched", "attention_scores_context", "argmax_ties", "sdpa_single", "sdpa_gqa",
         "elementwise_float_chain", "reshape_transpose_broadcast", "reduce_cases", "float_unary_math", "is_finite_case",
         "int_ops", "i8_negate_sub", "predicate_logic", "structural_ops", "pad_cases", "matmul_small"]


@pytest.mark.parametrize("name", CASES)
def test_case_matches_oracle(gpu_backend, name):
    b, args = getattr(cases, name)()
    got = run_backend(gpu_backend, b, args)
    assert_outputs(b, got, run_oracle(b, args), name)


def test_u8_chain_values_and_stats(gpu_backend):
    """Known answers and counters of src/backend/mlx_metal/execution_call.zig:147-390."""
    be = gpu_backend
    b, _ = cases.u8_chain()
    exe = be.compile_executable(b, [0])
    s = exe.stats()
    assert s["resident_constant_count"] == 1 and s["resident_constant_bytes"] == 4
    assert (s["program_value_count"], s["program_node_count"], s["program_edge_count"]) == (4, 3, 3)
    assert s["program_schedule_item_count"] == 3 and s["program_fusion_group_count"] == 1
    assert s["program_materialization_boundary_count"] == 1
    assert s["program_planned_release_count"] == 1 and s["program_planned_release_bytes"] == 4
    assert s["program_peak_live_value_count"] == 4 and s["program_peak_live_bytes"] == 16
    assert s["program_device_count"] == 1 and s["execute_count"] == 0
    assert s["last_execute_device_index"] == 2**64 - 1 and s["last_execute_local_hardware_id"] == -1
    lhs = be.buffer_from_host(np.array([1, 2, 3, 4], np.uint8))
    # wrong device index, missing and surplus arguments are refused and leave the counters alone
    for bad_args, dev in (([lhs], 1), ([], 0), ([lhs, lhs], 0)):
        with pytest.raises(be_mod.BackendError):
            be.execute_executable(exe, bad_args, device_index=dev)
    assert exe.stats()["execute_count"] == 0
    out = be.execute_executable(exe, [lhs])
    assert len(out) == 1 and out[0].dtype == P.U8 and out[0].dims == (4,)
    assert out[0].to_numpy().tolist() == [6, 15, 28, 45]
    s = exe.stats()
    assert s["execute_count"] == 1 and s["last_execute_device_index"] == 0 and s["last_execute_local_hardware_id"] == 0
    second = be.buffer_from_host(np.array([2, 4, 6, 8], np.uint8))
    out2 = be.execute_executable(exe, [second])
    assert out2[0].to_numpy().tolist() == [8, 21, 40, 65]
    assert exe.stats()["execute_count"] == 2 and exe.stats()["resident_constant_count"] == 1


@pytest.mark.parametrize("dtype", [P.F16, P.BF16_CODE, P.F32])
def test_dot_2x2_known_answer(gpu_backend, dtype):
    b, args = cases.dot_2x2(dtype)
    assert run_backend(gpu_backend, b, args)[0].reshape(-1).tolist() == [19.0, 22.0, 43.0, 50.0]


@pytest.mark.parametrize("dtype", [P.F16, P.BF16_CODE])
def test_reduce_rows_known_answer(gpu_backend, dtype):
    s, mx, mn = run_backend(gpu_backend, *cases.reduce_rows(dtype))
    assert s.tolist() == [3.0, 7.0] and mx.tolist() == [2.0, 4.0] and mn.tolist() == [1.0, 3.0]


def test_argmax_ties_and_nan(gpu_backend):
    val, idx = run_backend(gpu_backend, *cases.argmax_ties())
    assert val.tolist() == [7.0, 5.0] and idx.tolist() == [1, 1]
    v = np.array([[1.0, np.nan, 7.0, np.nan], [np.nan, 2.0, 3.0, 4.0]], np.float32)
    val, idx = run_backend(gpu_backend, *cases.argmax_ties(v))
    assert np.isnan(val).all() and idx.tolist() == [1, 0]


def test_argmax_bit_exact_on_wide_rows_with_ties(gpu_backend):
    """bf16 logits over a 128256-wide vocabulary tie often; the index must be the oracle's."""
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal((4, 128256), dtype=np.float32) * 0.3).astype(P.np_dtype(P.BF16_CODE))
    logits[2, :] = logits[2, 7]  # a whole row of ties
    b = PlanBuilder()
    p = b.parameter(P.BF16_CODE, logits.shape)
    val, idx = b.argmax(p, 1)
    b.set_outputs([val, idx])
    got = run_backend(gpu_backend, b, [logits])
    want = run_oracle(b, [logits])
    assert np.array_equal(got[1], want[1]) and got[1][2] == 0
    assert np.array_equal(got[0].view(np.uint16), want[0].view(np.uint16))


@pytest.mark.parametrize("dtype", [P.F32, P.F16, P.BF16_CODE])
def test_sdpa_random(gpu_backend, dtype):
    b, args = cases.sdpa_random(dtype)
    assert_outputs(b, run_backend(gpu_backend, b, args), run_oracle(b, args), "sdpa")


@pytest.mark.parametrize("name", ["tiny", "medium"])
def test_llama_like_block_golden(gpu_backend, name):
    """Against the reference's NumPy reference (rtol = atol = 2e-4, jax_llama_like_inference.py:246-252)."""
    data = np.load(os.path.join(GOLDEN, f"llama_like_{name}.npz"))
    keys = ("x", "norm_w", "wq", "wk", "wv", "wo", "w1", "w2", "w3")
    b, args = cases.llama_like_block(*[data[k] for k in keys])
    be = gpu_backend
    exe = be.compile_executable(b, [0])
    weight_bytes = sum(data[k].nbytes for k in keys[1:])
    assert exe.stats()["resident_constant_bytes"] - weight_bytes <= 4096  # resident-constant overhead budget
    for _ in range(3):
        got = run_backend(be, b, args, exe=exe)[0]
        np.testing.assert_allclose(got, data["expected"], rtol=2e-4, atol=2e-4)
    assert exe.stats()["execute_count"] == 3


def test_config1_fused_chain_and_reductions(gpu_backend):
    """f32 [4096,4096]: z = x*y + sin(x) - log1p(|y|), row sum / max / argmax in one kernel."""
    b, args = cases.op_suite_config1()
    got = run_backend(gpu_backend, b, args)
    want = run_oracle(b, args)
    x, y = (a.astype(np.float64) for a in args)
    z_abs_sum = np.sum(np.abs(x * y) + np.abs(np.sin(x)) + np.abs(np.log1p(np.abs(y))), axis=1)
    # row sums: relative to the magnitude that was summed (cancellation makes |sum| << sum|terms|)
    assert np.max(np.abs(got[0].astype(np.float64) - want[0]) / z_abs_sum) <= 1e-5
    assert_close(got[1], want[1], 1e-5, what="row max")
    # argmax: the oracle rounds a float64 z, the kernel's sinf / log1pf differ from that by an ulp, so a row whose two
    # best z lie within that ulp can pick the other index. Every differing row must be such a row: the z the oracle holds
    # at the kernel's index is within two float32 ulps of the oracle's maximum. All other rows are bit-exact.
    z32 = np.asarray(want[1], np.float32)
    zf = (x * y + np.sin(x) - np.log1p(np.abs(y))).astype(np.float32)
    differing = np.nonzero(got[2] != want[2])[0]
    picked = zf[differing, got[2][differing]]
    ulp = np.spacing(np.abs(z32[differing]))
    assert np.all(np.abs(picked.astype(np.float64) - z32[differing]) <= 2 * ulp), (len(differing), differing[:8])
    assert len(differing) <= 0.001 * len(z32)  # and there are few of them


@pytest.mark.parametrize("dtype", [P.F32, P.F16])
def test_config1_matmul_1024(gpu_backend, dtype):
    b, args = cases.matmul_config1(1024, dtype)
    got = run_backend(gpu_backend, b, args)[0].astype(np.float64)
    a64, b64 = args[0].astype(np.float64), args[1].astype(np.float64)
    want = a64 @ b64
    mag = np.abs(a64) @ np.abs(b64)  # error scales with the summed magnitudes
    rtol = 1e-5 if dtype == P.F32 else 2e-2
    assert np.max(np.abs(got - want) / mag) <= rtol
    if dtype == P.F16:
        assert_close(got, want.astype(np.float16), 2e-2, what="f16 matmul")


def test_streaming_dot_paths_against_f64(gpu_backend):
    """Skinny contractions: rhs[K,N] (split-K) and rhs[N,K] for m = 1..8, bf16 and f32."""
    rng = np.random.default_rng(9)
    for dtype, rtol in ((P.BF16_CODE, 2e-2), (P.F32, 1e-5), (P.F16, 2e-2)):
        dt = P.np_dtype(dtype)
        for m, k, n in ((1, 4096, 1024), (4, 512, 2048), (8, 1000, 264), (3, 64, 40)):
            lhs = rng.standard_normal((m, k), dtype=np.float32).astype(dt)
            rkn = rng.standard_normal((k, n), dtype=np.float32).astype(dt)
            b = PlanBuilder()
            pl, pr = b.parameter(dtype, lhs.shape), b.parameter(dtype, rkn.shape)
            prt = b.parameter(dtype, (n, k))
            b.set_outputs([b.dot_general(pl, pr, [1], [0]), b.dot_general(pl, prt, [1], [1])])
            rnk = np.ascontiguousarray(rkn.T)
            got = run_backend(gpu_backend, b, [lhs, rkn, rnk])
            want = lhs.astype(np.float64) @ rkn.astype(np.float64)
            mag = np.abs(lhs.astype(np.float64)) @ np.abs(rkn.astype(np.float64))
            for g in got:
                err = np.abs(g.astype(np.float64) - want)
                assert np.all(err <= rtol * mag + rtol * np.abs(want)), (dtype, m, k, n, float((err / mag).max()))
            # both layouts agree and repeated runs are bit-identical (fixed reduction order)
            again = run_backend(gpu_backend, b, [lhs, rkn, rnk])
            assert all(np.array_equal(a.view(np.uint8), c.view(np.uint8)) for a, c in zip(got, again))


@pytest.mark.parametrize("dtype", [P.BF16_CODE, P.F16])
def test_tensor_core_dot_shapes_against_f64(gpu_backend, dtype):
    """16-bit contractions on the tcgen05 path: one row up to several 256-row tiles, ragged k and n, both rhs layouts,
    three contractions sharing lhs in one launch; error bounded by the summed magnitudes, repeated runs bit-identical."""
    rng = np.random.default_rng(23)
    dt = P.np_dtype(dtype)
    rtol = 2e-2
    for m, k, n in ((1, 4096, 4096), (16, 64, 128), (32, 4096, 1024), (20, 200, 264), (5, 520, 136), (256, 512, 384),
                    (300, 1024, 1000), (600, 328, 520)):
        lhs = rng.standard_normal((m, k), dtype=np.float32).astype(dt)
        rkn = rng.standard_normal((k, n), dtype=np.float32).astype(dt)
        rkn2 = rng.standard_normal((k, 256), dtype=np.float32).astype(dt)
        b = PlanBuilder()
        pl, pr, pr2 = b.parameter(dtype, lhs.shape), b.parameter(dtype, rkn.shape), b.parameter(dtype, rkn2.shape)
        prt = b.parameter(dtype, (n, k))
        b.set_outputs([b.dot_general(pl, pr, [1], [0]), b.dot_general(pl, pr2, [1], [0]), b.dot_general(pl, prt, [1], [1])])
        exe = gpu_backend.compile_executable(b, [0])
        steps = [s for s in exe.describe()["kernel_plan"]["steps"] if s["type"] == "dot"]
        # three rows and more take the tensor-core kernel; one and two keep the CUDA-core streaming kernels by default
        assert steps and (m <= 2 or all(s["umma"] == 1 for s in steps)), steps
        assert any(s["group"] == 2 for s in steps), steps  # the two rhs[K,N] contractions share a launch
        rnk = np.ascontiguousarray(rkn.T)
        got = run_backend(gpu_backend, b, [lhs, rkn, rkn2, rnk], exe=exe)
        again = run_backend(gpu_backend, b, [lhs, rkn, rkn2, rnk], exe=exe)
        exe.destroy()
        l64 = lhs.astype(np.float64)
        for g, r in zip(got, (rkn, rkn2, rkn)):
            want = l64 @ r.astype(np.float64)
            mag = np.abs(l64) @ np.abs(r.astype(np.float64))
            err = np.abs(g.astype(np.float64) - want)
            assert g.shape == want.shape
            assert np.all(err <= rtol * mag * 0.05 + 2.0 ** -8 * np.abs(want)), (dtype, m, k, n, float((err / mag).max()))
        assert all(np.array_equal(a.view(np.uint8), c.view(np.uint8)) for a, c in zip(got, again))


def test_donated_slice_update_is_in_place(gpu_backend):
    be = gpu_backend
    b = PlanBuilder()
    cache = b.parameter(P.BF16_CODE, [2, 16, 2, 8])
    upd = b.parameter(P.BF16_CODE, [2, 1, 2, 8])
    pos = b.parameter(P.S32, [])
    zero = b.constant(np.int32(0))
    out = b.dynamic_update_slice(cache, upd, [zero, pos, zero, zero])
    b.set_outputs([out, b.reduce("reduce_sum", b.convert(out, P.F32), [0, 1, 2, 3])], donate={0: 0})
    exe = be.compile_executable(b, [0])
    rng = np.random.default_rng(2)
    c0 = rng.standard_normal((2, 16, 2, 8), dtype=np.float32).astype(P.np_dtype(P.BF16_CODE))
    u = rng.standard_normal((2, 1, 2, 8), dtype=np.float32).astype(P.np_dtype(P.BF16_CODE))
    want = run_oracle(b, [c0, u, np.array(5, np.int32)])
    cb, ub, pb = be.buffer_from_host(c0), be.buffer_from_host(u), be.buffer_from_host(np.array(5, np.int32))
    outs = be.execute_executable(exe, [cb, ub, pb])
    assert cb.is_donated and not ub.is_donated
    assert np.array_equal(outs[0].to_numpy().view(np.uint16), want[0].view(np.uint16))
    assert_close(outs[1].to_numpy(), want[1], 1e-5, atol_scale=float(np.abs(c0.astype(np.float32)).sum()))
    assert exe.stats()["donation_alias_output_count"] == 1
    with pytest.raises(be_mod.BackendError):  # a donated buffer cannot be used again
        be.execute_executable(exe, [cb, ub, pb])
    # position beyond the end clamps to the last row
    outs2 = be.execute_executable(exe, [outs[0], ub, be.buffer_from_host(np.array(99, np.int32))])
    got = outs2[0].to_numpy()
    assert np.array_equal(got[:, 15].view(np.uint16), u[:, 0].view(np.uint16))


def test_slice_updates_ride_in_the_producing_kernel(gpu_backend):
    """Two in-place updates of different donated buffers computed and stored by one generated kernel: one writes whole
    trailing rows (vector stores), the other a window inside the innermost axis (scalar stores); start indices clamp."""
    be = gpu_backend
    b = PlanBuilder()
    cache = b.parameter(P.BF16_CODE, [2, 16, 2, 8])
    table = b.parameter(P.F32, [6, 40])
    x = b.parameter(P.BF16_CODE, [2, 2, 8])
    y = b.parameter(P.F32, [2, 16])
    pos = b.parameter(P.S32, [])
    col = b.parameter(P.S32, [])
    zero = b.constant(np.int32(0))
    upd = b.reshape(x * x + x, [2, 1, 2, 8])
    out0 = b.dynamic_update_slice(cache, upd, [zero, pos, zero, zero])
    win = b.unary("tanh", y) * y
    out1 = b.dynamic_update_slice(table, win, [pos, col])
    b.set_outputs([out0, out1], donate={0: 0, 1: 1})
    exe = be.compile_executable(b, [0])
    steps = be.describe_kernels(b)["steps"]
    assert [s["type"] for s in steps] == ["fused"] and "dst1" in steps[0]["source"], [s["type"] for s in steps]
    rng = np.random.default_rng(31)
    c0 = rng.standard_normal((2, 16, 2, 8), dtype=np.float32).astype(P.np_dtype(P.BF16_CODE))
    t0 = rng.standard_normal((6, 40), dtype=np.float32)
    xs = rng.standard_normal((2, 2, 8), dtype=np.float32).astype(P.np_dtype(P.BF16_CODE))
    ys = rng.standard_normal((2, 16), dtype=np.float32)
    for p_, c_ in ((3, 7), (0, 0), (99, 99), (-4, -1), (15, 24)):
        args = [c0, t0, xs, ys, np.array(p_, np.int32), np.array(c_, np.int32)]
        want = run_oracle(b, args)
        outs = be.execute_executable(exe, [be.buffer_from_host(a) for a in args])
        got0, got1 = outs[0].to_numpy(), outs[1].to_numpy()
        assert_close(got0, want[0], 2e-2, what=f"cache pos={p_}")
        assert_close(got1, want[1], 1e-5, what=f"table pos={p_} col={c_}")
        # everything outside the windows is untouched, bit for bit
        r = min(max(p_, 0), 15)
        mask = np.ones(c0.shape, bool)
        mask[:, r] = False
        assert np.array_equal(got0.view(np.uint16)[mask], c0.view(np.uint16)[mask])
        r1, c1 = min(max(p_, 0), 4), min(max(c_, 0), 24)
        mask1 = np.ones(t0.shape, bool)
        mask1[r1:r1 + 2, c1:c1 + 16] = False
        assert np.array_equal(got1[mask1], t0[mask1])


def test_values_without_elements(gpu_backend):
    """Empty operands and results: no kernel is launched for them, the other outputs are unaffected, and a contraction
    with no rows returns an empty result."""
    be = gpu_backend
    b = PlanBuilder()
    x, y, z = b.parameter(P.F32, [0, 4]), b.parameter(P.F32, [0, 4]), b.parameter(P.F32, [3])
    w = b.parameter(P.F32, [4, 5])
    b.set_outputs([x + y, z * z, b.dot_general(x, w, [1], [0])])
    args = [np.zeros((0, 4), np.float32), np.zeros((0, 4), np.float32), np.array([1, 2, 3], np.float32),
            np.ones((4, 5), np.float32)]
    got = run_backend(be, b, args)
    want = run_oracle(b, args)
    assert got[0].shape == (0, 4) and got[2].shape == (0, 5)
    assert np.array_equal(got[1], want[1]) and np.array_equal(got[1], np.array([1, 4, 9], np.float32))


def test_buffer_round_trip_and_errors(gpu_backend):
    be = gpu_backend
    for dt in (np.float32, np.int32, np.uint8, np.int8, np.uint16, np.uint32, np.uint64, np.int64, np.float16, np.bool_):
        a = (np.arange(24).reshape(2, 3, 4) % 5).astype(dt)
        buf = be.buffer_from_host(a)
        assert buf.dims == (2, 3, 4) and buf.nbytes == a.nbytes
        assert np.array_equal(buf.to_numpy(), a)
        clone = be.clone_buffer(buf)
        assert np.array_equal(clone.to_numpy(), a)
    empty = be.buffer_from_host(np.zeros((0, 4), np.float32))
    assert empty.nbytes == 0 and empty.to_numpy().shape == (0, 4)
    z = be.allocate_buffer(P.F32, [3, 3])
    assert not z.to_numpy().any()
    big = np.arange(1 << 20, dtype=np.float32)  # larger than the pinned staging slot
    assert np.array_equal(be.buffer_from_host(big).to_numpy(), big)
    stats = be.memory_stats()
    assert stats["host_to_device_bytes"] >= big.nbytes and stats["device_to_host_bytes"] >= big.nbytes
    with pytest.raises(be_mod.BackendError):
        be.buffer_from_host(np.zeros(4, np.float32), device=99)
    # undersized destination
    import ctypes
    dst = np.zeros(2, np.float32)
    assert be.lib.pjrtx_b200_buffer_copy_to_host(z.handle, dst.ctypes.data_as(ctypes.c_void_p), dst.nbytes) == 0


@pytest.mark.timeout(600)
@pytest.mark.parametrize("kernel,dtype,heads,kv_heads,hd,kv_len", [
    ("cuda", P.BF16_CODE, 32, 8, 128, 300),
    ("mma", P.BF16_CODE, 32, 8, 128, 300),
    ("mma", P.F16, 16, 2, 64, 200),
    ("mma", P.BF16_CODE, 16, 2, 128, 150),
    ("cuda", P.F16, 16, 2, 64, 200),
    ("cuda", P.F32, 8, 4, 64, 100),
    ("default", P.BF16_CODE, 16, 4, 128, 40),    # a buffer shorter than a stage of the tensor-core kernel: CUDA cores
    ("default", P.BF16_CODE, 32, 8, 128, 64),    # exactly one stage: tensor-core kernel
    ("staged", P.BF16_CODE, 32, 8, 128, 300),
    ("staged3", P.BF16_CODE, 32, 8, 128, 384),
    ("staged", P.F16, 16, 2, 64, 200),
    ("staged", P.BF16_CODE, 16, 2, 128, 150),
    ("staged", P.BF16_CODE, 8, 8, 128, 130),
    ("staged", P.F16, 4, 2, 64, 260),
])
def test_decode_attention_every_visible_length(gpu_backend, monkeypatch, kernel, dtype, heads, kv_heads, hd, kv_len):
    """Split-KV decode attention with Llama-like head shapes: every visible length from 1 to the buffer size, so every
    ragged split of the key range is exercised (decode-shaped SDPA call: one query position). Both the CUDA-core and
    the warp-level tensor-core kernel, 4 and 8 query heads per KV head, head sizes 64 and 128; and the shared-memory
    staged kernel (PJRTX_B200_ATTENTION_STAGED=1) with 1, 2, 4 and 8 query heads per KV head, once with three splits
    of up to 128 keys (a full stage)."""
    be = gpu_backend
    if kernel.startswith("staged"):
        monkeypatch.delenv("PJRTX_B200_ATTENTION_MMA", raising=False)
        monkeypatch.setenv("PJRTX_B200_ATTENTION_STAGED", "1")
        if kernel == "staged3":
            monkeypatch.setenv("PJRTX_B200_ATTENTION_SPLITS", "3")
    elif kernel == "default":
        monkeypatch.delenv("PJRTX_B200_ATTENTION_MMA", raising=False)
    else:
        monkeypatch.setenv("PJRTX_B200_ATTENTION_MMA", "1" if kernel == "mma" else "0")
    rng = np.random.default_rng(23)
    dt = P.np_dtype(dtype)
    batch = 2
    q = rng.standard_normal((batch, 1, heads, hd), dtype=np.float32).astype(dt)
    k = rng.standard_normal((batch, kv_len, kv_heads, hd), dtype=np.float32).astype(dt)
    v = rng.standard_normal((batch, kv_len, kv_heads, hd), dtype=np.float32).astype(dt)
    b = PlanBuilder()
    pq, pk, pv = b.parameter(dtype, q.shape), b.parameter(dtype, k.shape), b.parameter(dtype, v.shape)
    pt = b.parameter(P.S32, [])
    b.set_outputs([b.custom_call("pjrtx.b200.scaled_dot_product_attention", [pq, pk, pv, pt], dtype, q.shape)])
    exe = be.compile_executable(b, [0])
    steps = exe.describe()["kernel_plan"]["steps"]
    assert [s["type"] for s in steps] == ["attention_decode"]
    assert steps[0]["mma"] == {"cuda": 0, "mma": 1, "staged": 2, "staged3": 2, "default": 1 if kv_len >= 64 else 0}[kernel]
    if kernel == "staged3":
        assert steps[0]["splits"] == 3
    bufs = [be.buffer_from_host(a) for a in (q, k, v)]
    for token in list(range(0, kv_len)) + [kv_len + 5]:
        tb = be.buffer_from_host(np.array(token, np.int32))
        got = be.execute_executable(exe, bufs + [tb])[0].to_numpy()
        if token % 37 == 0 or token >= kv_len - 2 or token in (15, 16, 63, 64, 65, 127, 128):
            want = run_oracle(b, [q, k, v, np.array(token, np.int32)])[0]
            assert_close(got, want, 1e-5 if dtype == P.F32 else 2e-2, what=f"{kernel} token {token}")
        assert np.isfinite(got.astype(np.float32)).all()


def test_executable_cache_compiles_reuses_and_evicts(gpu_backend):
    """src/runtime/client_residency_tests.zig:184-267 with real executables: the second compile of a fingerprint leases
    the resident executable (same handle, no compile), an idle executable over the byte budget is destroyed and its
    device memory returned, and the fingerprint compiles again afterwards with the same results."""
    be = gpu_backend
    cache = be_mod.ExecutableCache(be)
    b, _ = cases.u8_chain()
    lhs = be.buffer_from_host(np.array([1, 2, 3, 4], np.uint8))
    first = cache.compile(b, [0])
    assert not first.reused and first.fingerprint == be.plan_fingerprint(b, [0])
    e = cache.entry(first.fingerprint)
    assert e["resident"] and e["reference_count"] == 1 and e["resident_bytes"] >= 4 and e["compile_latency_us"] > 0
    second = cache.compile(b, [0])
    assert second.reused and second.handle == first.handle
    s = cache.stats()
    assert (s["misses"], s["hits"], s["resident_entries"], s["compile_latency_samples"]) == (1, 1, 1, 1)
    assert cache.entry(first.fingerprint)["reference_count"] == 2
    assert be.execute_executable(second, [lhs])[0].to_numpy().tolist() == [6, 15, 28, 45]
    assert first.stats()["execute_count"] == 1                  # one executable behind both leases
    second.destroy()
    first.destroy()
    e = cache.entry(first.fingerprint)
    assert e["resident"] and e["reference_count"] == 0
    held = be.memory_stats()["bytes_in_use"]
    cache.set_max_resident_bytes(0)
    e2 = cache.entry(first.fingerprint)
    assert not e2["resident"]
    assert be.memory_stats()["bytes_in_use"] <= held - e["resident_bytes"]
    s = cache.stats()
    assert (s["evictions"], s["evicted_resident_bytes"], s["resident_bytes"]) == (1, e["resident_bytes"], 0)
    third = cache.compile(b, [0])
    assert not third.reused
    assert be.execute_executable(third, [lhs])[0].to_numpy().tolist() == [6, 15, 28, 45]
    third.destroy()                                               # budget 0: evicted as soon as it is idle
    assert not cache.entry(first.fingerprint)["resident"]
    assert cache.stats()["evictions"] == 2
    cache.destroy()


@pytest.mark.parametrize("dtype,kv_heads,rep,seq,hd", [
    (P.BF16_CODE, 2, 4, 1, 64),      # a single position: one row tile, one stage, rows past the end
    (P.BF16_CODE, 2, 4, 63, 64),
    (P.BF16_CODE, 1, 1, 64, 128),    # one head per KV head: a row tile spans 64 positions
    (P.BF16_CODE, 2, 4, 65, 128),    # second key stage holds a single key
    (P.F16, 2, 8, 200, 64),          # eight heads per KV head, ragged last row tile
    (P.BF16_CODE, 1, 4, 333, 128),   # six key stages: the copy ring wraps
    (P.F16, 1, 3, 130, 128),         # positions straddle warps (rep does not divide 16)
])
def test_prefill_attention_matches_oracle(gpu_backend, dtype, kv_heads, rep, seq, hd):
    """Causal self-attention over whole sequences on the prefill kernel against the op-by-op oracle."""
    b, args = cases.prefill_attention(dtype=dtype, batch=2, kv_heads=kv_heads, rep=rep, seq=seq, head_dim=hd)
    exe = gpu_backend.compile_executable(b, [0])
    assert [s["type"] for s in exe.describe()["kernel_plan"]["steps"]] == ["attention_prefill"]
    got = run_backend(gpu_backend, b, args, exe=exe)
    assert_outputs(b, got, run_oracle(b, args), f"prefill attention {kv_heads}x{rep} seq {seq} hd {hd}")


def test_prefill_attention_same_as_written_chain(gpu_backend, monkeypatch):
    """The kernel and the unfused chain (dot -> softmax row kernel -> dot) agree within the 16-bit tolerance."""
    b, args = cases.prefill_attention(seq=150, rep=4, head_dim=128)
    fused = run_backend(gpu_backend, b, args)
    monkeypatch.setenv("PJRTX_B200_ATTENTION_PREFILL", "0")
    exe = gpu_backend.compile_executable(b, [0])
    assert "attention_prefill" not in [s["type"] for s in exe.describe()["kernel_plan"]["steps"]]
    plain = run_backend(gpu_backend, b, args, exe=exe)
    assert_close(fused[0], plain[0], 2e-2, what="prefill attention kernel vs chain")


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_survives(gpu_backend):
    """Failure detection without a GPU fault (the reference injects failures on the host, src/runtime/execution_call.zig:
    355-360): a CTA waits for a barrier nothing completes, gives up after 50 ms and raises the device's error word; the
    host reads it at the next synchronize, the word is cleared, and the device keeps computing correctly."""
    be = gpu_backend
    be.synchronize(0)
    t0 = be.record_event(0)
    be.bounded_wait_probe(0, timeout_ms=50)
    t1 = be.record_event(0)
    with pytest.raises(be_mod.BackendError, match=r"gave up a bounded wait \(code 31\)"):
        be.synchronize(0)
    assert 40.0 <= be.elapsed_ms(t0, t1) <= 500.0  # the wait ended by its time limit, not by a poll count
    be.synchronize(0)  # the word was cleared by the failed call
    b, args = cases.u8_chain()
    assert run_backend(be, b, args)[0].tolist() == [6, 15, 28, 45]


@pytest.mark.parametrize("m,k,n,dtype", [(16, 256, 256, P.BF16_CODE), (16, 256, 128, P.F16), (32, 1024, 384, P.BF16_CODE),
                                         (5, 512, 200, P.BF16_CODE), (32, 4096, 6144, P.BF16_CODE), (64, 512, 1000, P.F16)])
def test_int8_dequantising_contraction(gpu_backend, m, k, n, dtype):
    """dot_general(x, convert(convert(w s8 -> f16) * scale)) from three rows up reads the bytes themselves where the
    byte rows have a 16-byte pitch: the tensor core contracts the integers and the column scales multiply the f32
    accumulators. Against the exact contraction in f64 the only error left is the rounding of the output (one part in
    2^8 at bf16, 2^11 at f16, of the largest value); the other widths materialise the scaled weights and round each."""
    rng = np.random.default_rng(m * 1000 + n)
    npdt = P.np_dtype(dtype)
    x = rng.standard_normal((m, k), dtype=np.float32).astype(npdt)
    w = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    sc = (rng.uniform(0.5, 1.5, size=(n,)) / 127 / np.sqrt(k)).astype(np.float16)
    b = PlanBuilder()
    px, pw, ps = b.parameter(dtype, x.shape), b.parameter(P.S8, w.shape), b.parameter(P.F16, sc.shape)
    wf = b.convert(pw, P.F16) * b.broadcast_in_dim(ps, w.shape, [1])
    if dtype != P.F16:
        wf = b.convert(wf, dtype)
    b.set_outputs([b.dot_general(px, wf, [1], [0])])
    exe = gpu_backend.compile_executable(b, [0])
    dots = [s for s in exe.describe()["kernel_plan"]["steps"] if s["type"] == "dot"]
    assert len(dots) == 1 and dots[0]["rhs_s8"] == (1 if n % 16 == 0 else 0), dots  # byte rows need a 16-byte pitch
    got = gpu_backend.execute_executable(exe, [gpu_backend.buffer_from_host(a) for a in (x, w, sc)])[0].to_numpy().astype(np.float64)
    want = x.astype(np.float64) @ (w.astype(np.float64) * sc.astype(np.float64)[None, :])
    ulp = 2.0 ** (-8 if dtype == P.BF16_CODE else -11)
    bound = (1.01 if n % 16 == 0 else 3.0) * ulp * np.max(np.abs(want))
    assert np.max(np.abs(got - want)) <= bound, (np.max(np.abs(got - want)), np.max(np.abs(want)))
