"""StableHLO text importer: modules in the textual form (pretty and generic operation syntax) become plans that the
CPU oracle evaluates to the expected numbers; operations outside the subset produce the reference's diagnostic line.

The first group restates the reference's importer fixtures (src/compiler/stablehlo_import_tests.zig:24-37, 340-349,
366-373, 390-397, 414-424); the rest is written the way `jax.jit(...).lower(...).as_text()` prints the operations the
five benchmark configurations use."""
import numpy as np
import pytest

import pjrtx_b200
from pjrtx_b200 import plan as P
from pjrtx_b200.backend import BackendError
from tests.util import assert_close, run_oracle

REDUCE_GENERIC = """
module {
  func.func @main(%arg0: tensor<2x3xf32>) -> tensor<2xf32> {
    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %0 = "stablehlo.reduce"(%arg0, %cst) ({
    ^bb0(%lhs: tensor<f32>, %rhs: tensor<f32>):
      %sum = stablehlo.add %lhs, %rhs : tensor<f32>
      stablehlo.return %sum : tensor<f32>
    }) {dimensions = array<i64: 1>} : (tensor<2x3xf32>, tensor<f32>) -> tensor<2xf32>
    return %0 : tensor<2xf32>
  }
}
"""

ADD_TANH = """
module {
  func.func @main(%arg0: tensor<2xf32>, %arg1: tensor<2xf32>) -> tensor<2xf32> {
    %0 = stablehlo.add %arg0, %arg1 : tensor<2xf32>
    %1 = stablehlo.tanh %0 : tensor<2xf32>
    return %1 : tensor<2xf32>
  }
}
"""

SHARDED_ARG = """
sdy.mesh @mesh = <["x"=2]>
func.func @main(%arg0: tensor<4xf32> {sdy.sharding = #sdy.sharding<@mesh, [{"x"}]>}) -> tensor<4xf32> {
  %0 = stablehlo.add %arg0, %arg0 : tensor<4xf32>
  return %0 : tensor<4xf32>
}
"""

BARRIER = """
func.func @main(%arg0: tensor<4xf32>, %arg1: tensor<4xf32>) -> (tensor<4xf32>, tensor<4xf32>) {
  %0, %1 = "stablehlo.optimization_barrier"(%arg0, %arg1) : (tensor<4xf32>, tensor<4xf32>) -> (tensor<4xf32>, tensor<4xf32>)
  %2 = stablehlo.multiply %0, %1 : tensor<4xf32>
  return %2, %1 : tensor<4xf32>, tensor<4xf32>
}
"""

LEGACY_BROADCAST = """
func.func @main(%arg0: tensor<f32>) -> tensor<4xf32> {
  %0 = "stablehlo.broadcast"(%arg0) {
    broadcast_sizes = array<i64: 4>
  } : (tensor<f32>) -> tensor<4xf32>
  return %0 : tensor<4xf32>
}
"""

# softmax(q . k^T * scale masked by position) . v for one query row, written as JAX prints it
ATTENTION = """
module @jit_attend attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<1x4x8xf32>, %arg1: tensor<1x6x8xf32>, %arg2: tensor<1x6x8xf32>, %arg3: tensor<i32>) -> (tensor<1x4x8xf32> {jax.result_info = ""}) {
    %0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [0] x [0], contracting_dims = [2] x [2], precision = [DEFAULT, DEFAULT] : (tensor<1x4x8xf32>, tensor<1x6x8xf32>) -> tensor<1x4x6xf32>
    %cst = stablehlo.constant dense<0.353553385> : tensor<f32>
    %1 = stablehlo.broadcast_in_dim %cst, dims = [] : (tensor<f32>) -> tensor<1x4x6xf32>
    %2 = stablehlo.multiply %0, %1 : tensor<1x4x6xf32>
    %3 = stablehlo.iota dim = 2 : tensor<1x4x6xi32>
    %4 = stablehlo.broadcast_in_dim %arg3, dims = [] : (tensor<i32>) -> tensor<1x4x6xi32>
    %5 = stablehlo.compare  LE, %3, %4,  SIGNED : (tensor<1x4x6xi32>, tensor<1x4x6xi32>) -> tensor<1x4x6xi1>
    %cst_0 = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %6 = stablehlo.broadcast_in_dim %cst_0, dims = [] : (tensor<f32>) -> tensor<1x4x6xf32>
    %7 = stablehlo.select %5, %2, %6 : tensor<1x4x6xi1>, tensor<1x4x6xf32>
    %cst_1 = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %8 = stablehlo.reduce(%7 init: %cst_1) applies stablehlo.maximum across dimensions = [2] : (tensor<1x4x6xf32>, tensor<f32>) -> tensor<1x4xf32>
    %9 = stablehlo.broadcast_in_dim %8, dims = [0, 1] : (tensor<1x4xf32>) -> tensor<1x4x6xf32>
    %10 = stablehlo.subtract %7, %9 : tensor<1x4x6xf32>
    %11 = stablehlo.exponential %10 : tensor<1x4x6xf32>
    %cst_2 = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %12 = stablehlo.reduce(%11 init: %cst_2) applies stablehlo.add across dimensions = [2] : (tensor<1x4x6xf32>, tensor<f32>) -> tensor<1x4xf32>
    %13 = stablehlo.broadcast_in_dim %12, dims = [0, 1] : (tensor<1x4xf32>) -> tensor<1x4x6xf32>
    %14 = stablehlo.divide %11, %13 : tensor<1x4x6xf32>
    %15 = stablehlo.dot_general %14, %arg2, batching_dims = [0] x [0], contracting_dims = [2] x [1] : (tensor<1x4x6xf32>, tensor<1x6x8xf32>) -> tensor<1x4x8xf32>
    return %15 : tensor<1x4x8xf32>
  }
}
"""

# embedding lookup, cache update, rotate-half, argmax with the value / index pair reduce
DECODE_PIECES = """
module @jit_step {
  func.func public @main(%arg0: tensor<16x8xbf16>, %arg1: tensor<2xi32>, %arg2: tensor<2x5x8xbf16> {tf.aliasing_output = 1 : i32}, %arg3: tensor<i32>) -> (tensor<2xi32>, tensor<2x5x8xbf16>) {
    %0 = "stablehlo.gather"(%arg0, %arg1) <{dimension_numbers = #stablehlo.gather<offset_dims = [1], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 1>, indices_are_sorted = false, slice_sizes = array<i64: 1, 8>}> : (tensor<16x8xbf16>, tensor<2xi32>) -> tensor<2x8xbf16>
    %1 = stablehlo.slice %0 [0:2, 0:4] : (tensor<2x8xbf16>) -> tensor<2x4xbf16>
    %2 = stablehlo.slice %0 [0:2, 4:8] : (tensor<2x8xbf16>) -> tensor<2x4xbf16>
    %3 = stablehlo.negate %2 : tensor<2x4xbf16>
    %4 = stablehlo.concatenate %3, %1, dim = 1 : (tensor<2x4xbf16>, tensor<2x4xbf16>) -> tensor<2x8xbf16>
    %5 = stablehlo.reshape %4 : (tensor<2x8xbf16>) -> tensor<2x1x8xbf16>
    %c = stablehlo.constant dense<0> : tensor<i32>
    %6 = stablehlo.dynamic_update_slice %arg2, %5, %c, %arg3, %c : (tensor<2x5x8xbf16>, tensor<2x1x8xbf16>, tensor<i32>, tensor<i32>, tensor<i32>) -> tensor<2x5x8xbf16>
    %7 = stablehlo.convert %4 : (tensor<2x8xbf16>) -> tensor<2x8xf32>
    %8 = stablehlo.iota dim = 1 : tensor<2x8xi32>
    %cst = stablehlo.constant dense<0xFF800000> : tensor<f32>
    %c_0 = stablehlo.constant dense<0> : tensor<i32>
    %9:2 = stablehlo.reduce(%7 init: %cst), (%8 init: %c_0) across dimensions = [1] : (tensor<2x8xf32>, tensor<2x8xi32>, tensor<f32>, tensor<i32>) -> (tensor<2xf32>, tensor<2xi32>)
     reducer(%arg4: tensor<f32>, %arg6: tensor<f32>) (%arg5: tensor<i32>, %arg7: tensor<i32>)  {
      %10 = stablehlo.compare  GT, %arg4, %arg6,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %11 = stablehlo.compare  NE, %arg4, %arg4,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %12 = stablehlo.or %10, %11 : tensor<i1>
      %13 = stablehlo.compare  EQ, %arg4, %arg6,  FLOAT : (tensor<f32>, tensor<f32>) -> tensor<i1>
      %14 = stablehlo.compare  LT, %arg5, %arg7,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %15 = stablehlo.and %13, %14 : tensor<i1>
      %16 = stablehlo.or %12, %15 : tensor<i1>
      %17 = stablehlo.select %16, %arg4, %arg6 : tensor<i1>, tensor<f32>
      %18 = stablehlo.select %16, %arg5, %arg7 : tensor<i1>, tensor<i32>
      stablehlo.return %17, %18 : tensor<f32>, tensor<i32>
    }
    return %9#1, %6 : tensor<2xi32>, tensor<2x5x8xbf16>
  }
}
"""


@pytest.fixture(scope="module")
def be():
    return pjrtx_b200.Backend()


def test_reference_importer_fixtures(be):
    b = be.import_stablehlo_text(REDUCE_GENERIC)
    assert [i.kind for i in b.instructions] == ["constant", "reduce_sum"] and be.verify_plan(b) == ""
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    assert np.array_equal(run_oracle(b, [x])[0], x.sum(axis=1))

    b = be.import_stablehlo_text(ADD_TANH)
    assert [i.kind for i in b.instructions] == ["add", "tanh"] and be.verify_plan(b) == ""
    a, c = np.array([0.5, 1], np.float32), np.array([0.25, -1], np.float32)
    assert_close(run_oracle(b, [a, c])[0], np.tanh(a + c), 1e-6)

    b = be.import_stablehlo_text(SHARDED_ARG)
    assert b.num_partitions == 2 and b.parameter_shardings[0][0] == P.PARTITIONED and b.parameter_shardings[0][2] == 0
    assert b.parameter_shardings[0][1] == "mesh"

    b = be.import_stablehlo_text(BARRIER)
    # the two-operand barrier becomes one barrier per operand
    assert [i.kind for i in b.instructions] == ["optimization_barrier", "optimization_barrier", "multiply"] and len(b.output_ids) == 2
    x, y = np.arange(4, dtype=np.float32), np.full(4, 2, np.float32)
    got = run_oracle(b, [x, y])
    assert np.array_equal(got[0], x * y) and np.array_equal(got[1], y)

    b = be.import_stablehlo_text(LEGACY_BROADCAST)
    assert [i.kind for i in b.instructions] == ["broadcast_in_dim"]
    assert np.array_equal(run_oracle(b, [np.array(3, np.float32)])[0], np.full(4, 3, np.float32))


def test_attention_module_as_jax_prints_it(be):
    b = be.import_stablehlo_text(ATTENTION)
    assert be.verify_plan(b) == ""
    kinds = [i.kind for i in b.instructions]
    assert kinds.count("dot_general") == 2 and "reduce_max" in kinds and "reduce_sum" in kinds and "iota" in kinds
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 4, 8), dtype=np.float32)
    k = rng.standard_normal((1, 6, 8), dtype=np.float32)
    v = rng.standard_normal((1, 6, 8), dtype=np.float32)
    for pos in (0, 3, 5):
        got = run_oracle(b, [q, k, v, np.array(pos, np.int32)])[0]
        s = np.einsum("bqd,bkd->bqk", q, k) * np.float32(0.353553385)
        s[:, :, pos + 1:] = -np.inf
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        assert_close(got, np.einsum("bqk,bkd->bqd", p, v), 1e-5, what=f"pos {pos}")
    # the backend sees the same plan a hand-built one would give: the kernel planner accepts it
    steps = be.describe_kernels(b)["steps"]
    assert [s["type"] for s in steps].count("dot") == 2


def test_decode_pieces_gather_cache_update_argmax(be):
    b = be.import_stablehlo_text(DECODE_PIECES)
    assert be.verify_plan(b) == ""
    assert b.donated == [2] and b.aliases == [(1, 2)]
    rng = np.random.default_rng(4)
    dt = P.np_dtype(P.BF16_CODE)
    table = rng.standard_normal((16, 8), dtype=np.float32).astype(dt)
    ids = np.array([5, 11], np.int32)
    cache = rng.standard_normal((2, 5, 8), dtype=np.float32).astype(dt)
    got = run_oracle(b, [table, ids, cache, np.array(3, np.int32)])
    rows = table[ids].astype(np.float32)
    rot = np.concatenate([-rows[:, 4:], rows[:, :4]], axis=1)
    assert np.array_equal(got[0], rot.argmax(axis=1).astype(np.int32))
    want_cache = cache.astype(np.float32).copy()
    want_cache[:, 3] = rot
    assert np.array_equal(got[1].astype(np.float32), want_cache)


@pytest.mark.parametrize("text,needle", [
    ("func.func @main(%arg0: tensor<f32>) -> tensor<f32> {\n  %0 = stablehlo.while(%iterArg = %arg0) : tensor<f32>\n cond { } do { }\n  return %0 : tensor<f32>\n}",
     "unsupported op: op=stablehlo.while loc=2:3 dtype=unknown rank=unknown sharding=unspecified feature=stablehlo-op"),
    ("func.func @main(%arg0: tensor<2xf32>) -> tensor<2xf32> {\n  %0 = \"stablehlo.sort\"(%arg0) ({\n  }) : (tensor<2xf32>) -> tensor<2xf32>\n  return %0 : tensor<2xf32>\n}",
     "unsupported op: op=stablehlo.sort loc=2:3"),
    ("func.func @main(%arg0: tensor<2xf32>) -> tensor<2xf32> {\n  %0 = chlo.erf %arg0 : tensor<2xf32> -> tensor<2xf32>\n  return %0 : tensor<2xf32>\n}",
     "unsupported op: op=chlo.erf loc=2:3"),
])
def test_operations_outside_the_subset_are_reported_in_the_reference_format(be, text, needle):
    with pytest.raises(BackendError) as err:
        be.import_stablehlo_text(text)
    assert needle in str(err.value) and "feature=stablehlo-op" in str(err.value)


def test_importable_but_not_executable_operations_fail_at_legalization(be):
    """The plan vocabulary is the reference's, so e.g. cholesky imports (stablehlo_import_tests.zig:275-300); the
    backend then refuses it with its own legalization diagnostic."""
    b = be.import_stablehlo_text('func.func @main(%arg0: tensor<2x2xf32>) -> tensor<2x2xf32> {\n  %1 = "stablehlo.cholesky"(%arg0) '
                                 '<{lower = true}> : (tensor<2x2xf32>) -> tensor<2x2xf32>\n  return %1 : tensor<2x2xf32>\n}')
    assert [i.kind for i in b.instructions] == ["cholesky"] and be.verify_plan(b) == ""
    with pytest.raises(BackendError, match="pass=b200-backend-legalization .*op=cholesky.* feature=b200-op"):
        be.describe_kernels(b)


def test_malformed_text_is_reported_with_a_location(be):
    with pytest.raises(BackendError, match=r"invalid module: loc=\d+:\d+ detail=.* feature=stablehlo-text"):
        be.import_stablehlo_text("func.func @main(%arg0: tensor<2xf32>) -> tensor<2xf32> {\n  %0 = stablehlo.add %arg0, %nope : tensor<2xf32>\n}")
    with pytest.raises(BackendError, match="no func.func @main"):
        be.import_stablehlo_text("module {\n}")


@pytest.mark.gpu
def test_imported_modules_run_on_the_gpu(gpu_backend):
    be = gpu_backend
    from tests.util import run_backend

    b = be.import_stablehlo_text(ATTENTION)
    rng = np.random.default_rng(3)
    args = [rng.standard_normal((1, 4, 8), dtype=np.float32), rng.standard_normal((1, 6, 8), dtype=np.float32),
            rng.standard_normal((1, 6, 8), dtype=np.float32), np.array(4, np.int32)]
    assert_close(run_backend(be, b, args)[0], run_oracle(b, args)[0], 1e-5, what="attention")

    b = be.import_stablehlo_text(DECODE_PIECES)
    dt = P.np_dtype(P.BF16_CODE)
    args = [rng.standard_normal((16, 8), dtype=np.float32).astype(dt), np.array([5, 11], np.int32),
            rng.standard_normal((2, 5, 8), dtype=np.float32).astype(dt), np.array(3, np.int32)]
    got, want = run_backend(be, b, args), run_oracle(b, args)
    assert np.array_equal(got[0], want[0])
    assert np.array_equal(got[1].view(np.uint16), want[1].view(np.uint16))
