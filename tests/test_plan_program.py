"""Host logic on CPU: C-ABI exports, plan verifier, program graph counters, legalization, kernel planner, codegen."""
import ctypes
import os
import re

import numpy as np
import pytest

from pjrtx_b200 import PlanBuilder
from pjrtx_b200 import backend as be_mod
from pjrtx_b200 import plan as P
from pjrtx_b200.programs import llama
from tests import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(backend):
    header = open(os.path.join(ROOT, "include", "pjrtx_b200.h")).read()
    declared = set(re.findall(r"\b(pjrtx_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    raw = ctypes.CDLL(be_mod.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} is declared in include/pjrtx_b200.h but not exported"
    assert declared == set(be_mod.SYMBOLS), declared ^ set(be_mod.SYMBOLS)


def test_capabilities_and_version(backend):
    caps = backend.capabilities()
    assert caps["name"] == "b200_cuda" and caps["supports_device_buffers"] and not caps["supports_unified_memory"]
    assert backend.lib.pjrtx_b200_version_major() == 0


def test_program_graph_matches_reference_counters(backend):
    """Same plan and same expectations as src/backend/mlx_metal/execution_call.zig:147-298."""
    b, _ = cases.u8_chain()
    d = backend.describe_program(b)
    assert d["node_count"] == 3 and d["schedule_item_count"] == 3 and d["value_count"] == 4 and d["edge_count"] == 3
    assert [s["kind"] for s in d["schedule"]] == ["node", "fusion_group", "materialization_boundary"]
    assert d["schedule"][1] == {"kind": "fusion_group", "index": 0, "count": 2}
    assert [n["kind"] for n in d["nodes"]] == ["constant", "elementwise", "elementwise"]
    assert [n["fusion_group"] for n in d["nodes"]] == [-1, 0, 0]
    g = d["fusion_groups"][0]
    assert (g["first_node"], g["last_node"], g["node_count"]) == (1, 2, 2)
    assert g["input_values"] == [0, 1] and g["output_values"] == [3]
    assert d["edges"] == [[1, 0, 1], [2, 1, 2], [1, 0, 2]]
    assert d["materialization_boundaries"] == [3]
    v = d["values"]
    assert v[0]["producer_node"] == -1 and v[0]["last_use_node"] == 1 and not v[0]["is_output"]
    assert v[1]["producer_node"] == 0 and v[1]["last_use_node"] == 2
    assert v[2]["producer_node"] == 1 and v[2]["last_use_node"] == 2
    assert v[3]["producer_node"] == 2 and v[3]["is_output"] and v[3]["materialization_boundary"] == 0
    assert d["planned_release_count"] == 1 and d["planned_release_bytes"] == 4
    assert d["peak_live_value_count"] == 4 and d["peak_live_bytes"] == 16


def test_fusion_groups_close_on_reductions_and_dots(backend):
    """Reference rule (program_build.zig:79-99, 224-263): reductions and dots never join a view+elementwise group."""
    b = PlanBuilder()
    x = b.parameter(P.F32, [4, 8])
    y = b.unary("exp", x * x)
    s = b.reduce("reduce_sum", y, [1])
    z = b.unary("sqrt", s)
    w = b.matmul(b.reshape(z, [1, 4]), b.transpose(x, [0, 1]))
    b.set_outputs([w])
    d = backend.describe_program(b)
    kinds = [n["kind"] for n in d["nodes"]]
    assert kinds == ["elementwise", "elementwise", "reduction", "elementwise", "view", "view", "matmul"]
    assert [n["fusion_group"] for n in d["nodes"]] == [0, 0, -1, 1, 1, 1, -1]
    assert d["fusion_group_count"] == 2


def test_plan_verifier_diagnostics(backend):
    b = PlanBuilder()
    x = b.parameter(P.F32, [4])
    b.set_outputs([x + x])
    assert backend.verify_plan(b) == ""
    # use before definition
    bad = PlanBuilder()
    p = bad.parameter(P.F32, [4])
    out = bad._value(P.ROLE_RESULT, P.F32, [4])
    later = bad._value(P.ROLE_RESULT, P.F32, [4])
    bad.instructions.append(P.Instr("add", [p.id, later.id], [out.id], {}))
    bad.instructions.append(P.Instr("negate", [p.id], [later.id], {}))
    bad.set_outputs([out])
    msg = backend.verify_plan(bad)
    assert msg.startswith("invalid executable plan: pass=pjrtx-plan-verify instruction=0 value=2")
    assert "feature=value-graph" in msg
    # arity
    bad2 = PlanBuilder()
    p = bad2.parameter(P.F32, [4])
    o = bad2._value(P.ROLE_RESULT, P.F32, [4])
    bad2.instructions.append(P.Instr("add", [p.id], [o.id], {}))
    bad2.set_outputs([o])
    assert "feature=instruction-arity" in backend.verify_plan(bad2)
    # alias to a parameter that is not donated
    bad3 = PlanBuilder()
    p = bad3.parameter(P.F32, [4])
    bad3.set_outputs([p + p])
    bad3.aliases = [(0, 0)]
    assert "feature=donation-alias" in backend.verify_plan(bad3)
    # topology
    bad4 = PlanBuilder(num_partitions=2, device_assignment=[0])
    p = bad4.parameter(P.F32, [4])
    bad4.set_outputs([p + p])
    assert "feature=topology" in backend.verify_plan(bad4)


def test_legalization_diagnostics(backend):
    """Format of src/backend/mlx_metal/lowering_diagnostic.zig:31-45; unknown custom call reports its target as the feature."""
    b = PlanBuilder()
    x = b.parameter(P.F32, [4])
    b.set_outputs([b.custom_call("my.unknown.target", [x], P.F32, [4])])
    msg = backend.write_executable_lowering_diagnostic(b)
    assert msg.startswith("invalid executable plan: pass=b200-backend-legalization instruction=0 op=custom_call")
    assert msg.endswith("feature=my.unknown.target") and "dtype=f32 rank=1 shape=[4] sharding=internal" in msg
    # mixed-type dot is rejected: dequantisation must be convert + multiply feeding a same-type dot
    b = PlanBuilder()
    x = b.parameter(P.F16, [2, 4])
    w = b.parameter(P.S8, [4, 3])
    b._emit("dot_general", [x, w], P.F16, [2, 3], {"lhs_contracting_dimensions": [1], "rhs_contracting_dimensions": [0],
                                                   "lhs_batch_dimensions": [], "rhs_batch_dimensions": []})
    b.set_outputs([P.Val(b, len(b.values) - 1)])
    assert "feature=b200-dot-general" in backend.write_executable_lowering_diagnostic(b)
    # complex is out of scope
    b = PlanBuilder()
    x = b.parameter(P.C64, [2])
    b.set_outputs([b._emit("negate", [x], P.C64, [2])])
    assert "feature=b200-element-type" in backend.write_executable_lowering_diagnostic(b)
    # no device
    ok = PlanBuilder()
    x = ok.parameter(P.F32, [4])
    ok.set_outputs([x + x])
    assert backend.write_executable_lowering_diagnostic(ok, 1) == ""
    assert "feature=b200-device-assignment" in backend.write_executable_lowering_diagnostic(ok, 0)


def test_registered_custom_calls_become_fusible(backend):
    v0 = backend.custom_call_registry_version()
    backend.register_custom_call("test.unary.sqrt", "sqrt", 1)
    backend.register_custom_call("test.identity", "identity", 1)
    assert backend.custom_call_registry_version() == v0 + 2
    b = PlanBuilder()
    x = b.parameter(P.F32, [8])
    y = b.custom_call("test.unary.sqrt", [x], P.F32, [8])
    b.set_outputs([b.custom_call("test.identity", [y + y], P.F32, [8])])
    k = backend.describe_kernels(b)
    assert [s["type"] for s in k["steps"]] == ["fused"] and "sqrtf" in k["steps"][0]["source"]
    backend.unregister_custom_call("test.unary.sqrt")
    backend.unregister_custom_call("test.identity")
    assert "feature=test.unary.sqrt" in backend.write_executable_lowering_diagnostic(b)
    with pytest.raises(be_mod.BackendError):
        backend.register_custom_call("test.bad", "dot_general", 2)


def test_config1_is_one_row_kernel_and_compiles(backend):
    b, _ = cases.op_suite_config1(rows=64, cols=4096)
    k = backend.describe_kernels(b)
    assert len(k["steps"]) == 1
    st = k["steps"][0]
    assert st["row"] and st["rows"] == 64 and st["cols"] == 4096 and st["reduces"] == 3 and st["vec"] == 4
    assert st["inputs"] == 2 and st["outputs"] == 3
    assert "ldvec<float, 4>" in st["source"] and "block_reduce" in st["source"] and "arg_better" in st["source"]
    assert backend.compile_check(st["source"]) == ""


def test_decode_step_chains_the_streaming_contractions(backend, monkeypatch):
    """Small-batch decode with PJRTX_B200_DOT_FUSE / _CHAIN on: the RMSNorm and SiLU kernels become lhs transforms of the
    contractions they feed, the residual additions become epilogues, and o_proj -> gate/up -> down_proj -> next layer's
    q/k/v run as one launch."""
    monkeypatch.setenv("PJRTX_B200_DOT_FUSE", "1")
    monkeypatch.setenv("PJRTX_B200_DOT_CHAIN", "1")
    cfg = llama.TINY
    b, names = llama.build_decode_step(cfg, 2, 64)
    k = backend.describe_kernels(b)
    types = [s["type"] for s in k["steps"]]
    dots = [s for s in k["steps"] if s["type"] == "dot"]
    # first q/k/v alone (its norm also gathers the embedding rows), then one chain per layer
    assert len(dots) == cfg.layers + 1
    assert dots[0]["group"] == 3 and "segments" not in dots[0]
    for layer, d in enumerate(dots[1:]):
        assert d["segments"] == 4 and d["lhs_kinds"] == [0, 1, 2, 1] and d["residuals"] == 2
        last = layer == cfg.layers - 1
        per_layer = cfg.q_dim * cfg.d_model + 3 * cfg.d_model * cfg.ffn
        tail = cfg.d_model * cfg.vocab if last else cfg.d_model * (cfg.q_dim + 2 * cfg.kv_dim)
        assert d["weight_elems"] == per_layer + tail
    # three launches per layer (rotation + cache rows, attention, chain) plus embedding/tables, first norm, first q/k/v, argmax
    assert types.count("attention_decode") == cfg.layers and len(types) == 3 * cfg.layers + 4
    for src in {s["source"] for s in k["steps"] if s["type"] == "fused"}:
        assert backend.compile_check(src) == ""


def test_decode_step_kernel_plan(backend, monkeypatch):
    cfg = llama.TINY
    b, names = llama.build_decode_step(cfg, 2, 64)
    assert backend.verify_plan(b) == ""
    k = backend.describe_kernels(b)
    types = [s["type"] for s in k["steps"]]
    # per layer: q/k/v as one grouped launch, o_proj, gate/up as one grouped launch, down_proj; the
    # scores -> masked softmax -> context chain is recognised and becomes one split-KV attention step
    dots = [s for s in k["steps"] if s["type"] == "dot"]
    assert len(dots) == 4 * cfg.layers + 1
    assert sum(1 for s in dots if s["group"] == 3 and s["n"] == cfg.q_dim + 2 * cfg.kv_dim) == cfg.layers
    assert sum(1 for s in dots if s["group"] == 2 and s["n"] == 2 * cfg.ffn) == cfg.layers
    # every projection streams its weights through a TMA-fed persistent kernel: tensor cores for 16-bit floats
    assert all(s["path"] == 1 and (s["umma"] == 1 or s["tma"] == 1) for s in dots)
    assert types.count("attention_decode") == cfg.layers
    # the in-place KV-cache updates ride in the kernel that rotates q and k: no separate slice_update launches, and
    # nine launches per layer (norm, qkv, rope + cache rows, attention, o_proj, norm, gate/up, silu*up, down_proj)
    assert types.count("slice_update") == 0
    assert len(types) <= 9 * cfg.layers + 4
    fused = [s for s in k["steps"] if s["type"] == "fused"]
    assert sum(1 for s in fused if "dst1" in s["source"]) == cfg.layers
    # RMSNorm (+ residual add) is a single row kernel, so is the argmax over the vocabulary
    assert sum(1 for s in fused if s["row"] and s["cols"] == cfg.d_model) == 2 * cfg.layers + 1
    assert sum(1 for s in fused if s["row"] and s["cols"] == cfg.vocab) == 1
    for src in {s["source"] for s in fused}:
        assert backend.compile_check(src) == ""
    # with the slice-update fusion off the cache rows are written by their own in-place launches
    monkeypatch.setenv("PJRTX_B200_FUSE_SLICE_UPDATE", "0")
    k1 = backend.describe_kernels(b)
    assert [s["type"] for s in k1["steps"]].count("slice_update") == 2 * cfg.layers
    assert all(s["in_place"] for s in k1["steps"] if s["type"] == "slice_update")
    monkeypatch.delenv("PJRTX_B200_FUSE_SLICE_UPDATE")
    # without the recognition the same program runs as dot -> one softmax row kernel -> dot
    monkeypatch.setenv("PJRTX_B200_FUSE_ATTENTION", "0")
    k2 = backend.describe_kernels(b)
    types2 = [s["type"] for s in k2["steps"]]
    assert types2.count("attention_decode") == 0 and types2.count("dot") == 6 * cfg.layers + 1
    assert sum(1 for s in k2["steps"] if s["type"] == "fused" and s["row"] and s["cols"] == 64 and s["reduces"] == 2) == cfg.layers


def test_all_cases_plan_and_compile(backend):
    names = ["u8_chain", "dot_rhs_transposed", "dot_batched", "attention_scores_context", "argmax_ties", "sdpa_single",
             "sdpa_gqa", "sdpa_random", "elementwise_float_chain", "reshape_transpose_broadcast", "reduce_cases",
             "float_unary_math", "is_finite_case", "int_ops", "i8_negate_sub", "predicate_logic", "structural_ops",
             "matmul_small"]
    for name in names:
        b, _ = getattr(cases, name)()
        assert backend.verify_plan(b) == "", name
        k = backend.describe_kernels(b)
        for s in k["steps"]:
            if s["type"] == "fused":
                log = backend.compile_check(s["source"])
                assert log == "", f"{name}: {log[:800]}"


def test_tensor_parallel_partition_plan(backend):
    cfg = llama.TINY
    b, names = llama.build_decode_step(cfg, 2, 64, num_partitions=2)
    for part in range(2):
        k = backend.describe_kernels(b, partition=part)
        types = [s["type"] for s in k["steps"]]
        assert types.count("all_reduce") == 2 * cfg.layers       # after o_proj and down_proj
        assert types.count("all_gather") == 1                     # vocabulary-split logits before argmax
        dots = [s for s in k["steps"] if s["type"] == "dot"]
        assert any(s["n"] == (cfg.q_dim + 2 * cfg.kv_dim) // 2 for s in dots) and any(s["k"] == cfg.ffn // 2 for s in dots)


def test_execute_requires_gpu_and_fails_loudly(backend):
    if backend.lib.pjrtx_b200_device_count() > 0:
        pytest.skip("a device is present")
    b, _ = cases.u8_chain()
    with pytest.raises(be_mod.BackendError):
        backend.compile_executable(b, [0])
    with pytest.raises(be_mod.BackendError):
        backend.buffer_from_host(np.zeros(4, np.float32))


def test_prefill_attention_is_one_kernel(backend, monkeypatch):
    """The rank-5 causal chain (scores -> masked softmax -> context) of the prefill program maps onto the prefill
    attention kernel: scores and probabilities are never stored. Shapes the kernel does not cover, and the switch,
    leave the chain as written."""
    b, _ = cases.prefill_attention()
    steps = backend.describe_kernels(b)["steps"]
    assert [s["type"] for s in steps] == ["attention_prefill"]
    assert (steps[0]["batch"], steps[0]["kv_heads"], steps[0]["rep"], steps[0]["seq"], steps[0]["head_dim"]) == (2, 2, 4, 96, 64)
    b32, _ = cases.prefill_attention(head_dim=32)                   # head_dim outside {64, 128}
    assert "attention_prefill" not in [s["type"] for s in backend.describe_kernels(b32)["steps"]]
    bf, _ = cases.prefill_attention(dtype=P.F32)                    # 32-bit elements
    assert "attention_prefill" not in [s["type"] for s in backend.describe_kernels(bf)["steps"]]
    cfg = llama.TINY
    pb, _ = llama.build_prefill(cfg, 2, 24)
    types = [s["type"] for s in backend.describe_kernels(pb)["steps"]]
    assert types.count("attention_prefill") == cfg.layers
    assert types.count("dot") == 4 * cfg.layers + 1                 # q/k/v, o, gate/up, down (+ LM head)
    monkeypatch.setenv("PJRTX_B200_ATTENTION_PREFILL", "0")
    types0 = [s["type"] for s in backend.describe_kernels(pb)["steps"]]
    assert types0.count("attention_prefill") == 0 and types0.count("dot") == 6 * cfg.layers + 1


def test_partitioned_decode_keeps_attention_recognisable(backend):
    """Splatted scale / mask operands are rebuilt at the local shape, not sliced out of full-size tensors, so every
    partition still maps its attention block onto the split-KV kernel and carries no full-size mask."""
    cfg = llama.TINY
    b, _ = llama.build_decode_step(cfg, 2, 64, num_partitions=2)
    for part in range(2):
        k = backend.describe_kernels(b, partition=part)
        kinds = [s["type"] for s in k["steps"]]
        assert kinds.count("attention_decode") == cfg.layers
        assert kinds.count("all_reduce") == 2 * cfg.layers and kinds.count("all_gather") == 1


def test_plan_fingerprint_is_stable_and_sensitive(backend):
    """Cache key: equal for equal plans, different when an attribute, a constant, a donation or the custom-call
    registry changes (the fields of src/runtime/executable_fingerprint.zig:9-140)."""
    import re

    def build(scale=0.5, perm=(1, 0), donate=None):
        b = PlanBuilder()
        x = b.parameter(P.F32, [4, 8])
        y = b.transpose(x * np.float32(scale), list(perm))
        b.set_outputs([y], donate=donate)
        return b

    a = backend.plan_fingerprint(build())
    assert re.fullmatch(r"pjrtx-[0-9a-f]{16}", a)
    assert backend.plan_fingerprint(build()) == a
    assert backend.plan_fingerprint(build(scale=0.25)) != a
    c = PlanBuilder()
    x = c.parameter(P.F32, [4, 8])
    c.set_outputs([c.reshape(x * np.float32(0.5), [8, 4])])
    assert backend.plan_fingerprint(c) != a
    version = backend.lib.pjrtx_b200_custom_call_registry_version()
    assert backend.lib.pjrtx_b200_register_custom_call(b"tests.fingerprint.identity", b"identity", 1)
    try:
        assert backend.lib.pjrtx_b200_custom_call_registry_version() != version
        assert backend.plan_fingerprint(build()) != a
    finally:
        backend.lib.pjrtx_b200_unregister_custom_call(b"tests.fingerprint.identity")


def test_decode_attention_kernel_choice_and_grid(backend, monkeypatch):
    """Planner rules of the decode attention step (device independent, 148 SMs assumed): 16-bit caches with 4 or 8
    query heads per KV head, head size 64 / 128 and at least one 64-key stage go to the tensor-core kernel with one
    wave of two CTAs per SM and no split shorter than 128 keys; a shorter buffer, f32 caches or another head ratio go to
    the CUDA-core kernel, which keeps to one wave of one CTA per SM when there are fewer (sequence, KV head) pairs
    than SMs."""
    from pjrtx_b200 import PlanBuilder

    monkeypatch.delenv("PJRTX_B200_ATTENTION_MMA", raising=False)
    monkeypatch.delenv("PJRTX_B200_ATTENTION_STAGED", raising=False)
    monkeypatch.delenv("PJRTX_B200_ATTENTION_SPLITS", raising=False)

    def plan_of(dtype, batch, heads, kv_heads, hd, kv_len):
        b = PlanBuilder()
        pq = b.parameter(dtype, [batch, 1, heads, hd])
        pk = b.parameter(dtype, [batch, kv_len, kv_heads, hd])
        pv = b.parameter(dtype, [batch, kv_len, kv_heads, hd])
        pt = b.parameter(P.S32, [])
        b.set_outputs([b.custom_call("pjrtx.b200.scaled_dot_product_attention", [pq, pk, pv, pt], dtype, [batch, 1, heads, hd])])
        steps = backend.describe_kernels(b)["steps"]
        assert [s["type"] for s in steps] == ["attention_decode"]
        return steps[0]

    # 8B shape at batch 1: 8 pairs, 2304-key buffer -> tensor-core kernel, 18 splits of 128 keys (144 CTAs <= 296)
    st = plan_of(P.BF16_CODE, 1, 32, 8, 128, 2304)
    assert st["mma"] == 1 and st["splits"] == 18
    # the same with a longer buffer: as many splits as one wave of two CTAs per SM holds (296 // 8 = 37), at most kv_len // 128
    st = plan_of(P.BF16_CODE, 1, 32, 8, 128, 3744)
    assert st["mma"] == 1 and st["splits"] == 29
    # 256 pairs (batch 32): one split each
    st = plan_of(P.BF16_CODE, 32, 32, 8, 128, 2304)
    assert st["mma"] == 1 and st["splits"] == 1
    # one eighth of the 70B shape: 32 pairs -> 9 splits
    st = plan_of(P.BF16_CODE, 32, 8, 1, 128, 4352)
    assert st["mma"] == 1 and st["splits"] == 9
    # a buffer shorter than a stage, f32 caches, two heads per KV head: CUDA-core kernel
    assert plan_of(P.BF16_CODE, 2, 16, 4, 128, 40)["mma"] == 0
    assert plan_of(P.F32, 2, 8, 2, 64, 512)["mma"] == 0
    assert plan_of(P.F16, 2, 8, 4, 64, 512)["mma"] == 0
    # CUDA-core kernel with fewer pairs than SMs: one wave (148 // 8 = 18 splits, not 29)
    monkeypatch.setenv("PJRTX_B200_ATTENTION_MMA", "0")
    st = plan_of(P.BF16_CODE, 1, 32, 8, 128, 3744)
    assert st["mma"] == 0 and st["splits"] == 18
