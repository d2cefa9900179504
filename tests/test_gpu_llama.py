"""GPU parity of the Llama-shaped decode / prefill programs against the CPU oracle (teacher-forced)."""
import numpy as np
import pytest

from pjrtx_b200 import plan as P
from pjrtx_b200.programs import llama
from tests.util import assert_close, run_oracle

pytestmark = pytest.mark.gpu


def _decode_args(cfg, names, weights, caches, tokens, pos):
    return [np.asarray(tokens, np.int32), np.array(pos, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches


@pytest.mark.parametrize("batch", [1, 2, 16, 32])
def test_tiny_decode_steps_teacher_forced(gpu_backend, batch):
    """Four decode steps; every step the backend gets the oracle's token and caches' history.

    Logits: bf16 rel 2e-2 with max-abs error reported; next token: equal wherever the oracle's top-2 logits are
    further apart than the logit error; KV caches: bf16 rel 2e-2. The graph-replayed executable is reused across steps.
    """
    be = gpu_backend
    cfg = llama.TINY
    max_len, filled = 64, 40
    builder, names = llama.build_decode_step(cfg, batch, max_len, return_logits=True)
    weights = llama.make_weights(cfg, seed=0)
    caches = llama.make_kv_cache(cfg, batch, max_len, filled)
    exe = be.compile_executable(builder, [0])
    if batch > 2:  # batched decode projections run on the tensor cores
        dots = [s for s in exe.describe()["kernel_plan"]["steps"] if s["type"] == "dot"]
        assert dots and all(s["umma"] == 1 for s in dots), dots
    wbufs = [be.buffer_from_host(weights[n]) for n in names[2:2 + len(weights)]]
    cbufs = [be.buffer_from_host(c) for c in caches]
    tokens = np.arange(3, 3 + batch, dtype=np.int32)
    oracle_caches = caches
    worst = 0.0
    for step in range(4):
        pos = filled + step
        want = run_oracle(builder, _decode_args(cfg, names, weights, oracle_caches, tokens, pos))
        outs = be.execute_executable(exe, [be.buffer_from_host(tokens), be.buffer_from_host(np.array(pos, np.int32))] + wbufs + cbufs)
        got_tok, got_logits = outs[0].to_numpy(), outs[1].to_numpy()
        assert_close(got_logits, want[1], 2e-2, what=f"step {step} logits")
        err = float(np.max(np.abs(got_logits.astype(np.float32) - want[1].astype(np.float32))))
        worst = max(worst, err)
        ref = want[1].astype(np.float32)
        top2 = np.sort(ref, axis=1)[:, -2:]
        decisive = (top2[:, 1] - top2[:, 0]) > 2 * err
        assert np.array_equal(got_tok[decisive], want[0][decisive]), f"step {step}"
        for l, (g, w) in enumerate(zip(outs[2:], want[2:])):
            assert_close(g.to_numpy(), w, 2e-2, what=f"step {step} cache {l}")
        cbufs = outs[2:]                      # donated caches come back as outputs
        oracle_caches = want[2:]
        tokens = want[0]                      # teacher forcing
    stats = exe.stats()
    assert stats["execute_count"] == 4 and stats["donation_alias_output_count"] == 4 * 2 * cfg.layers
    assert stats["graph_capture_count"] == 1 and stats["graph_launch_count"] == 4
    print(f"logits max-abs error over 4 steps: {worst:.4e}")


@pytest.mark.parametrize("batch,chain", [(1, False), (2, False), (1, True), (2, True)])
def test_tiny_decode_with_transforms_folded_into_the_contractions(gpu_backend, monkeypatch, batch, chain):
    """The optional plan in which RMSNorm / SiLU run as lhs transforms of the streaming contractions and the residual
    additions as their epilogues, as separate launches and chained into one launch per layer (grid barriers between the
    segments): three teacher-forced steps against the oracle, replayed from one captured graph."""
    monkeypatch.setenv("PJRTX_B200_DOT_FUSE", "1")
    monkeypatch.setenv("PJRTX_B200_DOT_CHAIN", "1" if chain else "0")
    be = gpu_backend
    cfg = llama.TINY
    max_len, filled = 64, 40
    builder, names = llama.build_decode_step(cfg, batch, max_len, return_logits=True)
    weights = llama.make_weights(cfg, seed=0)
    caches = llama.make_kv_cache(cfg, batch, max_len, filled)
    exe = be.compile_executable(builder, [0])
    dots = [s for s in exe.describe()["kernel_plan"]["steps"] if s["type"] == "dot"]
    assert any(s.get("segments", 1) == (4 if chain else 1) and 1 in s.get("lhs_kinds", []) for s in dots), dots
    assert sum(s.get("residuals", 0) for s in dots) == 2 * cfg.layers
    wbufs = [be.buffer_from_host(weights[n]) for n in names[2:2 + len(weights)]]
    cbufs = [be.buffer_from_host(c) for c in caches]
    tokens = np.arange(3, 3 + batch, dtype=np.int32)
    oracle_caches = caches
    for step in range(3):
        pos = filled + step
        want = run_oracle(builder, _decode_args(cfg, names, weights, oracle_caches, tokens, pos))
        outs = be.execute_executable(exe, [be.buffer_from_host(tokens), be.buffer_from_host(np.array(pos, np.int32))] + wbufs + cbufs)
        assert_close(outs[1].to_numpy(), want[1], 2e-2, what=f"chain={chain} batch {batch} step {step} logits")
        cbufs = outs[2:]
        oracle_caches = want[2:]
        tokens = want[0]
    assert exe.stats()["graph_capture_count"] == 1


def test_argmax_of_decode_is_bit_exact_on_identical_logits(gpu_backend):
    """Greedy choice on the oracle's own logits must be the oracle's token, ties included."""
    from pjrtx_b200 import PlanBuilder
    from tests.util import run_backend

    rng = np.random.default_rng(4)
    logits = (rng.standard_normal((3, 1024), dtype=np.float32) * 0.05).astype(P.np_dtype(P.BF16_CODE))
    b = PlanBuilder()
    p = b.parameter(P.BF16_CODE, logits.shape)
    _, idx = b.argmax(p, 1)
    b.set_outputs([idx])
    assert np.array_equal(run_backend(gpu_backend, b, [logits])[0], run_oracle(b, [logits])[0])


def test_tiny_prefill(gpu_backend):
    be = gpu_backend
    cfg = llama.TINY
    batch, seq = 2, 32
    builder, names = llama.build_prefill(cfg, batch, seq)
    weights = llama.make_weights(cfg, seed=0)
    tokens = np.random.default_rng(2).integers(0, cfg.vocab, size=(batch, seq), dtype=np.int32)
    args = [tokens] + [weights[n] for n in names[1:]]
    want = run_oracle(builder, args)
    exe = be.compile_executable(builder, [0])
    outs = be.execute_executable(exe, [be.buffer_from_host(a) for a in args])
    for l, (g, w) in enumerate(zip(outs[1:], want[1:])):
        assert_close(g.to_numpy(), w, 2e-2, what=f"kv {l}")
    assert outs[0].to_numpy().shape == (batch,)


@pytest.mark.parametrize("batch,dtype", [(2, P.BF16_CODE), (16, P.BF16_CODE), (5, P.BF16_CODE), (16, P.F16)])
def test_int8_weight_only_decode(gpu_backend, monkeypatch, batch, dtype):
    """Dequantisation written as convert + multiply feeding dot_general. From three rows up the contractions read the
    bytes themselves (weights one byte wide in HBM; the tensor core contracts the integers and the column scales
    multiply the accumulators, which skips the rounding of every scaled weight to the element type); the result must
    be within tolerance of the oracle, which rounds as the program is written, and of the materialising path."""
    import dataclasses

    be = gpu_backend
    cfg = dataclasses.replace(llama.TINY, int8_weights=True, dtype=dtype)
    max_len, filled = 64, 40
    builder, names = llama.build_decode_step(cfg, batch, max_len, return_logits=True)
    weights = llama.make_weights(cfg, seed=0)
    caches = llama.make_kv_cache(cfg, batch, max_len, filled)
    tokens = (np.arange(batch, dtype=np.int32) * 37 + 5) % cfg.vocab
    args = [tokens, np.array(filled, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches
    want = run_oracle(builder, args)
    exe = be.compile_executable(builder, [0])
    dots = [s for s in exe.describe()["kernel_plan"]["steps"] if s["type"] == "dot"]
    assert all(s["rhs_s8"] == (1 if batch >= 3 else 0) for s in dots), dots
    outs = be.execute_executable(exe, [be.buffer_from_host(a) for a in args])
    logits = outs[1].to_numpy()
    assert_close(logits, want[1], 2e-2, what="int8 logits")
    if batch >= 3:
        monkeypatch.setenv("PJRTX_B200_FUSE_DEQUANT", "0")
        plain = be.compile_executable(builder, [0])
        assert all(s["rhs_s8"] == 0 for s in plain.describe()["kernel_plan"]["steps"] if s["type"] == "dot")
        ref = be.execute_executable(plain, [be.buffer_from_host(a) for a in args])[1].to_numpy()
        assert_close(logits, ref, 2e-2, what="in-kernel dequantisation vs materialised weights")


def test_unfused_attention_path_agrees(gpu_backend, monkeypatch):
    """The recognised attention step and the plain dot -> softmax -> dot steps give the same logits within tolerance."""
    be = gpu_backend
    cfg = llama.TINY
    batch, max_len, filled = 2, 64, 40
    builder, names = llama.build_decode_step(cfg, batch, max_len, return_logits=True)
    weights = llama.make_weights(cfg, seed=0)
    caches = llama.make_kv_cache(cfg, batch, max_len, filled)
    args = [np.array([5, 9], np.int32), np.array(filled, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches
    want = run_oracle(builder, args)
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("PJRTX_B200_FUSE_ATTENTION", flag)
        exe = be.compile_executable(builder, [0])
        kinds = [s["type"] for s in exe.describe()["kernel_plan"]["steps"]]
        assert (kinds.count("attention_decode") == cfg.layers) == (flag == "1")
        outs = be.execute_executable(exe, [be.buffer_from_host(a) for a in args])
        results.append(outs[1].to_numpy())
        assert_close(results[-1], want[1], 2e-2, what=f"logits fuse={flag}")
    assert_close(results[0], results[1], 2e-2, what="fused vs unfused")
