"""Shared helpers: run a plan through the C ABI and through the CPU oracle."""
import numpy as np

from oracle import plan_interp
from pjrtx_b200 import plan as P


def run_backend(be, builder, args, device=0, partition=None, exe=None):
    own = exe is None
    if exe is None:
        exe = be.compile_executable(builder, [device], partition=partition)
    bufs = [be.buffer_from_host(a, device) for a in args]
    outs = be.execute_executable(exe, bufs)
    res = [o.to_numpy() for o in outs]
    for b in bufs + outs:
        b.destroy()
    if own:
        exe.destroy()
    return res


def run_oracle(builder, args):
    return plan_interp.run_plan(builder, args)


def f64(a):
    return np.asarray(a).astype(np.float64)


def assert_close(got, want, rtol, atol_scale=None, what=""):
    """|got - want| <= atol + rtol*|want| with atol = rtol * (max |want| unless given)."""
    g, w = f64(got), f64(want)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    scale = float(np.max(np.abs(w[np.isfinite(w)]))) if atol_scale is None and np.isfinite(w).any() else (atol_scale or 1.0)
    atol = rtol * max(scale, 1e-30)
    both_nan = np.isnan(g) & np.isnan(w)
    same_inf = np.isinf(w) & (g == w)
    err = np.abs(g - w)
    ok = both_nan | same_inf | (err <= atol + rtol * np.abs(w))
    if not ok.all():
        bad = np.argwhere(~ok)[0]
        raise AssertionError(f"{what}: {(~ok).sum()} of {ok.size} outside rtol={rtol} atol={atol:g}; first at {tuple(bad)} "
                             f"got={g[tuple(bad)]!r} want={w[tuple(bad)]!r} max_err={np.nanmax(np.where(np.isfinite(err), err, 0))}")


TOL = {P.F32: 1e-5, P.F16: 2e-2, P.BF16_CODE: 2e-2}


def assert_outputs(builder, got, want, what=""):
    """Integers / predicates bit-exact; f32 rel 1e-5; f16/bf16 rel 2e-2 (atol = rtol * max|want|)."""
    assert len(got) == len(want)
    for k, (g, w, vid) in enumerate(zip(got, want, builder.output_ids)):
        code = builder.values[vid].dtype
        if code in TOL:
            assert_close(g, w, TOL[code], what=f"{what} output {k}")
        else:
            assert g.dtype == w.dtype and np.array_equal(g, w), f"{what} output {k}: integer results differ"
