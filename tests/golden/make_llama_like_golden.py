"""Generates tests/golden/llama_like_*.npz from the reference's own NumPy reference.

Run where a checkout of the reference is available, giving its root:
    python tests/golden/make_llama_like_golden.py <reference checkout>
It imports src/plugin/jax/jax_llama_like_inference.py (its `make_fixture` and `np_reference`, :206-252), evaluates
the two fixtures the reference's test uses (seed default_rng(7); shapes (2,4,8) and (4,16,32), :439-441) and stores
inputs and expected outputs. Machines that run the tests have no reference checkout, so the vectors are committed.
"""
import importlib.util
import os
import sys

import numpy as np


def main(reference_root: str) -> None:
    path = os.path.join(reference_root, "src/plugin/jax/jax_llama_like_inference.py")
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location("ref_llama_like", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    here = os.path.dirname(os.path.abspath(__file__))
    rng = np.random.default_rng(7)
    for name, (seq, dim, ff) in (("tiny", (2, 4, 8)), ("medium", (4, 16, 32))):
        fixture = mod.make_fixture(rng, seq, dim, ff)
        want = mod.np_reference(*fixture)
        keys = ("x", "norm_w", "wq", "wk", "wv", "wo", "w1", "w2", "w3")
        np.savez(os.path.join(here, f"llama_like_{name}.npz"), expected=want, **dict(zip(keys, fixture)))
        print(name, want.shape, float(np.abs(want).max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_llama_like_golden.py <reference checkout>")
    main(sys.argv[1])
