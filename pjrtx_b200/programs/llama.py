"""Llama-3-shaped decoder programs as executable plans.

These builders stand where `jax.jit` + the StableHLO importer stand in the
reference: they emit, op by op, the program a JAX Llama implementation lowers to
(RMSNorm as convert/multiply/reduce/rsqrt, RoPE as slice/negate/concatenate,
attention as dot_general → masked softmax → dot_general, SwiGLU, greedy argmax
as the two-operand reduce), with weights and KV caches as parameters and the
caches donated. Nothing here names a kernel: which ops fuse is decided by the
backend's planner. The reference's own model-shaped fixture is the llama-like
block of src/plugin/jax/jax_llama_like_inference.py:313-335.
"""
from __future__ import annotations

import dataclasses
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import plan as P
from ..plan import PlanBuilder, Val


@dataclasses.dataclass(frozen=True)
class LlamaConfig:
    layers: int
    d_model: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    eps: float = 1e-5
    rope_theta: float = 500000.0
    dtype: int = P.BF16_CODE
    int8_weights: bool = False  # weight-only int8 with per-output-channel f16 scales

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim


LLAMA3_8B = LlamaConfig(layers=32, d_model=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256)
LLAMA3_70B = LlamaConfig(layers=80, d_model=8192, heads=64, kv_heads=8, head_dim=128, ffn=28672, vocab=128256)
TINY = LlamaConfig(layers=2, d_model=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024)

LAYER_WEIGHTS = ("attn_norm", "wq", "wk", "wv", "wo", "mlp_norm", "w_gate", "w_up", "w_down")
LINEAR = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down", "lm_head")


def weight_shapes(cfg: LlamaConfig) -> List[Tuple[str, Tuple[int, ...]]]:
    """Parameter names and shapes in program order (without token, position and caches)."""
    out = [("embed", (cfg.vocab, cfg.d_model))]
    for l in range(cfg.layers):
        out += [
            (f"l{l}.attn_norm", (cfg.d_model,)), (f"l{l}.wq", (cfg.d_model, cfg.q_dim)),
            (f"l{l}.wk", (cfg.d_model, cfg.kv_dim)), (f"l{l}.wv", (cfg.d_model, cfg.kv_dim)),
            (f"l{l}.wo", (cfg.q_dim, cfg.d_model)), (f"l{l}.mlp_norm", (cfg.d_model,)),
            (f"l{l}.w_gate", (cfg.d_model, cfg.ffn)), (f"l{l}.w_up", (cfg.d_model, cfg.ffn)),
            (f"l{l}.w_down", (cfg.ffn, cfg.d_model)),
        ]
    out += [("final_norm", (cfg.d_model,)), ("lm_head", (cfg.d_model, cfg.vocab))]
    return out


def _is_linear(name: str) -> bool:
    return name.split(".")[-1] in LINEAR


def to_storage(x: np.ndarray, dtype_code: int) -> np.ndarray:
    """float32 -> storage dtype (round to nearest even)."""
    return x.astype(P.np_dtype(dtype_code))


_BLOCK_ELEMS = 1 << 22  # tensors are generated in row blocks of about this many elements, one RNG stream per block


def _row_blocks(shape) -> List[Tuple[int, int]]:
    rows = shape[0] if len(shape) > 1 else 1
    per_row = int(np.prod(shape[1:], dtype=np.int64)) if len(shape) > 1 else int(shape[0])
    step = max(1, _BLOCK_ELEMS // max(per_row, 1))
    return [(r, min(r + step, rows)) for r in range(0, rows, step)]


def make_weights(cfg: LlamaConfig, seed: int = 0, threads: int = 8, embed_period: int = 0) -> Dict[str, np.ndarray]:
    """Random-init weights ~N(0, 0.02) in the storage dtype (norm gains are 1 + N(0, 0.02)).

    `embed_period` > 0 fills the embedding table with a block of that many random rows repeated down the table (a
    decode step reads `batch` rows of it; full-width tests use this to keep host-side generation short).

    Each row block of each tensor draws from its own `default_rng([seed, index, block])`, so the values do not depend
    on how many threads generate them. With `int8_weights` linear weights are s8 ~U{-127..127} and `<name>.scale`
    holds per-output-channel f16 scales ~U(0.5, 1.5) * 0.02 * sqrt(3) / 127, which gives the dequantised weights the
    spread of the 16-bit initialisation (standard deviation about 0.02): with much larger weights the attention scores
    saturate the softmax and the logits amplify differences of one rounding in a weight.
    """
    dt = P.np_dtype(cfg.dtype)
    shapes = weight_shapes(cfg)
    out: Dict[str, np.ndarray] = {}
    jobs = []
    for index, (name, shape) in enumerate(shapes):
        quant = cfg.int8_weights and _is_linear(name)
        out[name] = np.empty(shape, dtype=np.int8 if quant else dt)
        if quant:
            out[name + ".scale"] = (np.random.default_rng([seed, index, 1 << 20]).uniform(0.5, 1.5, size=(shape[-1],)) * (0.02 * np.sqrt(3.0) / 127.0)).astype(np.float16)
        gen_shape = shape
        if name == "embed" and embed_period and embed_period < shape[0]:
            gen_shape = (embed_period,) + tuple(shape[1:])
        for block, (r0, r1) in enumerate(_row_blocks(gen_shape)):
            jobs.append((index, name, shape, quant, block, r0, r1))

    def gen(job):
        index, name, shape, quant, block, r0, r1 = job
        rng = np.random.default_rng([seed, index, block])
        sub = (r1 - r0,) + tuple(shape[1:]) if len(shape) > 1 else tuple(shape)
        dst = out[name][r0:r1] if len(shape) > 1 else out[name]
        if quant:
            dst[...] = rng.integers(-127, 128, size=sub, dtype=np.int8)
            return
        w = rng.standard_normal(size=sub, dtype=np.float32)
        w *= np.float32(0.02)
        if name.endswith("norm"):
            w += np.float32(1.0)
        dst[...] = to_storage(w, cfg.dtype)

    with ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
        list(pool.map(gen, jobs))
    if embed_period and "embed" in out and embed_period < out["embed"].shape[0]:
        table = out["embed"]
        for r0 in range(embed_period, table.shape[0], embed_period):
            n = min(embed_period, table.shape[0] - r0)
            table[r0:r0 + n] = table[:n]
    return out


def make_kv_cache(cfg: LlamaConfig, batch: int, max_len: int, filled: int, seed: int = 1) -> List[np.ndarray]:
    """Per layer K then V, [batch, max_len, kv_heads, head_dim], first `filled` positions ~N(0,1), rest zero."""
    dt = P.np_dtype(cfg.dtype)
    caches = []
    for l in range(cfg.layers):
        for which in range(2):
            rng = np.random.default_rng([seed, l, which])
            c = np.zeros((batch, max_len, cfg.kv_heads, cfg.head_dim), dtype=dt)
            if filled:
                c[:, :filled] = to_storage(rng.standard_normal(size=(batch, filled, cfg.kv_heads, cfg.head_dim), dtype=np.float32), cfg.dtype)
            caches.append(c)
    return caches


class _Emit:
    """Shared op sequences."""

    def __init__(self, b: PlanBuilder, cfg: LlamaConfig):
        self.b = b
        self.cfg = cfg

    def rms_norm(self, x: Val, w: Val) -> Val:
        b, cfg = self.b, self.cfg
        last = len(x.dims) - 1
        xf = b.convert(x, P.F32)
        ss = b.reduce("reduce_sum", xf * xf, [last])
        mean = ss * b.scalar_like(ss, np.float32(1.0 / x.dims[last]))
        r = b.unary("rsqrt", mean + b.scalar_like(mean, np.float32(cfg.eps)))
        rb = b.broadcast_in_dim(r, x.dims, list(range(last)))
        xn = b.convert(xf * rb, cfg.dtype)
        wb = b.broadcast_in_dim(w, x.dims, [last])
        return xn * wb

    def linear(self, x: Val, w: Val, scale: Optional[Val]) -> Val:
        """x @ W; with int8 weights the dequantisation is convert + multiply feeding the dot_general."""
        b, cfg = self.b, self.cfg
        if scale is not None:
            wf = b.convert(w, P.F16)
            wf = wf * b.broadcast_in_dim(scale, w.dims, [1])
            w = b.convert(wf, cfg.dtype) if cfg.dtype != P.F16 else wf
        return b.dot_general(x, w, [len(x.dims) - 1], [0])

    def rope_tables(self, positions: Val, lead_dims: Sequence[int], pos_axes: Sequence[int]) -> Tuple[Val, Val]:
        """cos/sin of shape lead_dims + [head_dim] in the model dtype; `positions` (s32) spans `pos_axes`."""
        b, cfg = self.b, self.cfg
        half = cfg.head_dim // 2
        inv_freq = (cfg.rope_theta ** (-np.arange(0, half, dtype=np.float64) * 2.0 / cfg.head_dim)).astype(np.float32)
        dims = list(lead_dims) + [half]
        pf = b.broadcast_in_dim(b.convert(positions, P.F32), dims, list(pos_axes))
        fr = b.broadcast_in_dim(b.constant(inv_freq), dims, [len(dims) - 1])
        ang = pf * fr
        ang2 = b.concatenate([ang, ang], len(dims) - 1)
        return b.convert(b.unary("cosine", ang2), cfg.dtype), b.convert(b.unary("sine", ang2), cfg.dtype)

    def rope(self, x: Val, cos: Val, sin: Val) -> Val:
        """x: [..., heads, head_dim]; cos/sin broadcast over the heads axis."""
        b, cfg = self.b, self.cfg
        half = cfg.head_dim // 2
        rank = len(x.dims)
        lo = b.slice(x, [0] * rank, list(x.dims[:-1]) + [half])
        hi = b.slice(x, [0] * (rank - 1) + [half], list(x.dims))
        rot = b.concatenate([-hi, lo], rank - 1)
        axes = list(range(rank - 2)) + [rank - 1]
        cb = b.broadcast_in_dim(cos, x.dims, axes)
        sb = b.broadcast_in_dim(sin, x.dims, axes)
        return x * cb + rot * sb

    def softmax_f32(self, s: Val, mask: Optional[Val]) -> Val:
        b = self.b
        last = len(s.dims) - 1
        if mask is not None:
            s = b.select(mask, s, b.scalar_like(s, np.float32(-np.inf)))
        m = b.reduce("reduce_max", s, [last])
        e = b.unary("exp", s - b.broadcast_in_dim(m, s.dims, list(range(last))))
        z = b.reduce("reduce_sum", e, [last])
        return e / b.broadcast_in_dim(z, s.dims, list(range(last)))


def build_decode_step(cfg: LlamaConfig, batch: int, max_len: int, num_partitions: int = 1,
                      return_logits: bool = False) -> Tuple[PlanBuilder, List[str]]:
    """One greedy decode step: (token[B], pos[], weights..., caches...) -> (next_token[B], [logits], caches...).

    Returns the builder and the parameter names in order. With `num_partitions > 1` the linear weights and
    caches carry Megatron-style split dimensions for the tensor-parallel planner.
    """
    b = PlanBuilder(num_partitions=num_partitions)
    e = _Emit(b, cfg)
    tp = num_partitions > 1
    B, D, H, G, hd, S = batch, cfg.d_model, cfg.heads, cfg.kv_heads, cfg.head_dim, max_len
    rep = H // G
    names: List[str] = ["token", "pos"]
    token = b.parameter(P.S32, [B])
    pos = b.parameter(P.S32, [])
    col = dict(sharding=P.PARTITIONED, split_dim=1, mesh="tp") if tp else {}
    row = dict(sharding=P.PARTITIONED, split_dim=0, mesh="tp") if tp else {}
    scale_split = dict(sharding=P.PARTITIONED, split_dim=0, mesh="tp") if tp else {}
    wdt = P.S8 if cfg.int8_weights else cfg.dtype
    params: Dict[str, Val] = {}

    def weight(name: str, shape, kind: str):
        linear = _is_linear(name)
        opts = {"col": col, "row": row, "none": {}}[kind]
        params[name] = b.parameter(wdt if linear else cfg.dtype, shape, **opts)
        names.append(name)
        if cfg.int8_weights and linear:
            # Scales follow the output channel: split with column-parallel weights, replicated for row-parallel ones.
            params[name + ".scale"] = b.parameter(P.F16, [shape[-1]], **(scale_split if kind == "col" else {}))
            names.append(name + ".scale")

    kinds = {"attn_norm": "none", "wq": "col", "wk": "col", "wv": "col", "wo": "row", "mlp_norm": "none",
             "w_gate": "col", "w_up": "col", "w_down": "row"}
    for name, shape in weight_shapes(cfg):
        short = name.split(".")[-1]
        if short == "embed" or short == "final_norm":
            weight(name, shape, "none")
        elif short == "lm_head":
            weight(name, shape, "col")
        else:
            weight(name, shape, kinds[short])
    cache_opts = dict(sharding=P.PARTITIONED, split_dim=2, mesh="tp") if tp else {}
    caches: List[Val] = []
    first_cache_param = len(names)
    for l in range(cfg.layers):
        for which in ("k", "v"):
            caches.append(b.parameter(cfg.dtype, [B, S, G, hd], **cache_opts))
            names.append(f"l{l}.{which}_cache")

    def sc(name):
        return params.get(name + ".scale")

    x = b.gather_rows(params["embed"], token)  # [B, D]
    cos, sin = e.rope_tables(pos, [], [])        # [hd]
    zero = b.constant(np.int32(0))
    key_pos = b.iota(P.S32, [B, G, rep, S], 3)
    visible = b.compare(key_pos, b.broadcast_in_dim(pos, [B, G, rep, S], []), P.LE)
    att_scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
    new_caches: List[Val] = []
    for l in range(cfg.layers):
        p = lambda n: params[f"l{l}.{n}"]
        h = e.rms_norm(x, p("attn_norm"))
        q = e.linear(h, p("wq"), sc(f"l{l}.wq"))
        k = e.linear(h, p("wk"), sc(f"l{l}.wk"))
        v = e.linear(h, p("wv"), sc(f"l{l}.wv"))
        q = e.rope(b.reshape(q, [B, H, hd]), b.broadcast_in_dim(cos, [B, hd], [1]), b.broadcast_in_dim(sin, [B, hd], [1]))
        k = e.rope(b.reshape(k, [B, G, hd]), b.broadcast_in_dim(cos, [B, hd], [1]), b.broadcast_in_dim(sin, [B, hd], [1]))
        kc = b.dynamic_update_slice(caches[2 * l], b.reshape(k, [B, 1, G, hd]), [zero, pos, zero, zero])
        vc = b.dynamic_update_slice(caches[2 * l + 1], b.reshape(v, [B, 1, G, hd]), [zero, pos, zero, zero])
        new_caches += [kc, vc]
        q4 = b.reshape(q, [B, G, rep, hd])
        scores = b.dot_general(q4, kc, [3], [3], [0, 1], [0, 2])  # [B, G, rep, S]
        sf = b.convert(scores, P.F32)
        sf = sf * b.scalar_like(sf, att_scale)
        probs = b.convert(e.softmax_f32(sf, visible), cfg.dtype)
        ctx = b.dot_general(probs, vc, [3], [1], [0, 1], [0, 2])  # [B, G, rep, hd]
        attn = e.linear(b.reshape(ctx, [B, H * hd]), p("wo"), sc(f"l{l}.wo"))
        x = x + attn
        h2 = e.rms_norm(x, p("mlp_norm"))
        gate = e.linear(h2, p("w_gate"), sc(f"l{l}.w_gate"))
        up = e.linear(h2, p("w_up"), sc(f"l{l}.w_up"))
        act = gate * b.unary("logistic", gate) * up
        x = x + e.linear(act, p("w_down"), sc(f"l{l}.w_down"))
    hf = e.rms_norm(x, params["final_norm"])
    logits = e.linear(hf, params["lm_head"], sc("lm_head"))  # [B, V]
    _, next_token = b.argmax(logits, 1)
    outs = [next_token] + ([logits] if return_logits else []) + new_caches
    base = 1 + (1 if return_logits else 0)
    donate = {base + i: first_cache_param + i for i in range(len(new_caches))}
    cache_out = (P.PARTITIONED, "tp", 2) if tp else (P.REPLICATED, "", -1)
    shardings = [(P.REPLICATED, "", -1)] * base + [cache_out] * len(new_caches)
    b.set_outputs(outs, donate=donate, shardings=shardings)
    return b, names


def build_prefill(cfg: LlamaConfig, batch: int, seq: int, last_only_logits: bool = True,
                  return_logits: bool = False) -> Tuple[PlanBuilder, List[str]]:
    """Prefill: (tokens[B,S], weights...) -> (next_token[B], [logits], k/v caches [B,S,G,hd] per layer).

    Causal attention is written as dot_general scores → masked softmax (max / sum reductions) → dot_general
    context, and the whole KV cache is an output. The LM head runs on the last position only when
    `last_only_logits` (what greedy decoding needs); otherwise on every position.
    """
    b = PlanBuilder()
    e = _Emit(b, cfg)
    B, S, D, H, G, hd = batch, seq, cfg.d_model, cfg.heads, cfg.kv_heads, cfg.head_dim
    rep = H // G
    names = ["tokens"]
    tokens = b.parameter(P.S32, [B, S])
    params: Dict[str, Val] = {}
    for name, shape in weight_shapes(cfg):
        params[name] = b.parameter(cfg.dtype, shape)
        names.append(name)
    x = b.reshape(b.gather_rows(params["embed"], b.reshape(tokens, [B * S])), [B, S, D])
    positions = b.iota(P.S32, [S], 0)
    cos, sin = e.rope_tables(positions, [S], [0])  # [S, hd]
    qi = b.iota(P.S32, [B, G, S, rep, S], 2)
    ki = b.iota(P.S32, [B, G, S, rep, S], 4)
    causal = b.compare(ki, qi, P.LE)
    att_scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
    outs_cache: List[Val] = []
    for l in range(cfg.layers):
        p = lambda n: params[f"l{l}.{n}"]
        h = e.rms_norm(x, p("attn_norm"))
        q = b.reshape(e.linear(h, p("wq"), None), [B, S, H, hd])
        k = b.reshape(e.linear(h, p("wk"), None), [B, S, G, hd])
        v = b.reshape(e.linear(h, p("wv"), None), [B, S, G, hd])
        cb = b.broadcast_in_dim(cos, [B, S, hd], [1, 2])
        sb = b.broadcast_in_dim(sin, [B, S, hd], [1, 2])
        q = e.rope(q, cb, sb)
        k = e.rope(k, cb, sb)
        outs_cache += [k, v]
        q5 = b.transpose(b.reshape(q, [B, S, G, rep, hd]), [0, 2, 1, 3, 4])  # [B, G, S, rep, hd]
        scores = b.dot_general(q5, k, [4], [3], [0, 1], [0, 2])              # [B, G, S, rep, S']
        sf = b.convert(scores, P.F32)
        sf = sf * b.scalar_like(sf, att_scale)
        probs = b.convert(e.softmax_f32(sf, causal), cfg.dtype)
        ctx = b.dot_general(probs, v, [4], [1], [0, 1], [0, 2])              # [B, G, S, rep, hd]
        ctx = b.reshape(b.transpose(ctx, [0, 2, 1, 3, 4]), [B, S, H * hd])
        x = x + e.linear(ctx, p("wo"), None)
        h2 = e.rms_norm(x, p("mlp_norm"))
        gate = e.linear(h2, p("w_gate"), None)
        up = e.linear(h2, p("w_up"), None)
        x = x + e.linear(gate * b.unary("logistic", gate) * up, p("w_down"), None)
    if last_only_logits:
        x = b.reshape(b.slice(x, [0, S - 1, 0], [B, S, D]), [B, D])
        logits = e.linear(e.rms_norm(x, params["final_norm"]), params["lm_head"], None)
        _, next_token = b.argmax(logits, 1)
    else:
        logits = e.linear(e.rms_norm(x, params["final_norm"]), params["lm_head"], None)  # [B, S, V]
        _, next_token = b.argmax(logits, 2)
    b.set_outputs([next_token] + ([logits] if return_logits else []) + outs_cache)
    return b, names
