"""Tensor-parallel planner checked numerically on CPU: two or four gloo ranks interpret their partition plans with the oracle,
exchanging all_reduce / all_gather over torch.distributed, and must reproduce the unpartitioned program."""
import os
import socket

import numpy as np
import pytest

from pjrtx_b200 import plan as P
from pjrtx_b200.programs import llama


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard(arr, split_dim, rank, world):
    if split_dim < 0:
        return arr
    n = arr.shape[split_dim] // world
    return np.ascontiguousarray(np.take(arr, range(rank * n, (rank + 1) * n), axis=split_dim))


def _config(world, int8):
    """Two KV heads shard over two ranks; more ranks get a copy with as many KV heads as ranks."""
    import dataclasses

    cfg = dataclasses.replace(llama.TINY, int8_weights=int8)
    return cfg if world <= 2 else dataclasses.replace(cfg, heads=2 * world, kv_heads=world)


def _worker(rank, world, port, int8, queue):
    import torch
    import torch.distributed as dist

    from oracle import plan_interp
    from pjrtx_b200 import Backend

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = _config(world, int8)
        batch, max_len, filled = 2, 32, 20
        full, names = llama.build_decode_step(cfg, batch, max_len, num_partitions=world, return_logits=True)
        weights = llama.make_weights(cfg, seed=0)
        caches = llama.make_kv_cache(cfg, batch, max_len, filled)
        args = [np.array([5, 9], np.int32), np.array(filled, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches
        part = Backend().partition_plan(full, rank)
        local = [_shard(a, sh[2] if sh[0] == P.PARTITIONED else -1, rank, world) for a, sh in zip(args, full.parameter_shardings)]

        def all_reduce(x, code):
            t = torch.from_numpy(np.asarray(x).astype(np.float32))
            dist.all_reduce(t)
            return t.numpy().astype(P.np_dtype(code))  # the collective sums in f32 and rounds once, like NCCL's bf16 ring does not; tolerance covers it

        def all_gather(x, code):
            t = torch.from_numpy(np.ascontiguousarray(np.asarray(x).view(np.uint8)))
            out = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(out, t)
            return np.stack([o.numpy().view(P.np_dtype(code)).reshape(x.shape) for o in out])

        got = plan_interp.run_plan(part, local, all_reduce=all_reduce, all_gather=all_gather)
        want = plan_interp.run_plan(full, args) if rank == 0 else None
        queue.put((rank, [np.asarray(g).astype(np.float32) if g.dtype.kind not in "iub" else g for g in got],
                   [np.asarray(w).astype(np.float32) if w.dtype.kind not in "iub" else w for w in want] if want else None,
                   [s["type"] if isinstance(s, dict) else s for s in []]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,int8", [(2, False), (2, True), (4, False)])
def test_partition_plans_reproduce_the_full_program(world, int8):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, int8, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, got, want, _ = queue.get(timeout=180)
        results[rank] = (got, want)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = results[0][1]
    cfg = _config(world, int8)
    for rank in range(world):
        got = results[rank][0]
        # logits are replicated after the all_gather; caches stay split along the KV-head axis
        scale = float(np.abs(want[1]).max())
        assert np.abs(got[1] - want[1]).max() <= 2e-2 * scale + 2e-2 * scale
        assert got[0].shape == want[0].shape
        for l in range(2 * cfg.layers):
            full_cache = want[2 + l]
            half = cfg.kv_heads // world
            np.testing.assert_allclose(got[2 + l], full_cache[:, :, rank * half:(rank + 1) * half], rtol=2e-2, atol=2e-2 * np.abs(full_cache).max())
    # every rank agrees on the greedy token
    for rank in range(1, world):
        assert np.array_equal(results[0][0][0], results[rank][0][0])
