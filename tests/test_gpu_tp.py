"""Tensor parallelism on real GPUs: one process per GPU, NCCL all_reduce / all_gather inside the executable.

Each rank compiles its partition of the tiny Llama-shaped decode step, feeds its own weight and cache shards, and must
reproduce the CPU oracle's logits of the unpartitioned program; once with NCCL's all-reduce, once with the one-kernel
all-reduce over peer-mapped memory. Skipped when fewer than two GPUs are visible.
NVLS is switched off so that a rank that dies mid-test leaves nothing bound inside the switch.
"""
import dataclasses
import os
import socket

import numpy as np
import pytest

from pjrtx_b200 import plan as P
from pjrtx_b200.programs import llama

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard(arr, split_dim, rank, world):
    if split_dim < 0:
        return arr
    n = arr.shape[split_dim] // world
    return np.ascontiguousarray(np.take(arr, range(rank * n, (rank + 1) * n), axis=split_dim))


def _worker(rank, world, port, batch, peer, queue, int8=False):
    import torch.distributed as dist

    import pjrtx_b200

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        _run_rank(rank, world, batch, peer, queue, dist, pjrtx_b200, int8)
    except Exception:  # report instead of leaving the parent to wait for its timeout
        import traceback

        queue.put((rank, "error", traceback.format_exc()))
        raise
    finally:
        dist.destroy_process_group()


def _config(world, int8=False):
    """Two KV heads shard over two ranks; four ranks get a copy with twice the heads. `int8`: weight-only int8 linear
    layers with f16 column scales (the scales shard with the columns they belong to)."""
    cfg = llama.TINY if world <= 2 else dataclasses.replace(llama.TINY, heads=2 * world, kv_heads=world)
    return dataclasses.replace(cfg, int8_weights=True) if int8 else cfg


def _run_rank(rank, world, batch, peer, queue, dist, pjrtx_b200, int8=False):
    if True:
        be = pjrtx_b200.Backend()
        cfg = _config(world, int8)
        max_len, filled = 64, 40
        full, names = llama.build_decode_step(cfg, batch, max_len, num_partitions=world, return_logits=True)
        weights = llama.make_weights(cfg, seed=0)
        caches = llama.make_kv_cache(cfg, batch, max_len, filled)
        tokens = np.arange(3, 3 + batch, dtype=np.int32)
        args = [tokens, np.array(filled, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches
        local = [_shard(a, sh[2] if sh[0] == P.PARTITIONED else -1, rank, world) for a, sh in zip(args, full.parameter_shardings)]
        uid = [be.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        be.comm_init(rank, uid[0], rank, world)
        if peer:  # all-reduce as one kernel per rank over peer-mapped memory instead of the library collective
            be.enable_peer_all_reduce(rank, rank, world, dist.all_gather_object)
        exe = be.compile_executable(full, [rank], partition=rank)
        dist.barrier()  # every rank has compiled: nobody reaches a collective while a peer is still in the compiler
        kinds = [s["type"] for s in exe.describe()["kernel_plan"]["steps"]]
        results = []
        bufs = [be.buffer_from_host(a, rank) for a in local]
        for step in range(2):  # the second execute replays the captured graph, collectives included
            outs = be.execute_executable(exe, bufs)
            results.append([o.to_numpy() for o in outs])
            # donated caches come back as outputs; feed them to the next step together with the same token / position
            bufs = bufs[:len(bufs) - len(caches)] + outs[2:]
        dist.barrier()
        queue.put((rank, kinds, [[np.asarray(o) if o.dtype.kind in "iub" else np.asarray(o).astype(np.float32) for o in r[:2]]
                                 for r in results]))


@pytest.mark.parametrize("world,batch,peer,int8", [(2, 2, False, False), (2, 16, False, False), (2, 2, True, False),
                                                   (2, 16, True, False), (2, 16, True, True),
                                                   (4, 16, False, False), (4, 2, True, False), (4, 16, True, False),
                                                   (8, 2, False, False), (8, 16, False, False), (8, 2, True, False),
                                                   (8, 16, True, False)])
def test_tensor_parallel_decode_matches_oracle(world, batch, peer, int8):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from oracle import plan_interp

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, batch, peer, queue, int8)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            rank, kinds, results = queue.get(timeout=300)
            assert kinds != "error", results
            got[rank] = (kinds, results)
    finally:
        for p in procs:
            p.join(timeout=120)
            if p.is_alive():
                p.terminate()
    assert all(p.exitcode == 0 for p in procs)

    cfg = _config(world, int8)
    max_len, filled = 64, 40
    full, names = llama.build_decode_step(cfg, batch, max_len, num_partitions=1, return_logits=True)
    weights = llama.make_weights(cfg, seed=0)
    caches = llama.make_kv_cache(cfg, batch, max_len, filled)
    tokens = np.arange(3, 3 + batch, dtype=np.int32)
    args = [tokens, np.array(filled, np.int32)] + [weights[n] for n in names[2:2 + len(weights)]] + caches
    want = plan_interp.run_plan(full, args)
    want_logits = np.asarray(want[1]).astype(np.float32)
    scale = float(np.abs(want_logits).max())
    for rank in range(world):
        kinds, results = got[rank]
        assert kinds.count("all_reduce") == 2 * cfg.layers and kinds.count("all_gather") == 1, kinds
        assert kinds.count("attention_decode") == cfg.layers, kinds  # the partitioned program keeps the recognisable form
        for step, (tok, logits) in enumerate(results):
            # the same token at the same position is decoded twice: the second pass overwrites the same cache row
            err = float(np.abs(np.asarray(logits, np.float32) - want_logits).max())
            print(f"world {world} batch {batch} peer {peer} rank {rank} step {step}: logits max-abs error {err:.4e} (scale {scale:.4e})")
            assert err <= 2e-2 * scale, (rank, step, err, scale)
            ref = np.sort(want_logits, axis=1)[:, -2:]
            decisive = (ref[:, 1] - ref[:, 0]) > 2 * err
            assert np.array_equal(np.asarray(tok)[decisive], np.asarray(want[0])[decisive])
    for rank in range(1, world):
        assert np.array_equal(got[0][1][0][0], got[rank][1][0][0])  # every rank picks the same tokens


def _absent_rank_worker(rank, world, port, queue):
    import torch.distributed as dist

    import pjrtx_b200
    from pjrtx_b200 import PlanBuilder
    from pjrtx_b200 import backend as be_mod

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["PJRTX_B200_PEER_TIMEOUT_MS"] = "300"  # the budget a launch gives its peers before it reports them missing
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        be = pjrtx_b200.Backend()
        uid = [be.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        be.comm_init(rank, uid[0], rank, world)
        n = 8192
        x = (np.arange(n, dtype=np.float32) % 13 + rank).astype(P.np_dtype(P.BF16_CODE))
        want = sum((np.arange(n, dtype=np.float32) % 13 + r) for r in range(world))

        def one_all_reduce():
            b = PlanBuilder()
            b.set_outputs([b.all_reduce(b.parameter(P.BF16_CODE, [n]))])
            return be.compile_executable(b, [rank])  # its only collective runs over peer memory: no library kernel waits

        report = {}
        # 1. both ranks present
        be.enable_peer_all_reduce(rank, rank, world, dist.all_gather_object)
        exe = one_all_reduce()
        dist.barrier()
        got = be.execute_executable(exe, [be.buffer_from_host(x, rank)])[0].to_numpy().astype(np.float32)
        report["first"] = bool(np.array_equal(got, want))
        dist.barrier()
        # 2. rank 1 stays away from one step (it leaves between steps; nothing of its own is in flight)
        if rank == 0:
            out = be.execute_executable(exe, [be.buffer_from_host(x, rank)])  # enqueues and returns
            try:
                be.synchronize(rank)
                report["timeout"] = "no error"
            except be_mod.BackendError as e:
                report["timeout"] = str(e)
            del out
        dist.barrier()
        # 3. fresh regions (new export / import zeroes the step words), both ranks present again
        be.enable_peer_all_reduce(rank, rank, world, dist.all_gather_object)
        exe2 = one_all_reduce()
        dist.barrier()
        got = be.execute_executable(exe2, [be.buffer_from_host(x, rank)])[0].to_numpy().astype(np.float32)
        be.synchronize(rank)
        report["recovered"] = bool(np.array_equal(got, want))
        dist.barrier()
        queue.put((rank, report))
    except Exception:
        import traceback

        queue.put((rank, {"error": traceback.format_exc()}))
        raise
    finally:
        dist.destroy_process_group()


def test_absent_rank_runs_out_a_bounded_wait_and_the_pair_recovers():
    """Failure detection without a GPU fault: one rank does not join a step of the peer-memory all-reduce. The other
    rank's kernel gives its peer 300 ms, raises the error word (code 21) and returns; the host reads it at the next
    synchronize and the context stays usable: after the ranks exchange fresh regions the collective works again."""
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    reports = {}
    try:
        for _ in range(2):
            rank, report = queue.get(timeout=300)
            reports[rank] = report
    finally:
        for p in procs:
            p.join(timeout=120)
            if p.is_alive():
                p.terminate()
    assert all("error" not in r for r in reports.values()), reports
    assert reports[0]["first"] and reports[1]["first"]
    assert "gave up a bounded wait (code 21)" in reports[0]["timeout"], reports[0]
    assert reports[0]["recovered"] and reports[1]["recovered"]
