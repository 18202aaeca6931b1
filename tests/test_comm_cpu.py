"""Gradient bucketing and the all-reduce exchange among two CPU ranks (gloo): bucket layout,
launch order, summed result, and the error for a partly produced bucket.  No GPU involved."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _build_arena(device="cpu"):
    from pydtnn_b200.arena import ParamArena
    arena = ParamArena(np.float32, device, chunk_elems=4096)
    shapes = [(7, 3), (100,), (64, 9), (5,), (300,), (17, 17), (2000,), (8,), (3000,)]
    views = [arena.alloc_param(np.full(s, i + 1, np.float32)) for i, s in enumerate(shapes)]
    return arena, views


def test_bucket_layout_is_contiguous_and_reverse_ordered():
    from pydtnn_b200.comm import GradientBucketer
    arena, views = _build_arena()
    assert len(arena.chunks) >= 2          # the last tensors spill into further chunks
    bk = GradientBucketer(arena, None, bucket_elems=600)
    bk.build()
    seen = set()
    for b in bk.buckets:
        assert b["end"] > b["start"]
        for idx in b["members"]:
            ci, off, numel = arena.entries[idx]
            assert ci == b["chunk"] and b["start"] <= off and off + numel <= b["end"]
            assert idx not in seen
            seen.add(idx)
    assert seen == set(range(len(arena.entries)))
    # first bucket holds the last-allocated tensor (its gradient is produced first in backward)
    assert len(arena.entries) - 1 in bk.buckets[0]["members"]


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        from pydtnn_b200.comm import GradientBucketer, init_process_group_from_env
        r, w = init_process_group_from_env(backend="gloo", timeout_s=60)
        assert (r, w) == (rank, world)
        arena, views = _build_arena()
        bk = GradientBucketer(arena, dist.group.WORLD, bucket_elems=600)
        bk.build()
        n = len(arena.entries)
        for step in range(2):
            bk.reset()
            for i, (_, dw) in enumerate(views):
                dw.t.fill_(float((rank + 1) * (i + 1) + step))
            for i in reversed(range(n)):          # backward order
                bk.mark_entries_ready([i])
            bk.wait_all()
            assert bk.launch_order == list(range(len(bk.buckets))), bk.launch_order
            for i, (_, dw) in enumerate(views):
                want = sum((rk + 1) * (i + 1) + step for rk in range(world))
                assert torch.all(dw.t == want), (i, dw.t.flatten()[:3], want)
        # a bucket that is only partly produced is reported, not silently skipped
        bk.reset()
        multi = next(b for b, bkt in enumerate(bk.buckets) if len(bkt["members"]) > 1)
        bk.mark_entries_ready([min(bk.buckets[multi]["members"])])
        try:
            bk.wait_all()
            q.put((rank, "no error raised"))
            return
        except RuntimeError as e:
            assert "partly produced" in str(e)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


def test_two_rank_allreduce_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


# ---- failure paths among CPU ranks: every failure is made on the host and must surface as CommError ----------

def _spawn(target, world, port_offset=0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000) + port_offset
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    return procs, q


def _never_joined_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world + 1))
        from pydtnn_b200.comm import CommError, init_process_group_from_env
        import time
        t0 = time.time()
        try:
            init_process_group_from_env(backend="gloo", timeout_s=5)
            q.put((rank, "joined a job whose last rank does not exist"))
        except CommError as e:
            q.put((rank, ("CommError", time.time() - t0, "did not form" in str(e))))
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))


def test_a_rank_that_never_joins_ends_the_others_with_a_clean_error():
    """WORLD_SIZE says 2, only rank 0 starts: the rendezvous runs into its 5 s limit and raises CommError."""
    procs, q = _spawn(_never_joined_worker, 1)
    rank, res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert res[0] == "CommError" and res[2], res
    assert res[1] < 60, res


def _mismatch_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        from pydtnn_b200.comm import CommError, GradientBucketer, init_process_group_from_env
        init_process_group_from_env(backend="gloo", timeout_s=30)
        arena, views = _build_arena()
        if rank == 1:
            arena.alloc_param(np.zeros((11,), np.float32))       # one tensor more than rank 0
        bk = GradientBucketer(arena, dist.group.WORLD, bucket_elems=600)
        try:
            bk.build()
            q.put((rank, "no error raised"))
        except CommError as e:
            q.put((rank, "CommError" if "differ between ranks" in str(e) else str(e)))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))


def test_ranks_whose_gradient_arenas_differ_are_refused_before_the_first_all_reduce():
    procs, q = _spawn(_mismatch_worker, 2, port_offset=1)
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results == [(0, "CommError"), (1, "CommError")], results


def _leaver_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        from pydtnn_b200.comm import CommError, GradientBucketer, init_process_group_from_env
        init_process_group_from_env(backend="gloo", timeout_s=8)
        arena, views = _build_arena()
        bk = GradientBucketer(arena, dist.group.WORLD, bucket_elems=600)
        bk.build()
        n = len(arena.entries)
        for i in reversed(range(n)):              # step 1: both ranks take part
            bk.mark_entries_ready([i])
        bk.wait_all()
        if rank == 1:
            q.put((rank, "left"))
            q.close()
            q.join_thread()                       # the message is on its way before the process goes
            os._exit(0)                           # leaves between steps, nothing in flight
        import time
        time.sleep(1.0)
        bk.reset()
        try:
            for i in reversed(range(n)):          # step 2: the peer is gone
                bk.mark_entries_ready([i])
            bk.wait_all()
            q.put((rank, "no error raised"))
        except CommError:
            q.put((rank, "CommError"))
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))


def test_a_rank_that_leaves_between_steps_fails_the_next_all_reduce_on_the_host():
    procs, q = _spawn(_leaver_worker, 2, port_offset=2)
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results == [(0, "CommError"), (1, "left")], results
