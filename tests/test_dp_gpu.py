"""Data-parallel step on two GPUs: two ranks on half batches must end with the same weights as one rank on the
whole batch (batch-norm-free network, so per-rank statistics do not differ), the replicas must stay bitwise
identical and the job's loss must be the loss of the whole batch.  The check itself is ``pydtnn_b200.dp_check``,
which the benchmark also runs (and reports) whenever it is launched on more than one GPU.  Needs two GPUs;
skipped otherwise."""
import os

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        torch.cuda.set_device(rank)
        from pydtnn_b200 import dp_check
        from pydtnn_b200.comm import init_process_group_from_env
        init_process_group_from_env()
        rec = dp_check.run(world, rank)
        q.put((rank, rec))
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_step_equals_single_rank_on_whole_batch():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for r in range(world):
        assert not isinstance(results[r], str), results[r]
        rec = results[r]
        assert rec["replicas_bitwise_identical"] is True
        assert rec["gradient_buckets"] >= 2
        assert rec["rel_l2_vs_single_rank"] <= 1e-5, rec
        assert rec["loss_abs_diff_vs_single_rank"] <= 1e-5, rec
        assert rec["ok"] is True
