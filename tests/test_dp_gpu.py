"""Data-parallel step on two GPUs: two ranks on half batches must end with the same weights as one
rank on the whole batch (BN-free network, so the per-rank statistics do not differ), and the replicas
must stay bitwise identical.  Needs two GPUs; skipped otherwise."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _build(batch, comm):
    from pydtnn_b200.layers import FC, AveragePool2D, Conv2D, Flatten, Input, MaxPool2D
    from pydtnn_b200.model import Model
    np.random.seed(0)
    m = Model(batch_size=batch, tensor_format="NHWC", dtype=np.float32, comm=comm, bucket_elems=20000)
    m.add(Input(shape=(16, 16, 32)))
    m.add(Conv2D(nfilters=64, filter_shape=(3, 3), padding=1, activation="relu", weights_initializer="he_uniform"))
    m.add(MaxPool2D(pool_shape=(2, 2), stride=2))
    m.add(Conv2D(nfilters=64, filter_shape=(3, 3), padding=1, stride=2, activation="relu", weights_initializer="he_uniform"))
    m.add(Conv2D(nfilters=128, filter_shape=(1, 1), activation="relu", weights_initializer="he_uniform"))
    m.add(AveragePool2D(pool_shape=(0, 0)))
    m.add(Flatten())
    m.add(FC(shape=(10,), activation="softmax", weights_initializer="he_uniform"))
    return m


def _data(total, seed=5):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((total, 16, 16, 32)).astype(np.float32), rng.integers(0, 10, total)


def _weights(m):
    return torch.cat([ch.w[:ch.used].clone() for ch in m.arena.chunks]).cpu().numpy()


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        torch.cuda.set_device(rank)
        from pydtnn_b200.comm import init_process_group_from_env
        from pydtnn_b200.optimizers import SGD
        init_process_group_from_env()
        per = 8
        m = _build(per, True)
        assert m.nprocs == world and len(m.bucketer.buckets) == 0     # buckets are built on first use
        opt = SGD(learning_rate=0.05, momentum=0.9)
        x, y = _data(per * world)
        for step in range(3):
            m.train_batch(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per], opt)
        m.synchronize()
        assert len(m.bucketer.buckets) >= 2 and m.bucketer.launch_order == list(range(len(m.bucketer.buckets)))
        q.put((rank, _weights(m)))
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_step_equals_single_rank_on_whole_batch():
    from pydtnn_b200.optimizers import SGD
    world, per = 2, 8
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
    assert np.array_equal(results[0], results[1])          # replicas applied the same reduced gradient
    torch.cuda.set_device(0)
    single = _build(per * world, None)
    opt = SGD(learning_rate=0.05, momentum=0.9)
    x, y = _data(per * world)
    for step in range(3):
        single.train_batch(x, y, opt)
    single.synchronize()
    w1 = _weights(single)
    rel = np.linalg.norm(results[0] - w1) / np.linalg.norm(w1)
    assert rel <= 1e-5, rel
