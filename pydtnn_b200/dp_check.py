"""Correctness check of the data-parallel step, run inside a multi-rank job.

The reference's scheme (pydtnn/backends/gpu/layers/layer_gpu.py:75-82, pydtnn/model.py:485-517): every rank holds
a replica, takes its slice of the global batch, and every gradient is summed over the ranks before the update, so
(a) the replicas stay identical and (b) the step equals a single-process step on the whole batch.

``run(world, rank)`` trains a small batch-norm-free network (statistics would differ per shard) for a few steps
on P shards, then checks both properties: the parameter arenas of all ranks are compared bit for bit (element-wise
MAX and MIN over the ranks of the parameters viewed as integers must agree), and rank 0 repeats the steps alone
on the concatenated batch and compares the parameters (relative L2).  The loss all-reduce is checked on the way:
the job's loss must equal the single-process loss on the whole batch.
"""
import numpy as np
import torch

STEPS = 3
PER_RANK = 8
REL_L2_BAR = 1e-5


def build_net(batch, comm, bucket_elems=20000, dtype=np.float32):
    """Conv 3x3 + ReLU, max pool, strided conv 3x3 + ReLU, conv 1x1 + ReLU, global average pool, FC + softmax:
    every convolution pass (fprop, wgrad, strided and plain dgrad), the FC layer and several gradient buckets."""
    from .layers import FC, AveragePool2D, Conv2D, Flatten, Input, MaxPool2D
    from .model import Model
    np.random.seed(0)                      # identical replicas
    m = Model(batch_size=batch, tensor_format="NHWC", dtype=dtype, comm=comm, bucket_elems=bucket_elems)
    m.add(Input(shape=(16, 16, 32)))
    m.add(Conv2D(nfilters=64, filter_shape=(3, 3), padding=1, activation="relu", weights_initializer="he_uniform"))
    m.add(MaxPool2D(pool_shape=(2, 2), stride=2))
    m.add(Conv2D(nfilters=64, filter_shape=(3, 3), padding=1, stride=2, activation="relu", weights_initializer="he_uniform"))
    m.add(Conv2D(nfilters=128, filter_shape=(1, 1), activation="relu", weights_initializer="he_uniform"))
    m.add(AveragePool2D(pool_shape=(0, 0)))
    m.add(Flatten())
    m.add(FC(shape=(10,), activation="softmax", weights_initializer="he_uniform"))
    return m


def data(total, seed=5):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((total, 16, 16, 32)).astype(np.float32), rng.integers(0, 10, total)


def weights(model):
    return torch.cat([ch.w[:ch.used] for ch in model.arena.chunks])


def run(world, rank, steps=STEPS, per_rank=PER_RANK):
    """Returns the ``dp_check`` record (same content on every rank; rank 0 holds the single-process comparison)."""
    import torch.distributed as dist
    from .optimizers import SGD
    x, y = data(per_rank * world)
    m = build_net(per_rank, True)
    opt = SGD(learning_rate=0.05, momentum=0.9)
    losses = []
    for _ in range(steps):
        loss = m.train_batch(x[rank * per_rank:(rank + 1) * per_rank], y[rank * per_rank:(rank + 1) * per_rank], opt)
        losses.append(loss.loss())
    m.synchronize()
    w = weights(m)
    bits = w.view(torch.int32).clone()
    hi, lo = bits.clone(), bits.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    identical = bool(torch.equal(hi, lo))
    rec = {"ranks": world, "steps": steps, "per_rank_batch": per_rank, "parameters": int(w.numel()),
           "gradient_buckets": len(m.bucketer.buckets), "replicas_bitwise_identical": identical,
           "rel_l2_vs_single_rank": None, "loss_abs_diff_vs_single_rank": None, "bar": REL_L2_BAR}
    out = torch.zeros(2, dtype=torch.float64, device=w.device)
    if rank == 0:
        single = build_net(per_rank * world, None)
        opt1 = SGD(learning_rate=0.05, momentum=0.9)
        losses1 = []
        for _ in range(steps):
            losses1.append(single.train_batch(x, y, opt1).loss())
        single.synchronize()
        w1 = weights(single).double()
        out[0] = torch.linalg.norm(w.double() - w1) / torch.linalg.norm(w1)
        out[1] = max(abs(a - b) for a, b in zip(losses, losses1))
    dist.broadcast(out, src=0)
    rec["rel_l2_vs_single_rank"] = float(out[0])
    rec["loss_abs_diff_vs_single_rank"] = float(out[1])
    rec["ok"] = identical and rec["rel_l2_vs_single_rank"] <= REL_L2_BAR and rec["loss_abs_diff_vs_single_rank"] <= 1e-5
    return rec
