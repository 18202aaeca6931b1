"""Rank-sliced batches, the pinned feeder, the per-operation tracer events and the performance counter, without a
GPU.  The slices are compared with what the reference's own ``Dataset.batch_generator`` produced
(tests/golden/batch_slices.json, written by tests/golden/make_batch_slices_golden.py)."""
import itertools
import json
import os

import numpy as np

from pydtnn_b200 import tracer as tr
from pydtnn_b200.datasets import PinnedFeeder, batch_generator
from pydtnn_b200.performance_counter import PerformanceCounter

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "batch_slices.json")


def test_rank_slices_match_the_reference_generator():
    cases = json.load(open(GOLDEN))
    assert len(cases) >= 10
    for case in cases:
        n, local, nprocs = case["nsamples"], case["local_batch"], case["nprocs"]
        x = np.arange(n, dtype=np.int64).reshape(-1, 1)
        y = x * 10
        for rank in range(nprocs):
            np.random.seed(1234)
            got = [[xb[:, 0].tolist(), (yb[:, 0] // 10).tolist(), int(bs)]
                   for xb, yb, bs in batch_generator(x, y, local, rank, nprocs, shuffle=case["shuffle"])]
            assert got == case["batches"][rank], (n, local, nprocs, case["shuffle"], rank)


def test_every_sample_is_dealt_exactly_once_per_pass():
    x = np.arange(203).reshape(-1, 1)
    rng_seed = 7
    seen = []
    for rank in range(4):
        for xb, yb, bs in batch_generator(x, x, 8, rank, 4, shuffle=True, rng=np.random.Generator(np.random.PCG64(rng_seed))):
            seen += xb[:, 0].tolist()
    assert sorted(seen) == list(range(203))


class _FakeModel:
    """The attributes PinnedFeeder reads, without a device."""
    def __init__(self, batch, shape):
        import torch
        self.batch_size, self.dtype = batch, np.float32

        class _A:
            pass
        y = _A(); y.ary = _A(); y.ary.shape = (batch, *shape)
        layer = _A(); layer.y = y
        self.layers = [layer]
        self.torch = torch


def test_pinned_feeder_skips_short_batches_and_announces_the_next_one():
    n, local = 45, 8
    x = np.arange(n * 6, dtype=np.float32).reshape(n, 2, 3)
    y = np.arange(n) % 5
    m = _FakeModel(local, (2, 3))
    feeder = PinnedFeeder(m, batch_generator(x, y, local, 0, 1, shuffle=False), pin=False)
    got, nexts = [], []
    for xb, yb, global_bs, nxt in feeder:
        got.append((xb.numpy().copy(), yb.numpy().copy(), global_bs))
        nexts.append(None if nxt is None else nxt[0])
    assert len(got) == 5 and feeder.skipped == 1            # 45 = 5 x 8 + a short batch of 5, dropped
    for i, (xb, yb, bs) in enumerate(got):
        assert np.array_equal(xb, x[i * 8:(i + 1) * 8]) and np.array_equal(yb, y[i * 8:(i + 1) * 8]) and bs == 8
    assert nexts[-1] is None and all(t is not None for t in nexts[:-1])
    # the tensor announced as next is the one the following iteration yields (so a staged upload is found again)
    feeder = PinnedFeeder(m, batch_generator(x, y, local, 0, 1, shuffle=False), pin=False)
    prev_next = None
    for xb, yb, global_bs, nxt in feeder:
        if prev_next is not None:
            assert xb is prev_next
        prev_next = None if nxt is None else nxt[0]


class _L:
    def __init__(self, lid, name):
        self.id, self.canonical_name_with_id = lid, f"{lid}_{name}"


def test_per_operation_events_follow_the_reference_numbering(tmp_path):
    assert tr.PYDTNN_OPS_EVENT == 60000002 and tr.PYDTNN_OPS_EVENTS == 36
    # spot values of pydtnn/tracers/events.py:33-70 (alphabetical within the reference's list)
    assert (tr.PYDTNN_OPS_ALLREDUCE_DW, tr.PYDTNN_OPS_BACKWARD_CUDNN_DB, tr.PYDTNN_OPS_BACKWARD_CUDNN_DW,
            tr.PYDTNN_OPS_BACKWARD_CUDNN_DX, tr.PYDTNN_OPS_FORWARD_CUBLAS_MATMUL, tr.PYDTNN_OPS_FORWARD_CUDNN,
            tr.PYDTNN_OPS_FORWARD_TRANSPOSE_Y) == (1, 6, 7, 8, 26, 27, 36)
    clock = itertools.count()
    t = tr.StepTracer(timer=lambda: next(clock), elapsed=lambda a, b: float(b - a), nvtx=None)
    conv = _L(3, "Conv2D")
    t.enable_tracing()                     # model-level events only
    with t.op_region(conv, tr.PYDTNN_OPS_FORWARD_CUDNN):
        pass
    assert t.records == []
    t.enable_tracing(ops=True)
    with t.region(conv, tr.PYDTNN_MDL_FORWARD):
        with t.op_region(conv, tr.PYDTNN_OPS_FORWARD_CUDNN):
            next(clock)
    ops = t.ops_summary()
    assert list(ops) == [3 * 36 + 27] and ops[3 * 36 + 27][0] == "3_Conv2D_forward_cudnn" and ops[3 * 36 + 27][1] == 1
    assert list(t.summary()) == [3 * 5 + 1]
    out = tmp_path / "trace.csv"
    t.write_output(out)
    lines = out.read_text().splitlines()
    assert lines[1].startswith("Model;16;3_Conv2D_forward;1;") and lines[2].startswith("Operations;135;3_Conv2D_forward_cudnn;1;")


def test_performance_counter_totals_and_last_half_estimate():
    pc = PerformanceCounter()
    for epoch in range(2):
        for step, t in enumerate((4.0, 1.0, 1.0, 1.0)):          # a slow first step, as after a cold start
            pc.add_training_time_and_batch_size(epoch, t, 64)
    pc.add_testing_time_and_batch_size(0, 2.0, 128)
    assert pc.num_epochs == 2 and pc.num_evaluations == 1
    assert pc.training_time == 14.0 and abs(pc.training_throughput - 512 / 14.0) < 1e-12
    assert pc.training_time_estimated_from_last_half_of_each_epoch == 8.0       # 2 x (1 + 1) x 4 / 2
    assert abs(pc.training_throughput_only_last_half_of_each_epoch - 512 / 8.0) < 1e-12
    assert pc.testing_throughput == 64.0 and pc.training_maximum_memory > 0
    assert any("Training throughput" in ln for ln in pc.report())
