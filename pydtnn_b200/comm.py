"""Gradient exchange for the data-parallel step: bucketed NCCL all-reduce overlapped with backward.

The reference sums every gradient tensor across ranks with its own ``ncclAllReduce`` after a host
``stream.synchronize()`` (pydtnn/backends/gpu/layers/layer_gpu.py:75-82; 212 calls per ResNet-50
step).  Here gradients live in a flat arena, so a *bucket* is an address range of that arena.
Buckets are cut from the end of the arena (the layers whose gradients are produced first in
backward) and each is reduced with one SUM all-reduce as soon as its last tensor has been written.
``torch.distributed`` orders the collective after the producing kernels with a stream event and
``Work.wait()`` makes the compute stream wait for it: no host synchronisation inside a step.
The loss gradient is already divided by the global batch (reference:
pydtnn/backends/cpu/losses/categorical_cross_entropy_cpu.py:34), so SUM gives the global mean.

The bucketer only touches torch tensors and a process group, so its logic runs unchanged among CPU
ranks over ``gloo`` (used by the tests)."""
import os

import torch
import torch.distributed as dist


def init_process_group_from_env(backend=None, timeout_s=120):
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (as set by
    ``torch.distributed.run``). Returns (rank, world_size); (0, 1) when not launched as a job.
    Replaces the MPI bootstrap + ncclCommInitRank of pydtnn/model.py:141-171."""
    import datetime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return dist.get_rank(), dist.get_world_size()


class GradientBucketer:
    def __init__(self, arena, group=None, bucket_elems=6 * 1024 * 1024):
        self.arena = arena
        self.group = group
        self.bucket_elems = int(bucket_elems)
        self.buckets = []          # dicts: chunk, start, end, members(set of entry idx)
        self.bucket_of = {}        # entry idx -> bucket idx
        self._pending = []
        self._works = []
        self._done = []
        self._built = False
        self.launch_order = []     # bucket indices in the order their all-reduce was issued (for tests)

    def build(self):
        self.buckets, self.bucket_of = [], {}
        per_chunk = {}
        for idx, (ci, off, numel) in enumerate(self.arena.entries):
            per_chunk.setdefault(ci, []).append((idx, off, numel))
        for ci in sorted(per_chunk, reverse=True):
            cur = None
            for idx, off, numel in reversed(per_chunk[ci]):
                if cur is None:
                    cur = dict(chunk=ci, start=off, end=off + numel, members=set())
                cur["start"] = off
                cur["members"].add(idx)
                if cur["end"] - cur["start"] >= self.bucket_elems:
                    self.buckets.append(cur)
                    cur = None
            if cur is not None:
                self.buckets.append(cur)
        for b, bk in enumerate(self.buckets):
            for idx in bk["members"]:
                self.bucket_of[idx] = b
        self._built = True
        self.reset()

    def reset(self):
        if not self._built:
            self.build()
        self._pending = [set(b["members"]) for b in self.buckets]
        self._works = [None] * len(self.buckets)
        self._done = [False] * len(self.buckets)
        self.launch_order = []

    def _view(self, b):
        bk = self.buckets[b]
        return self.arena.chunks[bk["chunk"]].dw[bk["start"]:bk["end"]]

    def _layer_entries(self, layer):
        return [self.arena.entry_of(getattr(layer, dw_).ary) for dw_ in layer.grad_vars.values()]

    def mark_entries_ready(self, entries):
        for idx in entries:
            b = self.bucket_of[idx]
            pend = self._pending[b]
            if idx in pend:
                pend.discard(idx)
                if not pend and self._works[b] is None:
                    self._works[b] = dist.all_reduce(self._view(b), op=dist.ReduceOp.SUM, group=self.group,
                                                     async_op=True)
                    self.launch_order.append(b)

    def mark_ready(self, layer):
        self.mark_entries_ready(self._layer_entries(layer))

    def wait_bucket(self, b):
        if self._works[b] is not None and not self._done[b]:
            self._works[b].wait()
            self._done[b] = True

    def wait_for(self, layer):
        for idx in self._layer_entries(layer):
            self.wait_bucket(self.bucket_of[idx])

    def wait_all(self):
        for b in range(len(self.buckets)):
            if self._works[b] is None and self._pending[b] != set(self.buckets[b]["members"]):
                raise RuntimeError(f"gradient bucket {b} was only partly produced: {sorted(self._pending[b])} missing")
            self.wait_bucket(b)
