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


class CommError(RuntimeError):
    """The exchange between ranks failed: a rank never joined, left, or disagrees about the gradient layout.
    Raised on the host; no kernel is left waiting (the reference's NCCL wrapper raises ``NcclError`` on a non-zero
    status, pydtnn/backends/gpu/libs/libnccl.py:54-77)."""


def init_process_group_from_env(backend=None, timeout_s=120):
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (as set by
    ``torch.distributed.run``). Returns (rank, world_size); (0, 1) when not launched as a job.
    Replaces the MPI bootstrap + ncclCommInitRank of pydtnn/model.py:141-171.  A job whose ranks do not all
    arrive within ``timeout_s`` seconds ends with ``CommError`` on the ranks that did."""
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
        try:
            dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        except Exception as e:
            if dist.is_initialized():
                dist.destroy_process_group()
            raise CommError(f"rank {os.environ.get('RANK', '?')} of {world}: the process group did not form within "
                            f"{timeout_s} s (a rank never joined?): {type(e).__name__}: {e}") from e
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
        self.before_launch = None  # called before an all-reduce is issued (the model joins its side stream there)

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
        self._check_same_layout()
        self._built = True
        self.reset()

    def _check_same_layout(self):
        """Every rank must cut the same buckets, or an all-reduce would pair ranges of different lengths (NCCL then
        hangs or corrupts memory).  The ranks compare a short signature of their bucket lists once, before the first
        all-reduce, and all of them raise if any differs."""
        if self.group is None:
            return
        sig = [len(self.arena.entries), len(self.buckets), sum(n for _, _, n in self.arena.entries)]
        h = 1469598103934665603
        for bk in self.buckets:
            for v in (bk["chunk"], bk["start"], bk["end"]):
                h = ((h ^ v) * 1099511628211) % (1 << 62)
        sig.append(h)
        mine = torch.tensor(sig, dtype=torch.int64, device=self.arena.device)
        world = dist.get_world_size(self.group)
        theirs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(theirs, mine, group=self.group)
        rows = [t.cpu().tolist() for t in theirs]
        if any(r != rows[0] for r in rows):
            raise CommError("gradient arenas differ between ranks (entries, buckets, elements, layout hash per rank): "
                            f"{rows}")

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
                    if self.before_launch is not None:
                        self.before_launch()
                    try:
                        self._works[b] = dist.all_reduce(self._view(b), op=dist.ReduceOp.SUM, group=self.group,
                                                         async_op=True)
                    except Exception as e:
                        raise CommError(f"all-reduce of gradient bucket {b} could not be issued: "
                                        f"{type(e).__name__}: {e}") from e
                    self.launch_order.append(b)

    def mark_ready(self, layer):
        self.mark_entries_ready(self._layer_entries(layer))

    def wait_bucket(self, b):
        if self._works[b] is not None and not self._done[b]:
            try:
                self._works[b].wait()
            except Exception as e:          # a rank that left or a collective that timed out surfaces here, on the host
                raise CommError(f"all-reduce of gradient bucket {b} failed: {type(e).__name__}: {e}") from e
            self._done[b] = True

    def wait_for(self, layer):
        for idx in self._layer_entries(layer):
            self.wait_bucket(self.bucket_of[idx])

    def wait_all(self):
        for b in range(len(self.buckets)):
            if self._works[b] is None and self._pending[b] != set(self.buckets[b]["members"]):
                raise RuntimeError(f"gradient bucket {b} was only partly produced: {sorted(self._pending[b])} missing")
            self.wait_bucket(b)
