"""Batches for the data-parallel step: which samples a rank takes, and how they reach the device.

``batch_generator`` restates the slicing rule of the reference's ``Dataset.batch_generator``
(pydtnn/datasets/dataset.py:160-197): the samples of a chunk are shuffled once with a permutation every rank
draws identically, the global batch ``[k, k + nprocs * local)`` is cut into ``nprocs`` consecutive slices and rank
``r`` takes the ``r``-th; what is left at the end (fewer than a global batch, but at least one sample per rank) is
dealt out as evenly as possible, the first ``remaining`` ranks taking one sample more.  The GPU back end works on
fixed-size buffers, so its step skips a batch whose local size differs from the model's (pydtnn/model.py:457-459);
``PinnedFeeder`` does the same.

``PinnedFeeder`` turns such a generator into the (x, labels) pairs ``Model.train_batch(..., next_batch=)`` wants:
two pairs of pinned host tensors used alternately, so that while step ``i`` runs on the device the host fills the
other pair with batch ``i + 1`` and its upload is already queued on the copy stream.
"""
import numpy as np


def batch_generator(x_data, y_data, local_batch_size=64, rank=0, nprocs=1, shuffle=True, rng=None):
    """Yields ``(x_local, y_local, global_batch_size)`` for one pass over ``x_data`` / ``y_data`` (arrays whose first
    axis is the sample).  ``rng``: a ``numpy.random.Generator`` seeded identically on every rank (the reference relies
    on ``np.random.seed`` being the same everywhere); None draws from NumPy's global state as the reference does."""
    nsamples = x_data.shape[0]
    order = np.arange(nsamples)
    if shuffle:
        (rng.shuffle if rng is not None else np.random.shuffle)(order)
    batch_size = local_batch_size * nprocs
    last = nsamples % batch_size
    if last < nprocs:                      # too few left-overs to give every rank a sample: fold them into a last full-size batch
        last += batch_size
    end_full = nsamples - last
    for start in range(0, end_full, batch_size):
        idx = order[start + rank * local_batch_size: start + (rank + 1) * local_batch_size]
        yield x_data[idx, ...], y_data[idx, ...], batch_size
    if last > 0 and end_full >= 0:
        each, remaining = divmod(last, nprocs)
        if rank < remaining:
            lo = end_full + rank * (each + 1)
            hi = lo + each + 1
        else:
            lo = end_full + remaining * (each + 1) + (rank - remaining) * each
            hi = lo + each
        idx = order[lo:hi]
        yield x_data[idx, ...], y_data[idx, ...], last


class PinnedFeeder:
    """Iterates over ``(x, labels, global_batch_size)`` with ``x`` and ``labels`` in pinned host tensors, skipping
    batches whose local size is not ``model.batch_size``.  Use:

        feeder = PinnedFeeder(model, batch_generator(x, y, model.batch_size, model.rank, model.nprocs))
        for x, labels, global_bs, nxt in feeder:
            model.train_batch(x, labels, optimizer, global_bs, next_batch=nxt)
    """

    def __init__(self, model, generator, pin=True, wait_upload=None):
        """``wait_upload``: called before a pair is overwritten; must return once the asynchronous upload that read the
        pair two steps earlier has finished (the model passes a wait on its copy stream's event).  Callers that read
        a result back every step, as the reference's loop does for its metrics, are past that point anyway."""
        import torch
        self.model = model
        self.gen = iter(generator)
        self.wait_upload = wait_upload
        in_shape = tuple(model.layers[0].y.ary.shape)
        tdt = torch.float64 if np.dtype(model.dtype) == np.float64 else torch.float32
        mk = (lambda *a, **k: torch.empty(*a, **k).pin_memory()) if pin else torch.empty
        self.slots = [(mk(in_shape, dtype=tdt), mk((model.batch_size,), dtype=torch.int32)) for _ in range(2)]
        self.skipped = 0

    def _fill(self, slot):
        """Copy the next full-size batch of the generator into pair ``slot``; returns its global batch size or None."""
        import torch
        for x, y, global_bs in self.gen:
            if x.shape[0] != self.model.batch_size:
                self.skipped += 1
                continue
            xs, ys = self.slots[slot]
            if self.wait_upload is not None:
                self.wait_upload()
            xs.copy_(torch.from_numpy(np.ascontiguousarray(x, dtype=self.model.dtype)).view(xs.shape))
            lab = y if y.ndim == 1 else np.argmax(y, axis=1)
            ys.copy_(torch.from_numpy(np.ascontiguousarray(lab, dtype=np.int32)))
            return global_bs
        return None

    def __iter__(self):
        slot = 0
        cur = self._fill(slot)
        while cur is not None:
            # the other pair may still be read by the upload queued two steps ago: that upload was consumed by the
            # step that has just been issued, whose first action was to wait for it, so it is free to refill
            nxt = self._fill(1 - slot)
            x, y = self.slots[slot]
            yield x, y, cur, (self.slots[1 - slot] if nxt is not None else None)
            slot, cur = 1 - slot, nxt
