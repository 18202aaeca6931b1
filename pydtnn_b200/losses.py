"""Categorical cross-entropy on softmax probabilities
(pydtnn/backends/gpu/losses/categorical_cross_entropy_gpu.py:30-69) with the accuracy metric
(pydtnn/backends/gpu/metrics/categorical_accuracy_gpu.py:30-60) computed in the same kernel.

The mean loss and the accuracy of the batch are summed on the device into two doubles.  In a
data-parallel job those two doubles are divided by the process count and summed over the ranks,
which is what the reference does on the host with ``[loss, metrics...] / nprocs`` and an MPI
all-reduce (pydtnn/model.py:426-438): every rank then reports the global numbers."""
import numpy as np

from . import _lib
from .tensor_gpu import TensorGPU, empty


class CategoricalCrossEntropy:
    def __init__(self, shape, model, eps=1e-8):
        self.shape = shape
        self.model = model
        self.eps = eps
        b = model.batch_size
        self.row_loss = empty((b,), model.dtype)
        self.hit = empty((b,), np.int32)
        self.totals = empty((2,), np.float64)      # [mean loss, accuracy %] of this rank, then of the job
        self.dx = TensorGPU(empty((b, shape[1]), model.dtype), model.tensor_format)
        self._work = None
        self._scaled = 1

    def __call__(self, y_pred, labels, global_batch_size):
        """``labels``: device int32 array (b,). Returns (self, dx): read the numbers with
        ``loss()`` / ``accuracy()``, which copy two doubles to the host."""
        m = self.model
        L = _lib.lib()
        _lib.check(L.b2c_cce_forward_backward(
            _lib.dtype_code(m.dtype), m.batch_size, self.shape[1], y_pred.ptr, labels.gpudata,
            int(global_batch_size), float(self.eps), self.row_loss.gpudata, self.hit.gpudata, self.dx.ptr,
            m.stream_handle))
        _lib.check(L.b2c_cce_totals(_lib.dtype_code(m.dtype), m.batch_size, self.row_loss.gpudata, self.hit.gpudata,
                                    self.totals.gpudata, m.stream_handle))
        self._work, self._scaled = None, 1
        if m.comm is not None:
            import torch.distributed as dist
            # ordered after the totals kernel by a stream event, like the gradient buckets; read back lazily
            self._work = dist.all_reduce(self.totals.t, op=dist.ReduceOp.SUM, group=m.comm, async_op=True)
            self._scaled = m.nprocs
        return self, self.dx

    def _read(self):
        if self._work is not None:
            self._work.wait()
            self._work = None
        v = self.totals.get() / self._scaled
        # the copy above waited for the step's kernels: a bounded in-kernel wait that ran out is reported here
        _lib.check(_lib.lib().b2c_check_device_status(None))
        return v

    def loss(self):
        """Mean loss over the global batch (all ranks)."""
        return float(self._read()[0])

    def accuracy(self):
        """Accuracy in per cent over the global batch (all ranks)."""
        return float(self._read()[1])

    def local_loss(self):
        """Mean loss of this rank's rows only."""
        return float(-np.sum(self.row_loss.get().astype(np.float64)) / self.model.batch_size)
