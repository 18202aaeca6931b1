"""Categorical cross-entropy on softmax probabilities
(pydtnn/backends/gpu/losses/categorical_cross_entropy_gpu.py:30-69) with the accuracy metric
(pydtnn/backends/gpu/metrics/categorical_accuracy_gpu.py:30-60) computed in the same kernel."""
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
        self.dx = TensorGPU(empty((b, shape[1]), model.dtype), model.tensor_format)

    def __call__(self, y_pred, labels, global_batch_size):
        """``labels``: device int32 array (b,). Returns (self, dx): read the numbers with
        ``loss()`` / ``accuracy()``, which copy b values to the host."""
        m = self.model
        _lib.check(_lib.lib().b2c_cce_forward_backward(
            _lib.dtype_code(m.dtype), m.batch_size, self.shape[1], y_pred.ptr, labels.gpudata,
            int(global_batch_size), float(self.eps), self.row_loss.gpudata, self.hit.gpudata, self.dx.ptr,
            m.stream_handle))
        return self, self.dx

    def loss(self):
        return float(-np.sum(self.row_loss.get().astype(np.float64)) / self.model.batch_size)

    def accuracy(self):
        return float(np.sum(self.hit.get()) * 100.0 / self.model.batch_size)
