"""Base of the GPU layers: buffer attributes and the gradient-exchange hooks
(pydtnn/backends/gpu/layers/layer_gpu.py:36-204).

The reference all-reduces every gradient tensor separately after a host synchronisation
(:78-82).  Here a layer only tells the model's gradient bucketer that its gradients are written;
the bucketer launches one NCCL all-reduce per contiguous bucket, ordered after the producing
kernels by a stream event, so no host synchronisation happens inside a step."""
from abc import ABC

from .... import tracer
from ....layers.base import Layer


class LayerGPU(Layer, ABC):

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.y = None
        self.weights_cpu = None
        self.biases_cpu = None
        self.x = None
        self.dx = None
        self.dw = None
        self.db = None

    def initialize(self, prev_shape, need_dx, x):
        self.x = x  # must be set before super().initialize()
        super().initialize(prev_shape, need_dx)

    # -- gradient exchange ---------------------------------------------------------------
    def _grad_tensors(self):
        return [getattr(self, dw_) for dw_ in self.grad_vars.values()]

    def reduce_weights_async(self):
        if self.model.comm is None or not self.grad_vars:
            return
        with self.model.tracer.op_region(self, tracer.PYDTNN_OPS_ALLREDUCE_DW):
            self.model.bucketer.mark_ready(self)

    def wait_allreduce_async(self):
        if self.model.comm is None or not self.grad_vars:
            return
        self.model.bucketer.wait_for(self)

    def reduce_weights_sync(self):
        if self.model.comm is None or not self.grad_vars:
            return
        self.model.bucketer.mark_ready(self)
        self.model.bucketer.wait_for(self)
