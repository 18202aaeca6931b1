"""FC on the b2c library (replaces the cuBLAS calls of pydtnn/backends/gpu/layers/fc_gpu.py:37-181).
Weights are (in, out) row-major as in the reference; biases (1, out)."""
import numpy as np

from .... import _lib, tracer
from ....layers import FC
from ....tensor_gpu import TensorGPU, empty
from .. import memory_allocation as wsp
from .layer_gpu import LayerGPU


class FCGPU(LayerGPU, FC):

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        self.weights_cpu = self.weights_initializer((*prev_shape, *self.shape), m.dtype)
        w_arr, dw_arr = m.arena.alloc_param(self.weights_cpu)
        self.weights = TensorGPU(w_arr, m.tensor_format)
        self.dw = TensorGPU(dw_arr, m.tensor_format)
        if self.use_bias:
            self.biases_cpu = self.biases_initializer((1, *self.shape), m.dtype)
            b_arr, db_arr = m.arena.alloc_param(self.biases_cpu)
            self.biases = TensorGPU(b_arr, m.tensor_format)
            self.db = TensorGPU(db_arr, m.tensor_format)
        self.y = TensorGPU(empty((m.batch_size, self.shape[0]), m.dtype), m.tensor_format)
        if self.need_dx:
            self.dx = TensorGPU(empty((m.batch_size, *prev_shape), m.dtype), m.tensor_format)
        self.nparams = self.weights.size + (self.biases.size if self.use_bias else 0)
        self._in, self._out = int(np.prod(prev_shape)), int(self.shape[0])
        self._dt = _lib.dtype_code(m.dtype)
        self._engine = getattr(m, "conv_engine", _lib.ENGINE_AUTO)
        wsp.require(_lib.lib().b2c_fc_workspace_bytes(self._dt, m.batch_size, self._in, self._out, self._engine))

    def forward(self, x):
        m = self.model
        self.x = x
        with m.tracer.op_region(self, tracer.PYDTNN_OPS_FORWARD_CUBLAS_MATMUL):       # the bias is added in the same call
            _lib.check(_lib.lib().b2c_fc_forward(self._dt, self._engine, m.batch_size, self._in, self._out, x.ptr,
                                                 self.weights.ptr, self.biases.ptr if self.use_bias else None,
                                                 self.y.ptr, wsp.ptr(), wsp.size(), m.stream_handle))
        return self.y

    def backward(self, dy):
        m = self.model
        L = _lib.lib()
        if not (m.tracer.enabled and m.tracer.ops):
            _lib.check(L.b2c_fc_backward(self._dt, self._engine, m.batch_size, self._in, self._out, self.x.ptr,
                                         dy.ptr, self.weights.ptr, self.dw.ptr, self.db.ptr if self.use_bias else None,
                                         self.dx.ptr if self.need_dx else None, wsp.ptr(), wsp.size(), m.stream_handle))
        else:
            # per-operation tracing: the weight (+ bias) gradient and the input gradient as separate calls, each in
            # its own event (the reference brackets its three cuBLAS calls the same way)
            with m.tracer.op_region(self, tracer.PYDTNN_OPS_BACKWARD_CUBLAS_MATMUL_DW):
                _lib.check(L.b2c_fc_backward(self._dt, self._engine, m.batch_size, self._in, self._out, self.x.ptr,
                                             dy.ptr, self.weights.ptr, self.dw.ptr, self.db.ptr if self.use_bias else None,
                                             None, wsp.ptr(), wsp.size(), m.stream_handle))
            if self.need_dx:
                with m.tracer.op_region(self, tracer.PYDTNN_OPS_BACKWARD_CUBLAS_MATMUL_DX):
                    _lib.check(L.b2c_fc_backward(self._dt, self._engine, m.batch_size, self._in, self._out, self.x.ptr,
                                                 dy.ptr, self.weights.ptr, None, None, self.dx.ptr, wsp.ptr(), wsp.size(),
                                                 m.stream_handle))
        if self.need_dx:
            return self.dx
