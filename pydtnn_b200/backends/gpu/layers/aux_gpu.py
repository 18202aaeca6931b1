"""GPU layers either side of the convolution: Input, BatchNormalization, Relu, Softmax, pooling,
AdditionBlock, Flatten, Dropout(identity in evaluation).  Each mirrors the attributes and hook
behaviour of its reference counterpart under pydtnn/backends/gpu/{layers,activations}/ with the
cuDNN call replaced by a call through the C ABI."""
import numpy as np

from .... import _lib
from ....layers import (AdditionBlock, AveragePool2D, BatchNormalization, Dropout, Flatten, Input, MaxPool2D, Relu,
                        Softmax)
from ....tensor_gpu import TensorGPU, empty, to_gpu, zeros
from ....utils import EVALUATE_MODE, PYDTNN_TENSOR_FORMAT_NCHW, TRAIN_MODE
from .. import memory_allocation as wsp
from .layer_gpu import LayerGPU


def _layout(model):
    return _lib.LAYOUT_NCHW if model.tensor_format == PYDTNN_TENSOR_FORMAT_NCHW else _lib.LAYOUT_NHWC


class InputGPU(LayerGPU, Input):
    """pydtnn/backends/gpu/layers/input_gpu.py:28-40"""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        self.y = TensorGPU(empty((self.model.batch_size, *self.shape), self.model.dtype), self.model.tensor_format)

    def forward(self, x):
        pass

    def backward(self, dy):
        pass


class BatchNormalizationGPU(LayerGPU, BatchNormalization):
    """pydtnn/backends/gpu/layers/batch_normalization_gpu.py:36-163; arithmetic of
    pydtnn/backends/cpu/layers/batch_normalization_cpu.py:59-129."""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        c = self.ci
        g_arr, dg_arr = m.arena.alloc_param(np.full((c,), self.gamma_init_val, m.dtype))
        b_arr, db_arr = m.arena.alloc_param(np.full((c,), self.beta_init_val, m.dtype))
        self.gamma, self.dgamma = TensorGPU(g_arr, m.tensor_format), TensorGPU(dg_arr, m.tensor_format)
        self.beta, self.dbeta = TensorGPU(b_arr, m.tensor_format), TensorGPU(db_arr, m.tensor_format)
        self.running_mean = TensorGPU(to_gpu(self.moving_mean_initializer((c,), m.dtype)), m.tensor_format)
        self.running_var = TensorGPU(to_gpu(self.moving_variance_initializer((c,), m.dtype)), m.tensor_format)
        self.save_mean = TensorGPU(empty((c,), m.dtype), m.tensor_format)
        self.save_inv_var = TensorGPU(empty((c,), m.dtype), m.tensor_format)
        self._inv_std = empty((c,), m.dtype)
        wsp.require_reduction_scratch(c)
        self.y = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        if self.need_dx:
            self.dx = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        self.fuse_relu = False           # set by the model's fusion pass (BN followed by ReLU)
        self.prestats = None             # (buffer, bytes) left by the preceding convolution's forward pass of this step
        self.residual = None             # (other branch, output) while an addition block folds its sum + ReLU in here
        self._dt = _lib.dtype_code(m.dtype)
        self._hw = self.hi * self.wi if self.spatial else 1
        self.updated_running_var = True

    def forward(self, x):
        m = self.model
        L = _lib.lib()
        self.x = x
        if m.mode == TRAIN_MODE and self.prestats is not None:
            # the convolution that wrote x already summed it per channel: statistics from those sums, one pass over x
            st, nbytes = self.prestats
            self.prestats = None
            addend, out, relu = (self.residual[0], self.residual[1], 1) if self.residual is not None else (None, self.y, int(self.fuse_relu))
            _lib.check(L.b2c_bn_train_forward_prestats(
                m.batch_size, self.ci, self._hw, x.ptr, st.data_ptr(), nbytes, self.gamma.ptr, self.beta.ptr,
                self.running_mean.ptr, self.running_var.ptr, float(self.momentum), float(self.epsilon), relu,
                addend.ptr if addend is not None else None, out.ptr, self.save_mean.ptr, self.save_inv_var.ptr,
                wsp.reduction_scratch().data_ptr(), wsp.reduction_scratch().numel() * 8, m.stream_handle))
            self.updated_running_var = True
            return out
        if m.mode == TRAIN_MODE and self.residual is not None:
            # last batch norm of a residual branch: out = relu(bn(x) + other branch), written to the block's ReLU
            addend, out = self.residual
            _lib.check(L.b2c_bn_train_forward_residual(
                self._dt, _layout(m), m.batch_size, self.ci, self._hw, x.ptr, self.gamma.ptr, self.beta.ptr,
                self.running_mean.ptr, self.running_var.ptr, float(self.momentum), float(self.epsilon), addend.ptr, 1,
                out.ptr, self.save_mean.ptr, self.save_inv_var.ptr, wsp.reduction_scratch().data_ptr(),
                wsp.reduction_scratch().numel() * 8, m.stream_handle))
            self.updated_running_var = True
            return out
        if m.mode == TRAIN_MODE:
            _lib.check(L.b2c_bn_train_forward(self._dt, _layout(m), m.batch_size, self.ci, self._hw, x.ptr,
                                              self.gamma.ptr, self.beta.ptr, self.running_mean.ptr,
                                              self.running_var.ptr, float(self.momentum), float(self.epsilon),
                                              int(self.fuse_relu), self.y.ptr, self.save_mean.ptr,
                                              self.save_inv_var.ptr, wsp.reduction_scratch().data_ptr(),
                                              wsp.reduction_scratch().numel() * 8, m.stream_handle))
            self.updated_running_var = True
        elif m.mode == EVALUATE_MODE:
            _lib.check(L.b2c_bn_inference(self._dt, _layout(m), m.batch_size, self.ci, self._hw, x.ptr,
                                          self.running_mean.ptr, self.inference_inv_std().gpudata, self.gamma.ptr,
                                          self.beta.ptr, int(self.fuse_relu), self.y.ptr, m.stream_handle))
        else:
            raise ValueError("Unexpected model mode")
        return self.y

    def inference_inv_std(self):
        """1 / sqrt(running_var + eps) on the device, recomputed (one small kernel, no host round trip) only after
        the running variance changed: a training step or a checkpoint load
        (pydtnn/backends/cpu/layers/batch_normalization_cpu.py:92-94 refreshes it under the same flag)."""
        if self.updated_running_var:
            _lib.check(_lib.lib().b2c_bn_inv_std(self._dt, self.ci, self.running_var.ptr, float(self.epsilon),
                                                 self._inv_std.gpudata, self.model.stream_handle))
            self.updated_running_var = False
        return self._inv_std

    def backward(self, dy):
        m = self.model
        _lib.check(_lib.lib().b2c_bn_train_backward(
            self._dt, _layout(m), m.batch_size, self.ci, self._hw, self.x.ptr, dy.ptr,
            self.y.ptr if self.fuse_relu else None, self.beta.ptr if self.fuse_relu else None, self.gamma.ptr,
            self.save_mean.ptr, self.save_inv_var.ptr,
            self.dgamma.ptr, self.dbeta.ptr, self.dx.ptr if self.need_dx else None,
            wsp.reduction_scratch().data_ptr(), wsp.reduction_scratch().numel() * 8, m.stream_handle))
        if self.need_dx:
            return self.dx


class ReluGPU(LayerGPU, Relu):
    """pydtnn/backends/gpu/activations/relu_gpu.py:40-68"""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        self.y = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        if self.need_dx:
            self.dx = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        self._dt = _lib.dtype_code(m.dtype)
        self.absorbed = False            # True when the preceding BatchNormalization applies the ReLU itself
        self.fed_by_block = False        # True when the preceding AdditionBlock writes max(sum, 0) into self.y
        self.bwd_by_block = False        # True when the following AdditionBlock writes the masked gradient into self.dx

    def forward(self, x):
        if self.absorbed:
            return x
        if self.fed_by_block:
            return self.y
        _lib.check(_lib.lib().b2c_relu_forward(self._dt, self.y.size, x.ptr, self.y.ptr, self.model.stream_handle))
        return self.y

    def backward(self, dy):
        if self.absorbed:
            return dy
        if self.bwd_by_block and self.model.mode == TRAIN_MODE:
            return self.dx
        if self.need_dx:
            _lib.check(_lib.lib().b2c_relu_backward(self._dt, self.y.size, dy.ptr, self.y.ptr, self.dx.ptr,
                                                    self.model.stream_handle))
            return self.dx


class SoftmaxGPU(LayerGPU, Softmax):
    """pydtnn/backends/gpu/activations/softmax_gpu.py:40-64"""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        self.y = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        if self.need_dx:
            self.dx = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        self._dt = _lib.dtype_code(m.dtype)
        self._rows, self._cols = int(x.ary.shape[0]), int(np.prod(x.ary.shape[1:]))

    def forward(self, x):
        _lib.check(_lib.lib().b2c_softmax_forward(self._dt, self._rows, self._cols, x.ptr, self.y.ptr,
                                                  self.model.stream_handle))
        return self.y

    def backward(self, dy):
        if self.need_dx:
            _lib.check(_lib.lib().b2c_softmax_backward(self._dt, self._rows, self._cols, dy.ptr, self.y.ptr,
                                                       self.dx.ptr, self.model.stream_handle))
            return self.dx


class DropoutGPU(LayerGPU, Dropout):
    """Identity in evaluation (the only mode the supported configurations use it in)."""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        self.y = x

    def forward(self, x):
        if self.model.mode == TRAIN_MODE:
            raise NotImplementedError("training-mode dropout is outside the supported path")
        return x

    def backward(self, dy):
        raise NotImplementedError("training-mode dropout is outside the supported path")


class FlattenGPU(LayerGPU, Flatten):
    """pydtnn/backends/gpu/layers/flatten_gpu.py:33-52 -- views, no copies."""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        self.y = TensorGPU(x.ary.reshape((self.model.batch_size, *self.shape)), self.model.tensor_format)

    def forward(self, x):
        self.y = TensorGPU(x.ary.reshape((self.model.batch_size, *self.shape)), self.model.tensor_format)
        return self.y

    def backward(self, dy):
        if self.need_dx:
            self.dx = TensorGPU(dy.ary.reshape((self.model.batch_size, *self.prev_shape)), self.model.tensor_format)
            return self.dx


class _Pool2DGPU(LayerGPU):
    """pydtnn/backends/gpu/layers/abstract_pool_2d_layer_gpu.py:36-102"""
    _is_max = 0

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        self.y = TensorGPU(empty((m.batch_size, *self.shape), m.dtype), m.tensor_format)
        if self._is_max:
            self.idx_max = empty((m.batch_size, *self.shape), np.int32)
        if self.need_dx:
            self.dx = TensorGPU(empty(x.ary.shape, m.dtype), m.tensor_format)
        self._dt = _lib.dtype_code(m.dtype)

    def _geom(self):
        return (self.model.batch_size, self.hi, self.wi, self.ci, self.kh, self.kw, self.vpadding, self.hpadding,
                self.vstride, self.hstride, self.vdilation, self.hdilation)

    def forward(self, x):
        m = self.model
        _lib.check(_lib.lib().b2c_pool_forward(self._dt, _layout(m), self._is_max, *self._geom(), x.ptr, self.y.ptr,
                                               self.idx_max.gpudata if self._is_max else None, m.stream_handle))
        return self.y

    def backward(self, dy):
        if self.need_dx:
            m = self.model
            _lib.check(_lib.lib().b2c_pool_backward(self._dt, _layout(m), self._is_max, *self._geom(), dy.ptr,
                                                    self.idx_max.gpudata if self._is_max else None, self.dx.ptr,
                                                    m.stream_handle))
            return self.dx


class MaxPool2DGPU(_Pool2DGPU, MaxPool2D):
    _is_max = 1


class AveragePool2DGPU(_Pool2DGPU, AveragePool2D):
    _is_max = 0


class AdditionBlockGPU(LayerGPU, AdditionBlock):
    """pydtnn/backends/gpu/layers/addition_block_gpu.py:30-85: run every path on the block input,
    sum the outputs into the first path's output; backward mirrors it."""

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        self.out_shapes = []
        for p_i, p in enumerate(self.paths):
            shape, cur = self.prev_shape, self.x
            for i, layer in enumerate(p):
                layer.set_model(m)
                layer.initialize(shape, self.need_dx, cur)
                cur = layer.y
                shape = layer.shape
                self.nparams += layer.nparams
                if layer.act:
                    raise NotImplementedError("activation arguments inside block paths are not supported")
            self.out_shapes.append(shape)
        assert all(o == self.out_shapes[0] for o in self.out_shapes)
        self.shape = self.out_shapes[0]
        if len(self.paths[0]) == 0:
            raise NotImplementedError("the first path of an AdditionBlock must not be empty")
        self.y = self.paths[0][-1].y
        self._dt = _lib.dtype_code(m.dtype)
        self.relu_after = None           # set by the model: the Relu layer that directly follows this block
        self.fold_sum = True             # let the first branch's last batch norm do the sum and that ReLU
        self.relu_before = None          # set by the model: the Relu layer whose output is this block's input

    def _fold_sum_into_last_bn(self):
        """Training step, two branches, the block feeds a ReLU and the first branch ends in a plain batch norm:
        that batch norm can add the other branch and apply the ReLU while it writes (one pass less over the block's
        largest tensors, and the batch-norm output itself is never stored)."""
        if self.model.mode != TRAIN_MODE or self.relu_after is None or len(self.paths) != 2 or not self.fold_sum:
            return None
        bn = self.paths[0][-1]
        if type(bn).__name__ != "BatchNormalizationGPU" or bn.fuse_relu:
            return None
        return bn

    def forward(self, x):
        L = _lib.lib()
        bn = self._fold_sum_into_last_bn()
        if bn is not None:
            other = x
            for layer in self.paths[1]:
                other = layer.forward(other)
            bn.residual = (other, self.relu_after.y)
            y = x
            for layer in self.paths[0]:
                y = layer.forward(y)
            bn.residual = None
            self.y = y
            return self.y
        last = len(self.paths) - 1
        for i, p in enumerate(self.paths):
            y_i = x
            for layer in p:
                y_i = layer.forward(y_i)
            if i == 0:
                self.y = y_i
            elif i == last and self.relu_after is not None:
                # residual sum and the ReLU that follows in one pass: relu.y = max(y + y_i, 0)
                _lib.check(L.b2c_add_relu(self._dt, self.y.size, self.y.ptr, y_i.ptr, self.relu_after.y.ptr,
                                          self.model.stream_handle))
            else:
                _lib.check(L.b2c_add_inplace(self._dt, self.y.size, self.y.ptr, y_i.ptr, self.model.stream_handle))
        return self.y

    def backward(self, dy):
        L = _lib.lib()
        dx0 = None
        for i, p in enumerate(self.paths):
            dx_i = dy
            for layer in reversed(p):
                dx_i = layer.backward(dx_i)
            if i == 0:
                dx0 = dx_i
            elif i == len(self.paths) - 1 and self.relu_before is not None:
                # the sum of the branch gradients and the backward of the ReLU that feeds this block in one pass
                r = self.relu_before
                _lib.check(L.b2c_add_relu_backward(self._dt, dx0.size, dx0.ptr, dx_i.ptr, r.y.ptr, r.dx.ptr,
                                                   self.model.stream_handle))
            else:
                _lib.check(L.b2c_add_inplace(self._dt, dx0.size, dx0.ptr, dx_i.ptr, self.model.stream_handle))
        self.dx = dx0
        return dx0

    def update_weights(self, optimizer):
        for layer in self.children:
            layer.update_weights(optimizer)

    def reduce_weights_async(self):
        for layer in self.children:
            layer.reduce_weights_async()

    def wait_allreduce_async(self):
        for layer in self.children:
            layer.wait_allreduce_async()

    def reduce_weights_sync(self):
        for layer in self.children:
            layer.reduce_weights_sync()
