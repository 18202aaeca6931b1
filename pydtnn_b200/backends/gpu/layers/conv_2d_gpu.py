"""Conv2D on the b2c library: same attributes, buffer ownership and hook behaviour as the
reference's cuDNN layer (pydtnn/backends/gpu/layers/conv_2d_gpu.py:37-231), with every cuDNN
call replaced by one call through the C ABI."""
import ctypes

import numpy as np

from .... import _lib, tracer
from ....layers import Conv2D, Conv2DBatchNormalization, Conv2DBatchNormalizationRelu, Conv2DRelu
from ....tensor_gpu import TensorGPU, empty
from ....utils import PYDTNN_TENSOR_FORMAT_NCHW, PYDTNN_TENSOR_FORMAT_NHWC, TRAIN_MODE
from .. import memory_allocation as wsp
from .layer_gpu import LayerGPU


class Conv2DGPU(LayerGPU, Conv2D):

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.desc = None
        self.engine = _lib.ENGINE_AUTO
        self.stats_for_bn = None         # set by the model's fusion pass: the BatchNormalization this layer feeds
        self.stats_bytes = 0

    def _make_desc(self):
        m = self.model
        nchw = m.tensor_format == PYDTNN_TENSOR_FORMAT_NCHW
        return _lib.ConvDesc(
            layout=_lib.LAYOUT_NCHW if nchw else _lib.LAYOUT_NHWC, dtype=_lib.dtype_code(m.dtype),
            w_layout=_lib.W_KCRS if nchw else _lib.W_KRSC, engine=getattr(m, "conv_engine", self.engine),
            n=m.batch_size, h=self.hi, w=self.wi, ci=self.ci, co=self.co, kh=self.kh, kw=self.kw,
            vpad=self.vpadding, hpad=self.hpadding, vstr=self.vstride, hstr=self.hstride,
            vdil=self.vdilation, hdil=self.hdilation)

    def initialize(self, prev_shape, need_dx, x):
        super().initialize(prev_shape, need_dx, x)
        m = self.model
        # filters are (co, kh, kw, ci) in NHWC, as in the reference's GPU layer (:49-51)
        if m.tensor_format == PYDTNN_TENSOR_FORMAT_NHWC:
            self.weights_shape = (self.co, *self.filter_shape, self.ci)
        self.weights_cpu = self.weights_initializer(self.weights_shape, m.dtype)
        w_arr, dw_arr = m.arena.alloc_param(self.weights_cpu)
        self.weights = TensorGPU(w_arr, m.tensor_format, tensor_type="filter")
        self.dw = TensorGPU(dw_arr, m.tensor_format, tensor_type="filter")
        if self.use_bias:
            bshape = (1, self.co, 1, 1) if m.tensor_format == PYDTNN_TENSOR_FORMAT_NCHW else (1, 1, 1, self.co)
            self.biases_cpu = self.biases_initializer(bshape, m.dtype)
            b_arr, db_arr = m.arena.alloc_param(self.biases_cpu)
            self.biases = TensorGPU(b_arr, m.tensor_format)
            self.db = TensorGPU(db_arr, m.tensor_format)
        self.y = TensorGPU(empty((m.batch_size, *self.shape), m.dtype), m.tensor_format)
        if self.need_dx:
            self.dx = TensorGPU(empty(self.x.ary.shape, m.dtype), m.tensor_format)
        self.desc = self._make_desc()
        L = _lib.lib()
        need = max(L.b2c_conv_workspace_bytes(ctypes.byref(self.desc), p) for p in
                   (_lib.PASS_FPROP, _lib.PASS_DGRAD, _lib.PASS_WGRAD))
        wsp.require(need)
        wsp.require_side(L.b2c_conv_workspace_bytes(ctypes.byref(self.desc), _lib.PASS_WGRAD))
        self._wgrad_done = None
        # A few-channel layer (the stem) lowers its input into the workspace in the forward pass; with a workspace of
        # its own the matrix is still there for the weight gradient (the reference's CPU layer keeps x_rows the same way).
        self._own_ws = None
        self._lowered_valid = False
        if L.b2c_conv_keeps_lowered_input(ctypes.byref(self.desc)):
            import torch
            self._own_ws = torch.empty(int(need), dtype=torch.uint8, device=self.y.ary.t.device)
        # can this layer's forward pass leave the batch sums of its output for a following batch norm?
        self.stats_bytes = int(L.b2c_conv_stats_bytes(ctypes.byref(self.desc)))

    @property
    def flops_per_pass(self):
        """2*M*K*Co, padding taps counted (the reference's model, pydtnn/performance_models.py:68-70)."""
        return 2 * self.model.batch_size * self.ho * self.wo * self.co * self.ci * self.kh * self.kw

    _OPS = {"fprop": tracer.PYDTNN_OPS_FORWARD_CUDNN, "wgrad": tracer.PYDTNN_OPS_BACKWARD_CUDNN_DW,
            "dgrad": tracer.PYDTNN_OPS_BACKWARD_CUDNN_DX}

    def _timed(self, name, call):
        """Run one pass inside its per-operation tracer event (off by default); when the model carries a
        ``conv_profile`` list, bracket it with CUDA events on the launching stream (read back by the benchmark
        after the timed region)."""
        prof = getattr(self.model, "conv_profile", None)
        if prof is None:
            with self.model.tracer.op_region(self, self._OPS[name]):
                _lib.check(call())
            return
        import torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(call())
        e1.record()
        prof.append((name, self, e0, e1))

    def forward(self, x):
        L = _lib.lib()
        self.x = x          # backward reads the tensor this call saw (a fused predecessor may hand over its own buffer)
        bn = self.stats_for_bn
        ws_ptr, ws_size = (self._own_ws.data_ptr(), self._own_ws.numel()) if self._own_ws is not None else (wsp.ptr(), wsp.size())
        self._lowered_valid = self._own_ws is not None and self.model.mode == TRAIN_MODE
        if bn is not None and self.model.mode == TRAIN_MODE:
            # training step, a batch norm follows: the same pass also sums y and y^2 per channel while the tiles leave
            st = wsp.conv_stats()
            self._timed("fprop", lambda: L.b2c_conv_fprop_stats(
                ctypes.byref(self.desc), x.ptr, self.weights.ptr, self.biases.ptr if self.use_bias else None,
                self.y.ptr, st.data_ptr(), self.stats_bytes, ws_ptr, ws_size, self.model.stream_handle))
            bn.prestats = (st, self.stats_bytes)
            return self.y
        self._timed("fprop", lambda: L.b2c_conv_fprop(
            ctypes.byref(self.desc), x.ptr, self.weights.ptr, self.biases.ptr if self.use_bias else None, None, 0,
            self.y.ptr, ws_ptr, ws_size, self.model.stream_handle))
        return self.y

    def _wgrad_call(self, dy, ws_ptr, ws_size, stream):
        """The weight-gradient call on ``stream``; a layer that still holds its forward pass's lowered input in its own
        workspace uses that instead of lowering x again."""
        L = _lib.lib()
        db = self.db.ptr if self.use_bias else None
        if self._lowered_valid:
            self._lowered_valid = False
            own = self._own_ws
            return lambda: L.b2c_conv_wgrad_lowered(ctypes.byref(self.desc), self.x.ptr, dy.ptr, self.dw.ptr, db, own.data_ptr(),
                                                    own.numel(), stream)
        return lambda: L.b2c_conv_wgrad(ctypes.byref(self.desc), self.x.ptr, dy.ptr, self.dw.ptr, db, ws_ptr, ws_size, stream)

    def backward(self, dy):
        L = _lib.lib()
        m = self.model
        side = m.side_stream_for_wgrad()
        if side is None:
            self._timed("wgrad", self._wgrad_call(dy, wsp.ptr(), wsp.size(), m.stream_handle))
            if self.need_dx:
                self._timed("dgrad", lambda: L.b2c_conv_dgrad(
                    ctypes.byref(self.desc), dy.ptr, self.weights.ptr, self.dx.ptr, wsp.ptr(), wsp.size(), m.stream_handle))
                return self.dx
            return None
        # The weight gradient only has to be there when the gradients are exchanged or applied, so it runs on a side
        # stream next to what follows on the main stream.  The input gradient is issued first: both kernels want every
        # SM, the one launched first gets them, and the input gradient is what the main stream's next kernels (the
        # HBM-bound backward of the layers before this one) wait for -- those then run alongside the weight gradient.
        # The side stream waits for dy; the model joins it before the gradients are used.
        import torch
        if self._wgrad_done is None:
            self._dy_ready, self._wgrad_done = torch.cuda.Event(), torch.cuda.Event()
        self._dy_ready.record()
        if self.need_dx:
            _lib.check(L.b2c_conv_dgrad(ctypes.byref(self.desc), dy.ptr, self.weights.ptr, self.dx.ptr, wsp.ptr(), wsp.size(),
                                        m.stream_handle))
        side.wait_event(self._dy_ready)
        sw = wsp.side()
        _lib.check(self._wgrad_call(dy, sw.data_ptr(), sw.numel(), side.cuda_stream)())
        self._wgrad_done.record(side)
        m.note_side_work(self._wgrad_done)
        return self.dx if self.need_dx else None


class _FusedConvInference(Conv2DGPU):
    """Inference-only Conv2D with the BN-scale / ReLU epilogue fused into the convolution.
    Backward is refused, as in the reference's fused layers
    (pydtnn/backends/cpu/layers/conv_2d_batch_normalization_relu_cpu.py:47-48, 96-97)."""
    _with_bn = False
    _with_relu = False

    def __init__(self, *args, from_parent=None, from_parent_2=None, **kwargs):
        if from_parent is None:
            super().__init__(*args, **kwargs)
        else:
            # built by the fusion pass from initialised layers: share their buffers and parameters
            self.__dict__.update(from_parent.__dict__)
            self.bn_layer = from_parent_2

    def _refresh_bn(self):
        """Point the epilogue at the batch-norm layer's vectors; its inv_std lives on the device and is recomputed
        there only after the running variance changed (no host copy, no allocation per call)."""
        bn = self.bn_layer
        inv_std = bn.inference_inv_std()
        if getattr(self, "_bn", None) is None:
            self._bn = _lib.BnParams(bn.running_mean.ary.gpudata, inv_std.gpudata, bn.gamma.ary.gpudata,
                                     bn.beta.ary.gpudata)

    def _relu_flag(self):
        # a batch norm that absorbed its ReLU for training (BN+ReLU fusion) keeps it when folded into the convolution
        return self._with_relu or (self._with_bn and getattr(self.bn_layer, "fuse_relu", False))

    def forward(self, x):
        from ....utils import TRAIN_MODE
        if self.model.mode == TRAIN_MODE:
            raise RuntimeError("Fused layers cannot be used in training mode!")
        if self._with_bn:
            self._refresh_bn()
        L = _lib.lib()
        self._timed("fprop", lambda: L.b2c_conv_fprop(
            ctypes.byref(self.desc), x.ptr, self.weights.ptr, self.biases.ptr if self.use_bias else None,
            ctypes.byref(self._bn) if self._with_bn else None, int(self._relu_flag()),
            self.y.ptr, wsp.ptr(), wsp.size(), self.model.stream_handle))
        return self.y

    def backward(self, dy):
        raise RuntimeError("Backward method of a fused layer should not be called")


class Conv2DReluGPU(_FusedConvInference, Conv2DRelu):
    _with_relu = True


class Conv2DBatchNormalizationGPU(_FusedConvInference, Conv2DBatchNormalization):
    _with_bn = True


class Conv2DBatchNormalizationReluGPU(_FusedConvInference, Conv2DBatchNormalizationRelu):
    _with_bn = True
    _with_relu = True
