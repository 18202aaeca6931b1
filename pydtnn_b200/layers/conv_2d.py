"""Conv2D front end: arguments, geometry and weight-shape rules of pydtnn/layers/conv_2d.py:28-78."""
from abc import ABC

import numpy as np

from .. import initializers
from ..utils import PYDTNN_TENSOR_FORMAT_NCHW, decode_tensor, encode_tensor
from .base import Layer


def _resolve_activation(name):
    if not name:
        return None
    from . import others
    table = {"relu": others.Relu, "softmax": others.Softmax}
    if name not in table:
        raise NotImplementedError(f"activation '{name}' is not available in this package")
    return table[name]


class Conv2D(Layer, ABC):

    def __init__(self, nfilters=1, filter_shape=(3, 3), grouping=None, padding=0, stride=1,
                 dilation=1, activation="", use_bias=True, weights_initializer="glorot_uniform",
                 biases_initializer="zeros"):
        super().__init__()
        if grouping is not None:
            raise NotImplementedError("grouped (depthwise / pointwise) convolutions are outside the supported path")
        self.co = nfilters
        self.filter_shape = tuple(filter_shape)
        self.grouping = grouping
        self.padding = padding
        self.stride = stride
        self.dilation = dilation
        self.vpadding, self.hpadding = (padding, padding) if isinstance(padding, int) else padding
        self.vstride, self.hstride = (stride, stride) if isinstance(stride, int) else stride
        self.vdilation, self.hdilation = (dilation, dilation) if isinstance(dilation, int) else dilation
        self.act = _resolve_activation(activation)
        self.use_bias = use_bias
        self.weights_initializer = getattr(initializers, weights_initializer)
        self.biases_initializer = getattr(initializers, biases_initializer)
        self.grad_vars = {"weights": "dw"}
        if self.use_bias:
            self.grad_vars["biases"] = "db"
        self.ci = self.hi = self.wi = self.kh = self.kw = self.ho = self.wo = 0
        self.weights_shape = None

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.hi, self.wi, self.ci = decode_tensor(prev_shape, self.model.tensor_format)
        self.kh, self.kw = self.filter_shape
        if self.model.tensor_format == PYDTNN_TENSOR_FORMAT_NCHW:
            self.weights_shape = (self.co, self.ci, *self.filter_shape)
        else:
            self.weights_shape = (self.ci, *self.filter_shape, self.co)
        self.ho = (self.hi + 2 * self.vpadding - self.vdilation * (self.kh - 1) - 1) // self.vstride + 1
        self.wo = (self.wi + 2 * self.hpadding - self.hdilation * (self.kw - 1) - 1) // self.hstride + 1
        self.shape = encode_tensor((self.ho, self.wo, self.co), self.model.tensor_format)
        self.nparams = int(np.prod(self.weights_shape)) + (self.co if self.use_bias else 0)
