"""Conv2D front end: the constructor arguments, geometry attributes and weight-shape rule other code reads
(interface of pydtnn/layers/conv_2d.py:28-78)."""
from abc import ABC

import numpy as np

from ..utils import PYDTNN_TENSOR_FORMAT_NCHW, decode_tensor, encode_tensor
from .base import Layer, ParametrisedLayerMixin, pair, window_output_extent


class Conv2D(ParametrisedLayerMixin, Layer, ABC):

    def __init__(self, nfilters=1, filter_shape=(3, 3), grouping=None, padding=0, stride=1,
                 dilation=1, activation="", use_bias=True, weights_initializer="glorot_uniform",
                 biases_initializer="zeros"):
        super().__init__()
        if grouping is not None:
            raise NotImplementedError("grouped (depthwise / pointwise) convolutions are outside the supported path")
        self._init_parameters(activation, use_bias, weights_initializer, biases_initializer)
        self.co, self.filter_shape, self.grouping = nfilters, tuple(filter_shape), grouping
        self.padding, self.stride, self.dilation = padding, stride, dilation
        (self.vpadding, self.hpadding), (self.vstride, self.hstride) = pair(padding), pair(stride)
        self.vdilation, self.hdilation = pair(dilation)
        # filled by initialize()
        self.hi = self.wi = self.ci = self.kh = self.kw = self.ho = self.wo = 0
        self.weights_shape = None

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        fmt = self.model.tensor_format
        self.hi, self.wi, self.ci = decode_tensor(prev_shape, fmt)
        self.kh, self.kw = self.filter_shape
        self.ho = window_output_extent(self.hi, self.kh, self.vpadding, self.vstride, self.vdilation)
        self.wo = window_output_extent(self.wi, self.kw, self.hpadding, self.hstride, self.hdilation)
        self.shape = encode_tensor((self.ho, self.wo, self.co), fmt)
        # filter tensor: (co, ci, kh, kw) in NCHW models, (ci, kh, kw, co) in NHWC models (the GPU layer re-states
        # the latter as (co, kh, kw, ci), see Conv2DGPU.initialize)
        self.weights_shape = (self.co, self.ci, self.kh, self.kw) if fmt == PYDTNN_TENSOR_FORMAT_NCHW \
            else (self.ci, self.kh, self.kw, self.co)
        self.nparams = int(np.prod(self.weights_shape)) + (self.co if self.use_bias else 0)
