"""Front ends of the layers either side of the convolution (shape rules only):
Input, BatchNormalization, Relu, Softmax, pooling, AdditionBlock, Flatten, Dropout and the three
fused inference shells (pydtnn/layers/*.py)."""
from abc import ABC

import numpy as np

from .. import initializers
from ..utils import decode_tensor, encode_tensor
from .base import Layer, pair, window_output_extent
from .conv_2d import Conv2D


class Input(Layer, ABC):
    def __init__(self, shape=(1,)):
        super().__init__(tuple(shape))

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        # model files give (h, w, c); store it in the model's tensor format (pydtnn/layers/input.py)
        self.shape = encode_tensor(self.shape, self.model.tensor_format)


class BatchNormalization(Layer, ABC):
    """pydtnn/layers/batch_normalization.py:28-62"""

    def __init__(self, beta=0.0, gamma=1.0, momentum=0.9, epsilon=1e-5, moving_mean_initializer="zeros",
                 moving_variance_initializer="zeros", sync_stats=False):
        super().__init__()
        if sync_stats:
            raise NotImplementedError("sync_stats is outside the supported path (statistics stay per replica)")
        self.gamma_init_val, self.beta_init_val = gamma, beta
        self.momentum, self.epsilon = momentum, epsilon
        self.moving_mean_initializer = getattr(initializers, moving_mean_initializer)
        self.moving_variance_initializer = getattr(initializers, moving_variance_initializer)
        self.grad_vars = {"beta": "dbeta", "gamma": "dgamma"}
        self.sync_stats = sync_stats
        self.spatial = self.co = self.ci = self.hi = self.wi = 0

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.shape = prev_shape
        self.spatial = len(self.shape) > 2
        if self.spatial:
            self.hi, self.wi, self.ci = decode_tensor(self.shape, self.model.tensor_format)
        else:
            self.hi = self.wi = 1
            self.ci = self.shape[0]
        self.co = self.ci
        self.nparams = 4 * self.ci


class Relu(Layer, ABC):
    def __init__(self, shape=(1,)):
        super().__init__(shape)

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.shape = prev_shape


class Softmax(Layer, ABC):
    def __init__(self, shape=(1,)):
        super().__init__(shape)

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.shape = prev_shape


class Dropout(Layer, ABC):
    def __init__(self, rate=0.5):
        super().__init__()
        self.rate = rate

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.shape = prev_shape


class Flatten(Layer, ABC):
    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.shape = (int(np.prod(prev_shape)),)


class _Pool2D(Layer, ABC):
    """pydtnn/layers/abstract_pool_2d_layer.py:28-57"""

    def __init__(self, pool_shape=(2, 2), padding=0, stride=1, dilation=1):
        super().__init__()
        self.pool_shape = tuple(pool_shape)
        self.padding, self.stride, self.dilation = padding, stride, dilation
        (self.vpadding, self.hpadding), (self.vstride, self.hstride) = pair(padding), pair(stride)
        self.vdilation, self.hdilation = pair(dilation)

    def initialize(self, prev_shape, need_dx=True):
        super().initialize(prev_shape, need_dx)
        self.hi, self.wi, self.ci = decode_tensor(prev_shape, self.model.tensor_format)
        if self.pool_shape[0] == 0:
            self.pool_shape = (self.hi, self.pool_shape[1])
        if self.pool_shape[1] == 0:
            self.pool_shape = (self.pool_shape[0], self.wi)
        self.kh, self.kw = self.pool_shape
        self.co = self.ci
        self.ho = window_output_extent(self.hi, self.kh, self.vpadding, self.vstride, self.vdilation)
        self.wo = window_output_extent(self.wi, self.kw, self.hpadding, self.hstride, self.hdilation)
        assert self.ho > 0 and self.wo > 0, "Output dimensions must be greater than 0"
        self.shape = encode_tensor((self.ho, self.wo, self.co), self.model.tensor_format)


class MaxPool2D(_Pool2D, ABC):
    pass


class AveragePool2D(_Pool2D, ABC):
    pass


class AdditionBlock(Layer, ABC):
    """Parallel paths whose outputs are summed; an empty path is the identity
    (pydtnn/layers/abstract_block_layer.py:25-61, pydtnn/layers/addition_block.py)."""

    def __init__(self, *paths):
        super().__init__()
        self.paths = [list(p) for p in paths]
        self.is_block_layer = True
        self.out_shapes = []


class Conv2DRelu(Conv2D, ABC):
    """Inference-only fusion shells built from already-initialised parents
    (pydtnn/layers/conv_2d_relu.py, conv_2d_batch_normalization.py, conv_2d_batch_normalization_relu.py:26-37)."""

    def __init__(self, *args, from_parent=None, **kwargs):
        if from_parent is None:
            super().__init__(*args, **kwargs)
        else:
            self.__dict__.update(from_parent.__dict__)


class Conv2DBatchNormalization(Conv2D, ABC):
    def __init__(self, *args, from_parent=None, from_parent_2=None, **kwargs):
        if from_parent is None:
            super().__init__(*args, **kwargs)
        else:
            self.__dict__.update(from_parent.__dict__)
            bn = {k: v for k, v in from_parent_2.__dict__.items()
                  if k in ("gamma", "beta", "running_mean", "running_var", "epsilon", "momentum")}
            self.__dict__.update(bn)
            self.bn_layer = from_parent_2


class Conv2DBatchNormalizationRelu(Conv2DBatchNormalization, ABC):
    pass
