"""FC front end (interface of pydtnn/layers/fc.py:27-42): ``shape`` is the number of output features."""
from abc import ABC

from .base import Layer, ParametrisedLayerMixin


class FC(ParametrisedLayerMixin, Layer, ABC):

    def __init__(self, shape=(1,), activation="", use_bias=True, weights_initializer="glorot_uniform",
                 biases_initializer="zeros"):
        super().__init__(tuple(shape))
        self._init_parameters(activation, use_bias, weights_initializer, biases_initializer)
