"""FC front end (pydtnn/layers/fc.py:27-42)."""
from abc import ABC

from .. import initializers
from .base import Layer
from .conv_2d import _resolve_activation


class FC(Layer, ABC):

    def __init__(self, shape=(1,), activation="", use_bias=True, weights_initializer="glorot_uniform",
                 biases_initializer="zeros"):
        super().__init__(tuple(shape))
        self.act = _resolve_activation(activation)
        self.use_bias = use_bias
        self.weights_initializer = getattr(initializers, weights_initializer)
        self.biases_initializer = getattr(initializers, biases_initializer)
        self.grad_vars = {"weights": "dw"}
        if self.use_bias:
            self.grad_vars["biases"] = "db"
