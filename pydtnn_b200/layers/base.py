"""Base classes of the layer API (pydtnn/layers/layer_and_activation_base.py:25-106,
pydtnn/layers/layer.py:28-32, pydtnn/backends/__init__.py:28-67)."""
import importlib
from abc import ABC, abstractmethod

import numpy as np


class PromoteToBackendMixin:
    """``Conv2D(...)`` returns a ``Conv2DGPU``: the class named ``<Name>GPU`` is looked up in
    ``pydtnn_b200.backends.gpu.layers`` and instantiated instead."""

    def __new__(cls, *args, **kwargs):
        if ".backends." in cls.__module__:
            return super().__new__(cls)
        module = importlib.import_module("pydtnn_b200.backends.gpu.layers")
        new_cls = getattr(module, cls.__name__ + "GPU", None)
        if new_cls is None:
            raise NotImplementedError(f"{cls.__name__} has no GPU back end in this package")
        instance = super().__new__(new_cls)
        instance.__init__(*args, **kwargs)
        return instance

    @property
    def canonical_name(self):
        name = self.__class__.__name__
        return name[:-3] if name.endswith("GPU") else name


class LayerAndActivationBase(ABC):

    def __init__(self, shape=()):
        self.nparams = 0
        self.shape = shape
        self.weights = np.array([])
        self.biases = np.array([])
        self.act = None
        self.grad_vars = {}
        self.fwd_time = np.zeros((4,), dtype=np.float32)
        self.bwd_time = np.zeros((4,), dtype=np.float32)
        self.paths = []
        self.need_dx = True
        self.reqs_allred = {}
        self.id = None
        self.model = None
        self.prev_shape = None
        self.is_block_layer = False
        self.stream_2 = None

    def set_model(self, parent_model):
        self.model = parent_model
        self.id = next(self.model.layer_id)

    def initialize(self, prev_shape, need_dx=True):
        self.prev_shape = prev_shape
        self.need_dx = need_dx

    @abstractmethod
    def forward(self, x):
        pass

    @abstractmethod
    def backward(self, dy):
        pass

    @abstractmethod
    def reduce_weights_async(self):
        pass

    @abstractmethod
    def wait_allreduce_async(self):
        pass

    @abstractmethod
    def reduce_weights_sync(self):
        pass

    @property
    def children(self):
        out = []
        for path in self.paths:
            out += [layer for layer in path]
        return out

    def update_weights(self, optimizer):
        optimizer.update(self)

    def __repr__(self):
        return f"{self.id}_{type(self).__name__}"


class Layer(PromoteToBackendMixin, LayerAndActivationBase, ABC):
    @property
    def canonical_name_with_id(self):
        return f"{self.id}_{self.canonical_name}"
