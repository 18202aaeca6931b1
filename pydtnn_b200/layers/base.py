"""The layer interface this package keeps from the reference (pydtnn/layers/layer_and_activation_base.py:25-106,
pydtnn/layers/layer.py:28-32, pydtnn/backends/__init__.py:28-67): which attributes every layer carries, which hooks a
back end must implement, and how a front-end constructor turns into its GPU class.  Other code reads these names
(``shape``, ``act``, ``grad_vars``, ``paths``, ``need_dx``, ``fwd_time`` ...), so they are part of the interface."""
import importlib
from abc import ABC, abstractmethod

import numpy as np

_BACKEND_MODULE = "pydtnn_b200.backends.gpu.layers"


def pair(value):
    """An int means the same extent vertically and horizontally; a pair is taken as (vertical, horizontal)."""
    return (value, value) if isinstance(value, int) else tuple(value)


def window_output_extent(size, window, padding, stride, dilation):
    """Positions of a sliding window along one axis (pydtnn/layers/conv_2d.py:75-76,
    pydtnn/layers/abstract_pool_2d_layer.py:52-53)."""
    return (size + 2 * padding - dilation * (window - 1) - 1) // stride + 1


class PromoteToBackendMixin:
    """Constructing ``Conv2D(...)`` yields a ``Conv2DGPU``: a class used outside the back-end package is replaced by
    the class of the same name plus ``GPU`` from the back-end package.  There is no CPU back end to fall back to."""

    def __new__(cls, *args, **kwargs):
        if ".backends." in cls.__module__:
            return super().__new__(cls)
        backend_cls = getattr(importlib.import_module(_BACKEND_MODULE), cls.__name__ + "GPU", None)
        if backend_cls is None:
            raise NotImplementedError(f"{cls.__name__} has no GPU back end in this package")
        obj = super().__new__(backend_cls)
        obj.__init__(*args, **kwargs)       # Python skips __init__ when __new__ returns another class's object
        return obj

    @property
    def canonical_name(self):
        name = type(self).__name__
        return name[:-3] if name.endswith("GPU") else name


class LayerAndActivationBase(ABC):
    """State shared by layers and activations, and the five hooks a back end implements."""

    def __init__(self, shape=()):
        # identity within a model (set by set_model / initialize)
        self.model, self.id, self.prev_shape = None, None, None
        # what the model and the optimiser read
        self.shape, self.nparams, self.need_dx = shape, 0, True
        self.weights, self.biases = np.array([]), np.array([])
        self.grad_vars = {}                # parameter attribute -> gradient attribute
        self.act = None                    # activation class appended after this layer by Model.add
        self.paths, self.is_block_layer = [], False
        # bookkeeping slots of the reference's time model and asynchronous exchange
        self.fwd_time = np.zeros((4,), dtype=np.float32)
        self.bwd_time = np.zeros((4,), dtype=np.float32)
        self.reqs_allred = {}
        self.stream_2 = None

    def set_model(self, parent_model):
        self.model = parent_model
        self.id = next(parent_model.layer_id)

    def initialize(self, prev_shape, need_dx=True):
        self.prev_shape, self.need_dx = prev_shape, need_dx

    @abstractmethod
    def forward(self, x):
        """Returns the layer's output handle (the same object on every call)."""

    @abstractmethod
    def backward(self, dy):
        """Fills the parameter gradients; returns the input gradient, or None when ``need_dx`` is False."""

    @abstractmethod
    def reduce_weights_async(self):
        """Start summing this layer's gradients over the ranks."""

    @abstractmethod
    def wait_allreduce_async(self):
        """Make the compute stream wait for that sum."""

    @abstractmethod
    def reduce_weights_sync(self):
        """Both of the above."""

    @property
    def children(self):
        return [layer for path in self.paths for layer in path]

    def update_weights(self, optimizer):
        optimizer.update(self)

    def __repr__(self):
        return f"{self.id}_{type(self).__name__}"


class Layer(PromoteToBackendMixin, LayerAndActivationBase, ABC):
    @property
    def canonical_name_with_id(self):
        return f"{self.id}_{self.canonical_name}"


class ParametrisedLayerMixin:
    """Constructor arguments Conv2D and FC share: activation name, bias switch and the two initialisers."""

    def _init_parameters(self, activation, use_bias, weights_initializer, biases_initializer):
        from .. import initializers
        self.act = resolve_activation(activation)
        self.use_bias = use_bias
        self.weights_initializer = getattr(initializers, weights_initializer)
        self.biases_initializer = getattr(initializers, biases_initializer)
        self.grad_vars = {"weights": "dw", "biases": "db"} if use_bias else {"weights": "dw"}


def resolve_activation(name):
    """Activation argument of Conv2D / FC -> the layer class Model.add appends (None for '')."""
    if not name:
        return None
    from . import others
    known = {"relu": others.Relu, "softmax": others.Softmax}
    if name not in known:
        raise NotImplementedError(f"activation '{name}' is not available in this package")
    return known[name]
