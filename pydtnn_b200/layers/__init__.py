"""Front-end layer classes: constructor signatures and shape rules of the reference's
``pydtnn.layers`` for the layers the convolution path and a ResNet/VGG/AlexNet step need.
Constructing one returns its GPU back-end subclass (``<Name>GPU``), the way the reference's
``PromoteToBackendMixin`` does (pydtnn/backends/__init__.py:28-51); there is no CPU back end."""
from .base import Layer, LayerAndActivationBase
from .conv_2d import Conv2D
from .fc import FC
from .others import (AdditionBlock, AveragePool2D, BatchNormalization, Conv2DBatchNormalization,
                     Conv2DBatchNormalizationRelu, Conv2DRelu, Dropout, Flatten, Input, MaxPool2D, Relu, Softmax)

__all__ = ["Layer", "LayerAndActivationBase", "Conv2D", "FC", "AdditionBlock", "AveragePool2D",
           "BatchNormalization", "Conv2DBatchNormalization", "Conv2DBatchNormalizationRelu", "Conv2DRelu",
           "Dropout", "Flatten", "Input", "MaxPool2D", "Relu", "Softmax"]
