"""GPU back-end layer classes, looked up by name (``<FrontEndName>GPU``) when a front-end class is
constructed -- the plug-in mechanism of pydtnn/backends/__init__.py:28-51 and
pydtnn/backends/gpu/layers/__init__.py:29-45."""
from .aux_gpu import (AdditionBlockGPU, AveragePool2DGPU, BatchNormalizationGPU, DropoutGPU, FlattenGPU, InputGPU,
                      MaxPool2DGPU, ReluGPU, SoftmaxGPU)
from .conv_2d_gpu import Conv2DBatchNormalizationGPU, Conv2DBatchNormalizationReluGPU, Conv2DGPU, Conv2DReluGPU
from .fc_gpu import FCGPU
from .layer_gpu import LayerGPU

__all__ = [n for n in dir() if n.endswith("GPU")]
