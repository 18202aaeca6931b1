"""Device tensor handle with the attributes the reference's ``TensorGPU`` exposes
(pydtnn/backends/gpu/tensor_gpu.py:31-66): ``.ary`` (device array with ``shape``, ``size``,
``get()``, ``set()``, ``reshape()``, ``gpudata``), ``.ptr`` (``ctypes.c_void_p``), ``.size`` and a
``.shape`` promoted to 4-D.  Storage comes from ``torch.empty``; torch is used for allocation and
host<->device copies only.
"""
import ctypes

import numpy as np
import torch

from .utils import PYDTNN_TENSOR_FORMAT_NCHW

_TORCH_DTYPE = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
                np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64}


class DeviceArray:
    """Stands in for ``pycuda.gpuarray.GPUArray`` for the members the layer code touches."""

    def __init__(self, tensor: torch.Tensor):
        assert tensor.is_contiguous()
        self.t = tensor

    @property
    def shape(self):
        return tuple(self.t.shape)

    @property
    def size(self):
        return self.t.numel()

    @property
    def dtype(self):
        return {v: k for k, v in _TORCH_DTYPE.items()}[self.t.dtype]

    @property
    def gpudata(self):
        return self.t.data_ptr()

    def get(self):
        return self.t.detach().cpu().numpy()

    def set(self, host):
        src = torch.from_numpy(np.ascontiguousarray(host, dtype=self.dtype)).reshape(self.t.shape)
        self.t.copy_(src, non_blocking=True)

    def set_async(self, host, stream=None):
        self.set(host)

    def reshape(self, shape):
        return DeviceArray(self.t.view(*shape))

    def fill(self, value):
        self.t.fill_(value)
        return self


def empty(shape, dtype, device=None):
    device = device or torch.device("cuda", torch.cuda.current_device())
    return DeviceArray(torch.empty(tuple(int(s) for s in shape), dtype=_TORCH_DTYPE[np.dtype(dtype)], device=device))


def zeros(shape, dtype, device=None):
    return empty(shape, dtype, device).fill(0)


def to_gpu(host, device=None):
    a = empty(host.shape, host.dtype, device)
    a.set(host)
    return a


class TensorGPU:
    def __init__(self, gpu_arr: DeviceArray, tensor_format, cudnn_dtype=None, tensor_type="tensor", desc=None,
                 gpudirect=False, cublas=False):
        if len(gpu_arr.shape) == 2:
            if tensor_format == PYDTNN_TENSOR_FORMAT_NCHW:
                self.shape = (*gpu_arr.shape, 1, 1)
            else:
                self.shape = (gpu_arr.shape[0], 1, 1, gpu_arr.shape[1])
        else:
            self.shape = gpu_arr.shape
        self.size = gpu_arr.size
        self.ary = gpu_arr
        self.tensor_format = tensor_format
        self.tensor_type = tensor_type
        self.desc = desc

    @property
    def ptr(self):
        return ctypes.c_void_p(self.ary.gpudata)

    def reshape(self, shape):
        self.ary = self.ary.reshape(shape)
        return self
