"""Flat parameter / gradient storage.

Every trainable tensor of a model is a view into a few large contiguous device buffers: one for
the parameters, one (same offsets) for their gradients and, once an optimiser needs it, one for
the velocities.  The weight-gradient kernels therefore write straight into the memory NCCL
all-reduces (no gather copy), a gradient bucket is an address range, and the SGD update is one
launch per buffer instead of one per tensor (the reference launches one elementwise kernel per
tensor, pydtnn/backends/gpu/optimizers/sgd_gpu.py:63-88)."""
import numpy as np
import torch

from .tensor_gpu import _TORCH_DTYPE, DeviceArray

ALIGN_ELEMS = 64


class _Chunk:
    def __init__(self, capacity, tdtype, device):
        self.w = torch.zeros(capacity, dtype=tdtype, device=device)
        self.dw = torch.zeros(capacity, dtype=tdtype, device=device)
        self.v = None
        self.used = 0
        self.capacity = capacity


class ParamArena:
    def __init__(self, dtype, device, chunk_elems=32 * 1024 * 1024):
        self.dtype = np.dtype(dtype)
        self.tdtype = _TORCH_DTYPE[self.dtype]
        self.device = torch.device(device)
        self.chunk_elems = int(chunk_elems)
        self.chunks = []
        self.entries = []      # (chunk index, offset, numel) in allocation (= forward) order
        self._by_ptr = {}      # gradient data_ptr -> entry index

    def alloc_param(self, host_array):
        """Copy ``host_array`` into the arena; returns (parameter view, gradient view)."""
        host_array = np.ascontiguousarray(host_array, dtype=self.dtype)
        numel = host_array.size
        padded = (numel + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        if not self.chunks or self.chunks[-1].used + padded > self.chunks[-1].capacity:
            self.chunks.append(_Chunk(max(self.chunk_elems, padded), self.tdtype, self.device))
        ci = len(self.chunks) - 1
        ch = self.chunks[ci]
        off = ch.used
        ch.used += padded
        w = ch.w[off:off + numel].view(*host_array.shape)
        dw = ch.dw[off:off + numel].view(*host_array.shape)
        w.copy_(torch.from_numpy(host_array))
        self.entries.append((ci, off, numel))
        self._by_ptr[dw.data_ptr()] = len(self.entries) - 1
        return DeviceArray(w), DeviceArray(dw)

    def entry_of(self, grad_array: DeviceArray):
        return self._by_ptr[grad_array.gpudata]

    def velocity(self, ci):
        ch = self.chunks[ci]
        if ch.v is None:
            ch.v = torch.zeros(ch.capacity, dtype=self.tdtype, device=self.device)
        return ch.v

    @property
    def nparams(self):
        return sum(n for _, _, n in self.entries)
