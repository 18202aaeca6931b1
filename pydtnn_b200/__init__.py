"""B200-native convolution / FC back end behind the PyDTNN layer API.

The compute path is ``libb2c.so`` (hand-written sm_100a CUDA behind the C ABI in
``include/b2c.h``); this package mirrors the reference's Layer / Model interface on top of it.
PyTorch is used for device memory, host<->device copies, streams and ``torch.distributed``."""
from . import _lib  # noqa: F401
from ._lib import B2CError  # noqa: F401

__version__ = "0.1.0"
