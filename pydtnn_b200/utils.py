"""Tensor-format helpers with the reference's names and meaning (pydtnn/utils/__init__.py:30-44)."""
import numpy as np

PYDTNN_TENSOR_FORMAT_NHWC, PYDTNN_TENSOR_FORMAT_NCHW = range(2)

TRAIN_MODE, EVALUATE_MODE, UNSPECIFIED_MODE = "train", "evaluate", "unspecified"


def encode_tensor(shape, tensor_format=PYDTNN_TENSOR_FORMAT_NHWC):
    """(h, w, c) -> per-sample shape in the given format."""
    if len(shape) == 3 and tensor_format == PYDTNN_TENSOR_FORMAT_NCHW:
        return (shape[2], shape[0], shape[1])
    return tuple(shape)


def decode_tensor(shape, tensor_format=PYDTNN_TENSOR_FORMAT_NHWC):
    """per-sample shape in the given format -> (h, w, c)."""
    if len(shape) == 3 and tensor_format == PYDTNN_TENSOR_FORMAT_NCHW:
        return (shape[1], shape[2], shape[0])
    return tuple(shape)


def np_dtype(dtype):
    dt = np.dtype(dtype)
    if dt not in (np.dtype(np.float32), np.dtype(np.float64)):
        raise TypeError(f"dtype {dt} is not supported (float32 or float64)")
    return dt
