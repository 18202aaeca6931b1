"""Weight initialisers with the reference's names (pydtnn/initializers/__init__.py:28-88).
Fans follow the reference's rule: dimension 0 is "out", dimension 1 is "in", the rest is the
receptive field (``_compute_fans``, :28-37).  Draws come from NumPy's global generator, which
the benchmark seeds, so replicas built with the same seed are identical."""
import numpy as np


def _compute_fans(shape):
    if len(shape) == 2:
        return shape[0], shape[1]
    receptive = int(np.prod(shape[2:]))
    return shape[1] * receptive, shape[0] * receptive


def _uniform(shape, dtype, limit):
    return np.random.uniform(-limit, limit, shape).astype(dtype)


def glorot_uniform(shape, dtype):
    fan_in, fan_out = _compute_fans(shape)
    return _uniform(shape, dtype, np.sqrt(6.0 / (fan_in + fan_out)))


def he_uniform(shape, dtype):
    fan_in, _ = _compute_fans(shape)
    return _uniform(shape, dtype, np.sqrt(6.0 / fan_in))


def he_normal(shape, dtype):
    fan_in, _ = _compute_fans(shape)
    return (np.random.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(dtype)


def lecun_uniform(shape, dtype):
    fan_in, _ = _compute_fans(shape)
    return _uniform(shape, dtype, np.sqrt(3.0 / fan_in))


def zeros(shape, dtype):
    return np.zeros(shape, dtype)


def ones(shape, dtype):
    return np.ones(shape, dtype)
