"""Checkpoint interop on the device: a file the reference wrote (``tests/golden/ref_checkpoint_*.npz``) loads into
the same network built from this package and reproduces the reference's evaluation output; the file written back
equals the reference's file array by array."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _net(layout, seed):
    from pydtnn_b200.layers import (FC, AdditionBlock, BatchNormalization, Conv2D, Flatten, Input, MaxPool2D, Relu,
                                    Softmax)
    from pydtnn_b200.model import Model
    np.random.seed(seed)
    m = Model(batch_size=4, tensor_format=layout, dtype=np.float32)
    m.add(Input(shape=(8, 8, 3)))
    m.add(Conv2D(nfilters=8, filter_shape=(3, 3), padding=1, weights_initializer="he_uniform"))
    m.add(BatchNormalization())
    m.add(Relu())
    m.add(AdditionBlock([Conv2D(nfilters=8, filter_shape=(3, 3), padding=1, weights_initializer="he_uniform"),
                         BatchNormalization()], []))
    m.add(Relu())
    m.add(MaxPool2D(pool_shape=(2, 2), stride=2))
    m.add(Flatten())
    m.add(FC(shape=(5,), weights_initializer="he_uniform"))
    m.add(Softmax())
    return m


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_reference_checkpoint_loads_and_reproduces_the_reference_output(layout, tmp_path):
    io = np.load(os.path.join(GOLD, "ref_checkpoint_io.npz"))
    ref_file = os.path.join(GOLD, f"ref_checkpoint_{layout}.npz")
    m = _net(layout, 1)
    assert m.load_weights_and_bias(ref_file) == []
    y = m.evaluate_batch(io[f"x_{layout}"]).ary.get()
    ref = io[f"y_{layout}"]
    assert np.linalg.norm(y.reshape(ref.shape) - ref) <= 1e-5 * np.linalg.norm(ref)

    # written back in the reference CPU layout: the same arrays under the same keys
    out = os.path.join(tmp_path, "back.npz")
    m.store_weights_and_bias(out, layout="cpu")
    a, b = np.load(ref_file), np.load(out)
    assert set(a) == set(b) - {"b2c_conv_weight_layout"}
    for k in a:
        assert a[k].shape == b[k].shape and np.array_equal(a[k], b[k]), k

    # and in the GPU layers' own layout into a differently initialised model
    out2 = os.path.join(tmp_path, "native.npz")
    m.store_weights_and_bias(out2, layout="gpu")
    m2 = _net(layout, 2)
    m2.evaluate_batch(io[f"x_{layout}"])          # an evaluation before the load must not leave stale statistics behind
    assert m2.load_weights_and_bias(out2) == []
    y2 = m2.evaluate_batch(io[f"x_{layout}"]).ary.get()
    assert np.array_equal(y, y2)
