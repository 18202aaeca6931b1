"""Write a checkpoint with the reference's own ``Model.store_weights_and_bias`` and the evaluation output of that
model on a fixed input, for the checkpoint interop test.

    python tests/golden/make_checkpoint_golden.py        # needs the reference tree and oracle/_ref built

Produces ``tests/golden/ref_checkpoint_<layout>.npz`` (the reference's file, unmodified) and
``tests/golden/ref_checkpoint_io.npz`` (input, output per layout).  The net: Input(8,8,3) -> Conv2D(8, 3x3, pad 1)
-> BatchNormalization -> Relu -> AdditionBlock([Conv2D(8, 3x3, pad 1), BatchNormalization], []) -> Relu
-> MaxPool2D(2, stride 2) -> Flatten -> FC(5) -> Softmax.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("PYDTNN_REFERENCE", "/root/reference")
sys.path.insert(0, os.path.join(REPO, "oracle", "_ref"))
sys.path.insert(0, REF)

from pydtnn.model import Model, TRAIN_MODE, EVALUATE_MODE  # noqa: E402
from pydtnn.layers import (Input, Conv2D, BatchNormalization, MaxPool2D, Flatten, FC, AdditionBlock)  # noqa: E402
from pydtnn.activations import Relu, Softmax  # noqa: E402
import pydtnn.backends.cpu.layers.batch_normalization_cpu as bn_mod  # noqa: E402


def build(layout):
    # model_name="" keeps the reference from building its default network first
    m = Model(dtype=np.float32, batch_size=4, enable_conv_gemm=False, enable_best_of=False, tensor_format=layout,
              model_name="")
    m.add(Input(shape=(8, 8, 3)))          # the reference takes (h, w, c) here for both tensor formats
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


def forward(m, x, mode):
    m.mode = mode
    for layer in m.layers[1:]:
        x = layer.forward(x)
    return x


def main():
    io = {}
    for layout in ("NHWC", "NCHW"):
        np.random.seed(7)
        m = build(layout)
        rng = np.random.Generator(np.random.PCG64(11))
        for layer in m.get_all_layers():
            # non-trivial values everywhere a checkpoint stores something
            if layer.canonical_name in ("Conv2D", "FC"):
                layer.biases = rng.standard_normal(layer.biases.shape).astype(np.float32)
            if layer.canonical_name == "BatchNormalization":
                layer.gamma = (1.0 + 0.1 * rng.standard_normal(layer.gamma.shape)).astype(np.float32)
                layer.beta = (0.1 * rng.standard_normal(layer.beta.shape)).astype(np.float32)
                layer.running_mean = (0.2 * rng.standard_normal(layer.running_mean.shape)).astype(np.float32)
                layer.running_var = (1.0 + 0.3 * rng.random(layer.running_var.shape)).astype(np.float32)
                layer.updated_running_var = True
                # the NCHW evaluation branch of the reference returns before it refreshes inv_std
                # (batch_normalization_cpu.py:50-52 against :90-92): give it the value the NHWC branch computes
                layer.inv_std = (1.0 / np.sqrt(layer.running_var + layer.epsilon)).astype(np.float32)
        x = rng.standard_normal((4, 8, 8, 3)).astype(np.float32)
        xl = x if layout == "NHWC" else np.ascontiguousarray(x.transpose(0, 3, 1, 2))
        y = forward(m, xl, EVALUATE_MODE)
        path = os.path.join(HERE, f"ref_checkpoint_{layout}")
        m.store_weights_and_bias(path)
        io[f"x_{layout}"] = xl
        io[f"y_{layout}"] = y
        print(layout, sorted(np.load(path + ".npz").keys()))
    np.savez_compressed(os.path.join(HERE, "ref_checkpoint_io.npz"), **io)


if __name__ == "__main__":
    main()
