"""Layer lists of the three networks the benchmark configurations name, written with this
package's front-end classes.  Shapes follow the reference model files
(pydtnn/models/resnet50_imagenet.py:24-63, vgg16_imagenet.py:23-37, alexnet_imagenet.py:23-39)."""
from .layers import (FC, AdditionBlock, AveragePool2D, BatchNormalization, Conv2D, Dropout, Flatten, Input,
                     MaxPool2D, Relu)


def create_resnet50_imagenet(model, input_hw=224, nclasses=1000, layout=None):
    """ResNet-50 v1.5: stem 7x7/2 convolution with bias and no BN/ReLU, 3x3/2 max pool, 16 bottleneck
    AdditionBlocks (the stride sits on the 3x3), global average pool, FC + softmax."""
    _ = model.add
    _(Input(shape=(input_hw, input_hw, 3)))
    _(Conv2D(nfilters=64, filter_shape=(7, 7), stride=2, padding=3, weights_initializer="he_uniform"))
    _(MaxPool2D(pool_shape=(3, 3), stride=2, padding=1))
    expansion = 4
    layout = layout or [[64, 3, 1], [128, 4, 2], [256, 6, 2], [512, 3, 2]]
    for n_filt, res_blocks, stride in layout:
        for r in range(res_blocks):
            if r > 0:
                stride = 1
            _(AdditionBlock(
                [Conv2D(nfilters=n_filt, filter_shape=(1, 1), stride=1, weights_initializer="he_uniform"),
                 BatchNormalization(), Relu(),
                 Conv2D(nfilters=n_filt, filter_shape=(3, 3), stride=stride, padding=1, weights_initializer="he_uniform"),
                 BatchNormalization(), Relu(),
                 Conv2D(nfilters=n_filt * expansion, filter_shape=(1, 1), stride=1, weights_initializer="he_uniform"),
                 BatchNormalization()],
                [Conv2D(nfilters=n_filt * expansion, filter_shape=(1, 1), stride=stride, weights_initializer="he_uniform"),
                 BatchNormalization()] if r == 0 or stride != 1 else []))
            _(Relu())
    _(AveragePool2D(pool_shape=(0, 0)))
    _(Flatten())
    _(FC(shape=(nclasses,), activation="softmax"))


def create_vgg16_imagenet(model, input_hw=224, nclasses=1000, batch_norm=False, with_dropout=False):
    """13 3x3 convolutions (+ReLU) in 5 stages with 2x2/2 max pools, then FC 4096-4096-1000.
    ``batch_norm`` inserts a BatchNormalization after every convolution (benchmark configuration 3)."""
    _ = model.add
    _(Input(shape=(input_hw, input_hw, 3)))
    for n_filt, convs in ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3)):
        for _i in range(convs):
            if batch_norm:
                _(Conv2D(nfilters=n_filt, filter_shape=(3, 3), padding=1, weights_initializer="he_uniform"))
                _(BatchNormalization())
                _(Relu())
            else:
                _(Conv2D(nfilters=n_filt, filter_shape=(3, 3), padding=1, activation="relu", weights_initializer="he_uniform"))
        _(MaxPool2D(pool_shape=(2, 2), stride=2))
    _(Flatten())
    _(FC(shape=(4096,), activation="relu", weights_initializer="he_uniform"))
    if with_dropout:
        _(Dropout(rate=0.5))
    _(FC(shape=(4096,), activation="relu", weights_initializer="he_uniform"))
    if with_dropout:
        _(Dropout(rate=0.5))
    _(FC(shape=(nclasses,), activation="softmax", weights_initializer="he_uniform"))


def create_vgg16bn_imagenet(model, **kw):
    create_vgg16_imagenet(model, batch_norm=True, **kw)


def create_alexnet_imagenet(model, nclasses=1000):
    """5 convolutions (11x11/4, 5x5, 3x3 x3) + 3 FC on 227x227 inputs; dropout is the identity in
    evaluation, the only mode the benchmark uses this network in."""
    _ = model.add
    _(Input(shape=(227, 227, 3)))
    _(Conv2D(nfilters=96, filter_shape=(11, 11), padding=0, stride=4, activation="relu", weights_initializer="he_uniform"))
    _(MaxPool2D(pool_shape=(3, 3), stride=2))
    _(Conv2D(nfilters=256, filter_shape=(5, 5), padding=2, stride=1, activation="relu", weights_initializer="he_uniform"))
    _(MaxPool2D(pool_shape=(3, 3), stride=2))
    _(Conv2D(nfilters=384, filter_shape=(3, 3), padding=1, stride=1, activation="relu", weights_initializer="he_uniform"))
    _(Conv2D(nfilters=384, filter_shape=(3, 3), padding=1, stride=1, activation="relu", weights_initializer="he_uniform"))
    _(Conv2D(nfilters=256, filter_shape=(3, 3), padding=1, stride=1, activation="relu", weights_initializer="he_uniform"))
    _(MaxPool2D(pool_shape=(3, 3), stride=2))
    _(Flatten())
    _(FC(shape=(4096,), activation="relu", weights_initializer="he_uniform"))
    _(Dropout(rate=0.5))
    _(FC(shape=(4096,), activation="relu", weights_initializer="he_uniform"))
    _(Dropout(rate=0.5))
    _(FC(shape=(nclasses,), activation="softmax", weights_initializer="he_uniform"))
