"""Build the CPU-oracle twin of a GPU model (same layer list, same parameters)."""
import numpy as np

from oracle import cpu_model as cm
from pydtnn_b200.utils import PYDTNN_TENSOR_FORMAT_NCHW


def _real(layers):
    """Dropout is the identity in evaluation and has no CPU node."""
    return [l for l in layers if l.canonical_name != "Dropout"]


def _spec(layers):
    spec = []
    for l in _real(layers):
        name = l.canonical_name
        if name == "Conv2D":
            spec.append(("conv", l.co, l.kh, l.vstride, l.vpadding))
        elif name == "BatchNormalization":
            spec.append(("bn",))
        elif name == "Relu":
            spec.append(("relu",))
        elif name == "MaxPool2D":
            spec.append(("maxpool", l.kh, l.vstride, l.vpadding))
        elif name == "AveragePool2D":
            spec.append(("gap",) if (l.kh, l.kw) == (l.hi, l.wi) else ("avgpool", l.kh, l.vstride, l.vpadding))
        elif name == "Flatten":
            spec.append(("flatten",))
        elif name == "FC":
            spec.append(("fc", l.shape[0]))
        elif name == "Softmax":
            spec.append(("softmax",))
        elif name == "AdditionBlock":
            spec.append(("add", *[_spec(p) for p in l.paths]))
        else:
            raise ValueError(name)
    return spec


def _copy(layers, nodes, nchw):
    for l, n in zip(_real(layers), nodes):
        name = l.canonical_name
        if name == "Conv2D":
            w = l.weights.ary.get()
            n.w = w.copy() if nchw else np.ascontiguousarray(w.transpose(3, 1, 2, 0))
            n.b = l.biases.ary.get().reshape(-1).copy()
        elif name == "BatchNormalization":
            n.gamma, n.beta = l.gamma.ary.get().copy(), l.beta.ary.get().copy()
        elif name == "FC":
            n.w, n.b = l.weights.ary.get().copy(), l.biases.ary.get().reshape(-1).copy()
        elif name == "AdditionBlock":
            for lp, npth in zip(l.paths, n.paths):
                _copy(lp, npth, nchw)


def cpu_twin(model):
    nchw = model.tensor_format == PYDTNN_TENSOR_FORMAT_NCHW
    in_shape = model.layers[0].shape
    hwc = (in_shape[1], in_shape[2], in_shape[0]) if nchw else in_shape
    net = cm.CpuNet(_spec(model.layers[1:]), hwc, model.batch_size, model.dtype, "NCHW" if nchw else "NHWC")
    _copy(model.layers[1:], net.nodes, nchw)
    return net


def grads_of(layer, nchw):
    """Gradients of a GPU layer in the oracle's layouts, keyed like the CPU node attributes."""
    name = layer.canonical_name
    if name == "Conv2D":
        dw = layer.dw.ary.get()
        return {"dw": dw if nchw else dw.transpose(3, 1, 2, 0), "db": layer.db.ary.get().reshape(-1)}
    if name == "BatchNormalization":
        return {"dgamma": layer.dgamma.ary.get(), "dbeta": layer.dbeta.ary.get()}
    if name == "FC":
        return {"dw": layer.dw.ary.get(), "db": layer.db.ary.get().reshape(-1)}
    return {}


def params_of(layer, nchw):
    name = layer.canonical_name
    if name == "Conv2D":
        w = layer.weights.ary.get()
        return {"w": w if nchw else w.transpose(3, 1, 2, 0), "b": layer.biases.ary.get().reshape(-1)}
    if name == "BatchNormalization":
        return {"gamma": layer.gamma.ary.get(), "beta": layer.beta.ary.get()}
    if name == "FC":
        return {"w": layer.weights.ary.get(), "b": layer.biases.ary.get().reshape(-1)}
    return {}


def walk_pairs(layers, nodes):
    for l, n in zip(_real(layers), nodes):
        yield l, n
        if l.canonical_name == "AdditionBlock":
            for lp, npth in zip(l.paths, n.paths):
                yield from walk_pairs(lp, npth)
