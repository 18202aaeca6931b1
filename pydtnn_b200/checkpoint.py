"""Checkpoint interop with the reference's NPZ scheme.

The reference stores one array per trainable tensor under ``"<layer id>_<canonical layer name>_<attribute>"``
(attributes of ``grad_vars`` plus ``running_mean`` / ``running_var`` for batch normalisation), walking addition
and concatenation blocks path by path (pydtnn/model.py:351-387). Arrays are written in the storing back end's
own layout, and its loader only reshapes, so a file written by the reference CPU back end holds convolution
filters as ``(ci, kh, kw, co)`` (NHWC models, pydtnn/layers/conv_2d.py:57-78) or ``(co, ci, kh, kw)`` (NCHW),
while its GPU back end and this package keep ``(co, kh, kw, ci)`` for NHWC (conv_2d_gpu.py:49-51). The functions
here convert between the three on the way in and out, so that weights trained on either side load on the other.

Files written here carry one extra key, ``b2c_conv_weight_layout``, naming the filter layout of the file; the
reference loader looks up its own keys only and ignores it.
"""
import numpy as np

from .utils import PYDTNN_TENSOR_FORMAT_NCHW

LAYOUT_KEY = "b2c_conv_weight_layout"
# axes of each layout in terms of (co, ci, kh, kw)
_AXES = {"KCRS": "kcrs", "KRSC": "krsc", "CRSK": "crsk"}


def convert_conv_weights(w, src, dst):
    """Reorder a 4-D filter array between the layouts ``KCRS`` (co,ci,kh,kw), ``KRSC`` (co,kh,kw,ci) and
    ``CRSK`` (ci,kh,kw,co)."""
    if src == dst:
        return np.ascontiguousarray(w)
    a, b = _AXES[src], _AXES[dst]
    return np.ascontiguousarray(np.transpose(w, [a.index(ch) for ch in b]))


def reference_cpu_layout(tensor_format):
    """Filter layout of the reference's CPU back end for a model of this tensor format."""
    return "KCRS" if tensor_format == PYDTNN_TENSOR_FORMAT_NCHW else "CRSK"


def native_layout(tensor_format):
    """Filter layout of the GPU layers (the reference's GPU back end and this package)."""
    return "KCRS" if tensor_format == PYDTNN_TENSOR_FORMAT_NCHW else "KRSC"


def _resolve(layout, tensor_format):
    if layout in ("cpu", "reference-cpu"):
        return reference_cpu_layout(tensor_format)
    if layout in ("gpu", "native", "reference-gpu"):
        return native_layout(tensor_format)
    if layout in _AXES:
        return layout
    raise ValueError(f"unknown checkpoint filter layout {layout!r}")


def _walk(layers):
    for layer in layers:
        if layer.canonical_name in ("AdditionBlock", "ConcatenationBlock"):
            for path in layer.paths:
                yield from _walk(path)
        else:
            yield layer


def _keys(layer):
    keys = list(layer.grad_vars)
    if layer.canonical_name == "BatchNormalization":
        keys += ["running_var", "running_mean"]
    return keys


def state_dict(model, layout="cpu"):
    """All stored tensors of ``model`` as host arrays under the reference's key names, convolution filters in
    ``layout`` (``"cpu"``: what the reference CPU back end of the same tensor format holds; ``"gpu"``: the GPU
    layers' own layout; or an explicit ``KCRS`` / ``KRSC`` / ``CRSK``)."""
    target = _resolve(layout, model.tensor_format)
    native = native_layout(model.tensor_format)
    d = {}
    for layer in _walk(model.layers):
        name = layer.canonical_name
        for key in _keys(layer):
            arr = getattr(layer, key).ary.get()
            if name == "Conv2D" and key == "weights":
                arr = convert_conv_weights(arr, native, target)
            elif key == "biases" or name == "BatchNormalization":
                arr = np.ascontiguousarray(arr.reshape(-1))        # the reference CPU layers hold plain vectors
            d[f"{layer.id}_{name}_{key}"] = arr
    d[LAYOUT_KEY] = np.array(target)
    return d


def load_state_dict(model, d, layout=None):
    """Copy the arrays of ``d`` (a mapping as ``numpy.load`` returns it) into the model's device tensors.
    ``layout`` names the filter layout of the file when it carries no ``b2c_conv_weight_layout`` key
    (default ``"cpu"``, a file written by the reference CPU back end). Returns the list of missing keys."""
    if LAYOUT_KEY in d:
        source = str(np.asarray(d[LAYOUT_KEY]))
    else:
        source = _resolve(layout or "cpu", model.tensor_format)
    native = native_layout(model.tensor_format)
    missing = []
    for layer in _walk(model.layers):
        name = layer.canonical_name
        if name == "BatchNormalization":
            layer.updated_running_var = True       # as the reference: inv_std is refreshed at the next evaluation
        for key in _keys(layer):
            base = f"{layer.id}_{name}_{key}"
            if base not in d:
                print(f"Could not find '{base}' for layer '{name}' in file!")
                missing.append(base)
                continue
            arr = np.asarray(d[base])
            dst = getattr(layer, key).ary
            if name == "Conv2D" and key == "weights":
                want = convert_conv_weights(np.empty(dst.shape, np.int8), native, source).shape
                if tuple(arr.shape) != tuple(want):
                    raise ValueError(f"{base}: shape {arr.shape} is not the {source} form {want} of this layer's filter")
                arr = convert_conv_weights(arr, source, native)
            if arr.size != dst.size:
                raise ValueError(f"{base}: {arr.size} elements in the file, {dst.size} in the layer")
            dst.set(np.ascontiguousarray(arr, dtype=dst.dtype).reshape(dst.shape))
    return missing


def store_weights_and_bias(model, filename, layout="cpu"):
    """Counterpart of the reference's ``Model.store_weights_and_bias`` (rank 0 writes)."""
    if getattr(model, "rank", 0) != 0:
        return
    np.savez_compressed(filename, **state_dict(model, layout))


def load_weights_and_bias(model, filename, layout=None):
    """Counterpart of the reference's ``Model.load_weights_and_bias``."""
    with np.load(filename) as d:
        return load_state_dict(model, d, layout)
