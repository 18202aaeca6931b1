"""Checkpoint interop, the parts that need no GPU: filter layout conversions, key naming and the layouts of
the files the reference itself wrote (``tests/golden/ref_checkpoint_*.npz``, made by
``tests/golden/make_checkpoint_golden.py`` with the reference's ``Model.store_weights_and_bias``)."""
import os

import numpy as np
import pytest

from pydtnn_b200 import checkpoint as ck
from pydtnn_b200.utils import PYDTNN_TENSOR_FORMAT_NCHW, PYDTNN_TENSOR_FORMAT_NHWC

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_filter_layout_conversions_are_permutations():
    rng = np.random.Generator(np.random.PCG64(3))
    co, ci, kh, kw = 5, 3, 2, 4
    kcrs = rng.standard_normal((co, ci, kh, kw)).astype(np.float32)
    krsc = kcrs.transpose(0, 2, 3, 1)
    crsk = kcrs.transpose(1, 2, 3, 0)
    forms = {"KCRS": kcrs, "KRSC": krsc, "CRSK": crsk}
    for a in forms:
        for b in forms:
            out = ck.convert_conv_weights(forms[a], a, b)
            assert out.flags["C_CONTIGUOUS"]
            assert np.array_equal(out, forms[b]), (a, b)


@pytest.mark.parametrize("layout,fmt", [("NHWC", PYDTNN_TENSOR_FORMAT_NHWC), ("NCHW", PYDTNN_TENSOR_FORMAT_NCHW)])
def test_reference_files_hold_the_layouts_the_module_assumes(layout, fmt):
    d = np.load(os.path.join(GOLD, f"ref_checkpoint_{layout}.npz"))
    # Conv2D(8 filters, 3x3) on 3 channels, then Conv2D(8, 3x3) on 8 channels
    want = {"CRSK": (3, 3, 3, 8), "KCRS": (8, 3, 3, 3)}[ck.reference_cpu_layout(fmt)]
    assert d["1_Conv2D_weights"].shape == want
    assert d["5_Conv2D_weights"].shape == ((8, 3, 3, 8) if layout == "NHWC" else (8, 8, 3, 3))
    assert d["10_FC_weights"].shape == (128, 5)
    for k in ("gamma", "beta", "running_mean", "running_var"):
        assert d[f"2_BatchNormalization_{k}"].shape == (8,)
    assert ck.LAYOUT_KEY not in d


class _Ary:
    def __init__(self, a):
        self.a = a

    shape = property(lambda s: s.a.shape)
    size = property(lambda s: s.a.size)
    dtype = property(lambda s: s.a.dtype)

    def get(self):
        return self.a.copy()

    def set(self, h):
        self.a[...] = h


class _T:
    def __init__(self, a):
        self.ary = _Ary(a)


class _Layer:
    paths = []

    def __init__(self, lid, name, **tensors):
        self.id, self.canonical_name = lid, name
        self.grad_vars = {k: "d" + k for k in tensors if not k.startswith("running")}
        for k, v in tensors.items():
            setattr(self, k, _T(v))


class _Block(_Layer):
    def __init__(self, lid, paths):
        self.id, self.canonical_name, self.grad_vars, self.paths = lid, "AdditionBlock", {}, paths


class _Model:
    rank = 0

    def __init__(self, fmt, seed):
        rng = np.random.Generator(np.random.PCG64(seed))
        r = lambda *s: rng.standard_normal(s).astype(np.float32)
        wshape = (4, 3, 3, 2) if fmt == PYDTNN_TENSOR_FORMAT_NHWC else (4, 2, 3, 3)
        self.tensor_format = fmt
        self.layers = [_Layer(0, "Input"), _Layer(1, "Conv2D", weights=r(*wshape), biases=r(1, 1, 1, 4)),
                       _Block(2, [[_Layer(3, "BatchNormalization", gamma=r(4), beta=r(4), running_mean=r(4), running_var=r(4))], []]),
                       _Layer(4, "FC", weights=r(16, 3), biases=r(3))]


@pytest.mark.parametrize("fmt", [PYDTNN_TENSOR_FORMAT_NHWC, PYDTNN_TENSOR_FORMAT_NCHW])
@pytest.mark.parametrize("layout", ["cpu", "gpu"])
def test_state_dict_round_trip_and_key_names(fmt, layout, tmp_path):
    a, b = _Model(fmt, 1), _Model(fmt, 2)
    d = ck.state_dict(a, layout)
    assert set(d) == {"1_Conv2D_weights", "1_Conv2D_biases", "3_BatchNormalization_gamma", "3_BatchNormalization_beta",
                      "3_BatchNormalization_running_mean", "3_BatchNormalization_running_var", "4_FC_weights",
                      "4_FC_biases", ck.LAYOUT_KEY}
    assert d["1_Conv2D_biases"].shape == (4,)
    if fmt == PYDTNN_TENSOR_FORMAT_NHWC:
        assert d["1_Conv2D_weights"].shape == ((2, 3, 3, 4) if layout == "cpu" else (4, 3, 3, 2))
    path = os.path.join(tmp_path, "ck.npz")
    ck.store_weights_and_bias(a, path, layout)
    assert ck.load_weights_and_bias(b, path) == []
    for la, lb in zip(ck._walk(a.layers), ck._walk(b.layers)):
        for k in ck._keys(la):
            assert np.array_equal(getattr(la, k).ary.a, getattr(lb, k).ary.a), (la.id, k)


def test_a_file_without_the_layout_key_is_read_as_reference_cpu_and_bad_shapes_are_refused():
    a, b = _Model(PYDTNN_TENSOR_FORMAT_NHWC, 1), _Model(PYDTNN_TENSOR_FORMAT_NHWC, 2)
    d = ck.state_dict(a, "cpu")
    del d[ck.LAYOUT_KEY]
    del d["4_FC_biases"]
    assert ck.load_state_dict(b, d) == ["4_FC_biases"]
    assert np.array_equal(a.layers[1].weights.ary.a, b.layers[1].weights.ary.a)
    with pytest.raises(ValueError):
        ck.load_state_dict(b, d, layout="KCRS")
