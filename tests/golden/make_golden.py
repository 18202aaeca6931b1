"""Generate the golden vectors in this directory by running the reference itself.

Run once, in a container where the reference checkout is mounted and ``oracle/build_oracle.py``
has compiled its Cython kernels into ``oracle/_ref``:

    python tests/golden/make_golden.py [<reference checkout>]

The script imports the reference package, stands up its own CPU layer classes
(``Conv2DCPU``, ``FCCPU``, ``BatchNormalizationCPU``, pooling, ReLU, softmax, the
cross-entropy loss and the SGD optimiser) the way its unit tests do
(pydtnn/tests/conv2d_conv_gemm.py:31-64), feeds them seeded inputs and stores inputs and
outputs as small ``.npz`` files.  It also stores the hand-made known-answer cases of
``Conv2DConvGemmTestCase`` (pydtnn/tests/conv2d_conv_gemm.py:72-103, 211-314), taking the tensors
from the imported test class rather than retyping them.

Nothing at test time needs the reference: the tests only read the ``.npz`` files.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
sys.path.insert(0, os.path.join(REPO, "oracle", "_ref"))
sys.path.insert(0, REF)

from pydtnn.model import Model, TRAIN_MODE, EVALUATE_MODE  # noqa: E402
import pydtnn.backends.cpu.layers.conv_2d_cpu as conv_mod  # noqa: E402
from pydtnn.backends.cpu.layers.conv_2d_cpu import Conv2DCPU  # noqa: E402
from pydtnn.backends.cpu.layers.fc_cpu import FCCPU  # noqa: E402
import pydtnn.backends.cpu.layers.batch_normalization_cpu as bn_mod  # noqa: E402
from pydtnn.backends.cpu.layers.batch_normalization_cpu import BatchNormalizationCPU  # noqa: E402
from pydtnn.backends.cpu.layers.max_pool_2d_cpu import MaxPool2DCPU  # noqa: E402
from pydtnn.backends.cpu.layers.average_pool_2d_cpu import AveragePool2DCPU  # noqa: E402
from pydtnn.backends.cpu.activations.relu_cpu import ReluCPU  # noqa: E402
from pydtnn.backends.cpu.activations.softmax_cpu import SoftmaxCPU  # noqa: E402
from pydtnn.backends.cpu.losses.categorical_cross_entropy_cpu import CategoricalCrossEntropyCPU  # noqa: E402
from pydtnn.backends.cpu.metrics.categorical_accuracy_cpu import CategoricalAccuracyCPU  # noqa: E402
from pydtnn.backends.cpu.optimizers.sgd_cpu import SGDCPU  # noqa: E402


class P:
    pass


def make_model(batch, layout, dtype, mode=TRAIN_MODE):
    p = P()
    p.batch_size = batch
    p.enable_conv_gemm = False
    p.enable_best_of = False
    p.tensor_format = layout
    m = Model(dtype=dtype, **vars(p))
    m.mode = mode
    return m


def _transpose_1023_any_dtype(a):
    # The reference's 1023 transpose kernel is float32-only (transpose_cython.pyx:90-102);
    # a permutation has no arithmetic, so np.transpose stands in for float64.
    return np.ascontiguousarray(a.transpose(1, 0, 2, 3))


# (n, h, w, ci, co, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil)
CONV_CASES = [
    (2, 8, 8, 3, 4, 3, 3, 1, 1, 1, 1, 1, 1),
    (2, 9, 7, 4, 5, 3, 2, 1, 0, 2, 1, 1, 1),
    (1, 10, 10, 2, 3, 3, 3, 2, 2, 1, 1, 2, 2),
    (3, 7, 7, 8, 8, 1, 1, 0, 0, 2, 2, 1, 1),
    (2, 12, 12, 3, 6, 5, 5, 2, 2, 2, 2, 1, 1),
    (1, 11, 11, 3, 4, 7, 7, 3, 3, 2, 2, 1, 1),
    (2, 6, 6, 16, 32, 3, 3, 1, 1, 1, 1, 1, 1),
    (1, 5, 9, 2, 2, 2, 3, 0, 1, 1, 2, 1, 1),
]


def conv_goldens():
    out = {}
    for ci_, case in enumerate(CONV_CASES):
        n, h, w, ci, co, kh, kw, vp, hp, vs, hs, vd, hd = case
        for layout in ("NHWC", "NCHW"):
            for dtype in (np.float32, np.float64):
                rng = np.random.Generator(np.random.PCG64(1000 + ci_))
                model = make_model(n, layout, dtype)
                if dtype == np.float64:
                    conv_mod.best_transpose_1023 = _transpose_1023_any_dtype
                layer = Conv2DCPU(nfilters=co, filter_shape=(kh, kw), padding=(vp, hp), stride=(vs, hs),
                                  dilation=(vd, hd), use_bias=True)
                layer.set_model(model)
                layer.initialize(prev_shape=(h, w, ci) if layout == "NHWC" else (ci, h, w))
                x_nhwc = rng.standard_normal((n, h, w, ci)).astype(dtype)
                w_nhwc = (rng.standard_normal((ci, kh, kw, co)) * np.sqrt(2.0 / (ci * kh * kw))).astype(dtype)
                b = rng.standard_normal((co,)).astype(dtype)
                ho, wo = layer.ho, layer.wo
                dy_nhwc = rng.standard_normal((n, ho, wo, co)).astype(dtype)
                if layout == "NHWC":
                    x, wt, dy = x_nhwc, w_nhwc, dy_nhwc
                else:
                    x = np.ascontiguousarray(x_nhwc.transpose(0, 3, 1, 2))
                    wt = np.ascontiguousarray(w_nhwc.transpose(3, 0, 1, 2))
                    dy = np.ascontiguousarray(dy_nhwc.transpose(0, 3, 1, 2))
                layer.weights = wt.copy()
                layer.biases = b.copy()
                y = layer.forward(x)
                dx = layer.backward(dy)
                key = f"c{ci_}_{layout}_{np.dtype(dtype).name}"
                out[key + "_geom"] = np.array(case, dtype=np.int64)
                for name, arr in (("x", x), ("w", wt), ("b", b), ("dy", dy), ("y", y),
                                  ("dw", layer.dw), ("db", layer.db), ("dx", dx)):
                    out[f"{key}_{name}"] = np.ascontiguousarray(arr)
    np.savez_compressed(os.path.join(HERE, "conv_ref.npz"), **out)
    print("conv_ref.npz", len(out))


def known_answer_goldens():
    """Hand-made tensors of Conv2DConvGemmTestCase, NCHW float32, all-ones filters."""
    from pydtnn.tests.conv2d_conv_gemm import Conv2DConvGemmTestCase as T
    from pydtnn.tests.common import D
    out = {}
    combos = []
    for xname in ("x_2x4", "x_4x4", "x_4x8", "x_8x8"):
        for wname in ("w_1x1", "w_1x2", "w_2x2", "w_3x3"):
            for stride in ((1, 1), (2, 2), (3, 3), (1, 2)):
                x = getattr(T, xname)
                w = getattr(T, wname)
                if w.shape[2] > x.shape[2] or w.shape[3] > x.shape[3]:
                    continue
                combos.append((xname, wname, stride))
    for i, (xname, wname, stride) in enumerate(combos):
        x = getattr(T, xname)
        w = getattr(T, wname)
        model = make_model(1, "NCHW", np.float32)
        layer = Conv2DCPU(nfilters=1, filter_shape=w.shape[2:], padding=0, stride=stride, use_bias=True)
        layer.set_model(model)
        layer.initialize(prev_shape=x.shape[1:])
        layer.weights = w.copy()
        layer.biases = np.zeros((1,), np.float32)
        y = layer.forward(x)
        dy = np.ones_like(y)
        dx = layer.backward(dy)
        out[f"k{i}_x"] = x
        out[f"k{i}_w"] = w
        out[f"k{i}_stride"] = np.array(stride, dtype=np.int64)
        out[f"k{i}_y"] = y
        out[f"k{i}_dw"] = layer.dw
        out[f"k{i}_dx"] = dx
    out["count"] = np.array(len(combos))
    np.savez_compressed(os.path.join(HERE, "conv_known_answer.npz"), **out)
    print("conv_known_answer.npz", len(combos))


def fc_goldens():
    out = {}
    for i, (b, fin, fout) in enumerate([(4, 10, 7), (8, 33, 17), (3, 64, 10)]):
        for dtype in (np.float32, np.float64):
            rng = np.random.Generator(np.random.PCG64(2000 + i))
            model = make_model(b, "NHWC", dtype)
            layer = FCCPU(shape=(fout,), use_bias=True)
            layer.set_model(model)
            layer.initialize(prev_shape=(fin,))
            x = rng.standard_normal((b, fin)).astype(dtype)
            w = rng.standard_normal((fin, fout)).astype(dtype)
            bias = rng.standard_normal((fout,)).astype(dtype)
            dy = rng.standard_normal((b, fout)).astype(dtype)
            layer.weights, layer.biases = w.copy(), bias.copy()
            y = layer.forward(x)
            dx = layer.backward(dy)
            key = f"f{i}_{np.dtype(dtype).name}"
            for name, arr in (("x", x), ("w", w), ("b", bias), ("dy", dy), ("y", y), ("dw", layer.dw),
                              ("db", layer.db), ("dx", dx)):
                out[f"{key}_{name}"] = arr
    np.savez_compressed(os.path.join(HERE, "fc_ref.npz"), **out)
    print("fc_ref.npz", len(out))


def aux_goldens():
    """Layers either side of the convolution in a whole training step (NHWC and NCHW)."""
    out = {}
    for layout in ("NHWC", "NCHW"):
        for dtype in (np.float32, np.float64):
            tag = f"{layout}_{np.dtype(dtype).name}"
            rng = np.random.Generator(np.random.PCG64(3000))
            n, h, w, c = 4, 6, 6, 5
            shp = (h, w, c) if layout == "NHWC" else (c, h, w)
            to_l = (lambda a: a) if layout == "NHWC" else (lambda a: np.ascontiguousarray(a.transpose(0, 3, 1, 2)))
            x = to_l(rng.standard_normal((n, h, w, c)).astype(dtype) * 2 + 0.5)
            dy = to_l(rng.standard_normal((n, h, w, c)).astype(dtype))
            # batch normalisation, training mode then inference with the updated statistics
            model = make_model(n, layout, dtype)
            if dtype == np.float64:
                # same float32-only transposes as in the convolution (transpose_cython.pyx:25-88)
                bn_mod.best_transpose_0231 = lambda a: np.ascontiguousarray(a.transpose(0, 2, 3, 1))
                bn_mod.best_transpose_0312 = lambda a: np.ascontiguousarray(a.transpose(0, 3, 1, 2))
            bn = BatchNormalizationCPU()
            bn.set_model(model)
            bn.initialize(prev_shape=shp)
            bn.gamma = rng.standard_normal((c,)).astype(dtype)
            bn.beta = rng.standard_normal((c,)).astype(dtype)
            g0, b0 = bn.gamma.copy(), bn.beta.copy()
            y = bn.forward(x)
            dx = bn.backward(dy)
            out[f"bn_{tag}_x"], out[f"bn_{tag}_dy"] = x, dy
            out[f"bn_{tag}_gamma"], out[f"bn_{tag}_beta"] = g0, b0
            out[f"bn_{tag}_y"], out[f"bn_{tag}_dx"] = y, dx
            out[f"bn_{tag}_dgamma"], out[f"bn_{tag}_dbeta"] = bn.dgamma, bn.dbeta
            out[f"bn_{tag}_running_mean"], out[f"bn_{tag}_running_var"] = bn.running_mean, bn.running_var
            model.mode = EVALUATE_MODE
            out[f"bn_{tag}_y_eval"] = bn.forward(x)
            out[f"bn_{tag}_inv_std"] = bn.inv_std
            model.mode = TRAIN_MODE
            # ReLU
            rl = ReluCPU(shape=shp)
            rl.set_model(model)
            rl.initialize(prev_shape=shp)
            out[f"relu_{tag}_y"] = rl.forward(x)
            out[f"relu_{tag}_dx"] = rl.backward(dy)
            # max pool 3x3 stride 2 pad 1 and 2x2 stride 2; global average pool
            for pname, cls, kw in (("mp3", MaxPool2DCPU, dict(pool_shape=(3, 3), stride=2, padding=1)),
                                   ("mp2", MaxPool2DCPU, dict(pool_shape=(2, 2), stride=2, padding=0)),
                                   ("ap3", AveragePool2DCPU, dict(pool_shape=(3, 3), stride=2, padding=1)),
                                   ("gap", AveragePool2DCPU, dict(pool_shape=(0, 0)))):
                pl = cls(**kw)
                pl.set_model(model)
                pl.initialize(prev_shape=shp)
                py = pl.forward(x)
                pdy = rng.standard_normal(py.shape).astype(dtype)
                out[f"{pname}_{tag}_y"] = py
                out[f"{pname}_{tag}_dy"] = pdy
                out[f"{pname}_{tag}_dx"] = pl.backward(pdy)
    for dtype in (np.float32, np.float64):
        tag = np.dtype(dtype).name
        rng = np.random.Generator(np.random.PCG64(3100))
        b, ncls = 6, 11
        model = make_model(b, "NHWC", dtype)
        logits = rng.standard_normal((b, ncls)).astype(dtype) * 3
        labels = rng.integers(0, ncls, size=(b,))
        y_targ = np.zeros((b, ncls), dtype)
        y_targ[np.arange(b), labels] = 1
        sm = SoftmaxCPU(shape=(ncls,))
        sm.set_model(model)
        sm.initialize(prev_shape=(ncls,))
        probs = sm.forward(logits)
        loss_fn = CategoricalCrossEntropyCPU(shape=(b, ncls), model=model)
        loss, dprobs = loss_fn(probs, y_targ, b * 2)
        dlogits = sm.backward(dprobs)
        acc = CategoricalAccuracyCPU(shape=(b, ncls), model=model)(probs, y_targ)
        for name, arr in (("logits", logits), ("labels", labels), ("probs", probs), ("loss", np.array(loss)),
                          ("dprobs", dprobs), ("dlogits", dlogits), ("acc", np.array(acc))):
            out[f"sm_{tag}_{name}"] = arr
        # SGD with momentum, two consecutive updates of one tensor
        class L:
            pass
        lay = L()
        lay.model = model
        lay.grad_vars = {"weights": "dw"}
        lay.weights = rng.standard_normal((7, 5)).astype(dtype)
        out[f"sgd_{tag}_w0"] = lay.weights.copy()
        opt = SGDCPU(learning_rate=0.01, momentum=0.9, nesterov=False, decay=1e-4, dtype=dtype)
        for step in range(2):
            lay.dw = rng.standard_normal((7, 5)).astype(dtype)
            out[f"sgd_{tag}_dw{step}"] = lay.dw.copy()
            opt.update(lay)
            out[f"sgd_{tag}_w{step + 1}"] = lay.weights.copy()
    np.savez_compressed(os.path.join(HERE, "aux_ref.npz"), **out)
    print("aux_ref.npz", len(out))


if __name__ == "__main__":
    conv_goldens()
    known_answer_goldens()
    fc_goldens()
    aux_goldens()
