"""The CPU checker against the golden vectors produced by the reference itself (CPU only)."""
import os

import numpy as np
import pytest

from oracle import aux_oracle as ao
from oracle import conv_oracle as co

GOLD = os.path.join(os.path.dirname(__file__), "golden")
BACKENDS = ["numpy"] + (["c"] if co.c_lib() is not None else []) + \
           (["ref"] if "im2row_nhwc_cython" in co.ref_kernels() else [])


def _geom(arr, n_override=None):
    n, h, w, ci, cout, kh, kw, vp, hp, vs, hs, vd, hd = [int(v) for v in arr]
    return co.Geom(n, h, w, ci, cout, kh, kw, vp, hp, vs, hs, vd, hd)


@pytest.fixture(scope="module")
def conv_ref():
    return np.load(os.path.join(GOLD, "conv_ref.npz"))


def _tol(dtype):
    # the reference's own unit tests compare with np.allclose defaults for float32
    # (pydtnn/tests/conv2d_conv_gemm.py:181-183); float64 must agree to 1e-12
    return dict(rtol=1e-5, atol=1e-6) if np.dtype(dtype) == np.float32 else dict(rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_conv_against_reference_outputs(conv_ref, backend, layout, dtype):
    ncases = len({k.split("_")[0] for k in conv_ref.files})
    assert ncases == 8
    for i in range(ncases):
        key = f"c{i}_{layout}_{dtype}"
        g = _geom(conv_ref[key + "_geom"])
        x, w, b, dy = (conv_ref[f"{key}_{n}"] for n in ("x", "w", "b", "dy"))
        keep = {}
        y = co.conv2d_forward(x, w, b, g, layout, backend, keep)
        dw, db, dx = co.conv2d_backward(x, dy, w, g, layout, True, True, backend, keep)
        t = _tol(dtype)
        np.testing.assert_allclose(y, conv_ref[key + "_y"], **t)
        np.testing.assert_allclose(dw, conv_ref[key + "_dw"], **t)
        np.testing.assert_allclose(db, conv_ref[key + "_db"], **t)
        np.testing.assert_allclose(dx, conv_ref[key + "_dx"], **t)
        assert y.dtype == np.dtype(dtype) and dx.shape == x.shape


@pytest.mark.parametrize("backend", BACKENDS)
def test_known_answer_cases_are_exact(backend):
    """Hand-made power-of-two tensors with all-ones filters: every result is exactly
    representable, so equality is bitwise."""
    ka = np.load(os.path.join(GOLD, "conv_known_answer.npz"))
    for i in range(int(ka["count"])):
        x, w = ka[f"k{i}_x"], ka[f"k{i}_w"]
        vs, hs = [int(v) for v in ka[f"k{i}_stride"]]
        g = co.Geom(x.shape[0], x.shape[2], x.shape[3], x.shape[1], w.shape[0], w.shape[2], w.shape[3],
                    0, 0, vs, hs, 1, 1)
        y = co.conv2d_forward(x, w, np.zeros(1, np.float32), g, "NCHW", backend)
        assert np.array_equal(y, ka[f"k{i}_y"])
        dw, _, dx = co.conv2d_backward(x, np.ones_like(y), w, g, "NCHW", True, True, backend)
        assert np.array_equal(dw, ka[f"k{i}_dw"])
        assert np.array_equal(dx, ka[f"k{i}_dx"])


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_index_maps_agree_bitwise_across_backends(conv_ref, layout):
    for i in range(8):
        g = _geom(conv_ref[f"c{i}_{layout}_float32_geom"])
        m_np = co.index_map_nhwc(g) if layout == "NHWC" else co.index_map_nchw(g)
        if co.c_lib() is not None:
            assert np.array_equal(m_np, co.index_map_c(g, layout))
        # the map reproduces the reference's own lowering exactly (gather is a permutation + zeros)
        x = conv_ref[f"c{i}_{layout}_float32_x"]
        gathered = np.where(m_np >= 0, x.reshape(-1)[np.maximum(m_np, 0)], np.float32(0))
        for backend in BACKENDS[1:]:
            low = co.im2row_nhwc(x, g, backend) if layout == "NHWC" else co.im2col_nchw(x, g, backend)
            assert np.array_equal(gathered, low)


def test_fc_against_reference_outputs():
    ref = np.load(os.path.join(GOLD, "fc_ref.npz"))
    for i in range(3):
        for dtype in ("float32", "float64"):
            key = f"f{i}_{dtype}"
            x, w, b, dy = (ref[f"{key}_{n}"] for n in ("x", "w", "b", "dy"))
            t = _tol(dtype)
            np.testing.assert_allclose(co.fc_forward(x, w, b), ref[key + "_y"], **t)
            dw, db, dx = co.fc_backward(x, dy, w)
            np.testing.assert_allclose(dw, ref[key + "_dw"], **t)
            np.testing.assert_allclose(db, ref[key + "_db"], **t)
            np.testing.assert_allclose(dx, ref[key + "_dx"], **t)


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_aux_layers_against_reference_outputs(layout, dtype):
    ref = np.load(os.path.join(GOLD, "aux_ref.npz"))
    tag = f"{layout}_{dtype}"
    t = dict(rtol=2e-5, atol=2e-6) if dtype == "float32" else dict(rtol=1e-11, atol=1e-12)
    x, dy = ref[f"bn_{tag}_x"], ref[f"bn_{tag}_dy"]
    gamma, beta = ref[f"bn_{tag}_gamma"], ref[f"bn_{tag}_beta"]
    c = gamma.shape[0]
    zeros = np.zeros(c, x.dtype)
    y, cache, rm, rv = ao.bn_train_forward(x, gamma, beta, zeros, zeros, 0.9, 1e-5, layout)
    np.testing.assert_allclose(y, ref[f"bn_{tag}_y"], **t)
    np.testing.assert_allclose(rm, ref[f"bn_{tag}_running_mean"], **t)
    np.testing.assert_allclose(rv, ref[f"bn_{tag}_running_var"], **t)
    dgamma, dbeta, dx = ao.bn_train_backward(dy, cache, gamma, layout)
    np.testing.assert_allclose(dgamma, ref[f"bn_{tag}_dgamma"], **t)
    np.testing.assert_allclose(dbeta, ref[f"bn_{tag}_dbeta"], **t)
    np.testing.assert_allclose(dx, ref[f"bn_{tag}_dx"], **t)
    inv_std = (1.0 / np.sqrt(rv + 1e-5)).astype(x.dtype)
    if layout == "NHWC":
        np.testing.assert_allclose(inv_std, ref[f"bn_{tag}_inv_std"], **t)
    else:
        # In NCHW evaluation the reference returns before it refreshes inv_std from the
        # running variance (pydtnn/backends/cpu/layers/batch_normalization_cpu.py:50-52 vs
        # :90-92), so its output uses the stale initial value; the formula is checked with
        # the value it actually used.
        inv_std = ref[f"bn_{tag}_inv_std"]
    np.testing.assert_allclose(ao.bn_inference(x, rm, inv_std, gamma, beta, layout), ref[f"bn_{tag}_y_eval"], **t)
    ry, mask = ao.relu_forward(x)
    assert np.array_equal(ry, ref[f"relu_{tag}_y"])
    assert np.array_equal(ao.relu_backward(dy, mask), ref[f"relu_{tag}_dx"])
    for pname, kind, args in (("mp3", "max", (3, 3, 1, 1, 2, 2)), ("mp2", "max", (2, 2, 0, 0, 2, 2)),
                              ("ap3", "avg", (3, 3, 1, 1, 2, 2)), ("gap", "avg", (6, 6, 0, 0, 1, 1))):
        pdy = ref[f"{pname}_{tag}_dy"]
        if kind == "max":
            py, idx = ao.max_pool_forward(x, *args, layout=layout)
            pdx = ao.max_pool_backward(pdy, idx, x.shape, *args, layout=layout)
        else:
            py = ao.avg_pool_forward(x, *args, layout=layout)
            pdx = ao.avg_pool_backward(pdy, x.shape, *args, layout=layout)
        np.testing.assert_allclose(py, ref[f"{pname}_{tag}_y"], **t)
        np.testing.assert_allclose(pdx, ref[f"{pname}_{tag}_dx"], **t)


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_softmax_loss_sgd_against_reference_outputs(dtype):
    ref = np.load(os.path.join(GOLD, "aux_ref.npz"))
    t = dict(rtol=2e-5, atol=1e-7) if dtype == "float32" else dict(rtol=1e-12, atol=1e-14)
    logits, labels = ref[f"sm_{dtype}_logits"], ref[f"sm_{dtype}_labels"]
    b, ncls = logits.shape
    y_targ = np.zeros((b, ncls), logits.dtype)
    y_targ[np.arange(b), labels] = 1
    probs = ao.softmax_forward(logits)
    np.testing.assert_allclose(probs, ref[f"sm_{dtype}_probs"], **t)
    loss, dprobs = ao.categorical_cross_entropy(probs, y_targ, 2 * b)
    np.testing.assert_allclose(loss, ref[f"sm_{dtype}_loss"], **t)
    np.testing.assert_allclose(dprobs, ref[f"sm_{dtype}_dprobs"], **t)
    np.testing.assert_allclose(ao.softmax_backward(dprobs, probs), ref[f"sm_{dtype}_dlogits"], **t)
    np.testing.assert_allclose(ao.categorical_accuracy(probs, y_targ), ref[f"sm_{dtype}_acc"])
    w = ref[f"sgd_{dtype}_w0"]
    v = np.zeros_like(w)
    for step in range(2):
        w, v = ao.sgd_update(w, ref[f"sgd_{dtype}_dw{step}"], v, 0.01, 0.9, False, 1e-4)
        np.testing.assert_allclose(w, ref[f"sgd_{dtype}_w{step + 1}"], **t)


def test_geometry_formula_matches_reference_definition():
    g = co.Geom(64, 32, 32, 64, 64, 3, 3, 1, 1, 1, 1, 1, 1)
    assert (g.ho, g.wo, g.m, g.k) == (32, 32, 65536, 576)
    assert g.flops == 2 * 65536 * 576 * 64
    g = co.Geom(1, 224, 224, 3, 64, 7, 7, 3, 3, 2, 2, 1, 1)
    assert (g.ho, g.wo) == (112, 112)
