"""Parity of the layers either side of the convolution (batch norm, ReLU, pooling, softmax,
cross-entropy, SGD, residual sum) with the reference's golden vectors and the CPU oracle. GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import aux_oracle as ao
from pydtnn_b200 import _lib
from tests.gpu_util import DEV, assert_parity, dev, stream

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _lay(layout):
    return _lib.LAYOUT_NHWC if layout == "NHWC" else _lib.LAYOUT_NCHW


def _nchw_dims(x, layout):
    if layout == "NHWC":
        n, h, w, c = x.shape
    else:
        n, c, h, w = x.shape
    return n, h, w, c


def _bn_train(x, dy, gamma, beta, layout, fuse_relu=False, mask_from="both"):
    L = _lib.lib()
    dt = _lib.dtype_code(x.dtype)
    n, h, w, c = _nchw_dims(x, layout)
    xd, dyd, gd, bd = dev(x), dev(dy), dev(gamma), dev(beta)
    rm, rv = torch.zeros(c, dtype=xd.dtype, device=DEV), torch.zeros(c, dtype=xd.dtype, device=DEV)
    y, dx = torch.empty_like(xd), torch.empty_like(xd)
    sm, si = torch.empty_like(rm), torch.empty_like(rm)
    dg, db = torch.empty_like(rm), torch.empty_like(rm)
    scratch = torch.empty(64 * 2 * c, dtype=torch.float64, device=DEV)
    _lib.check(L.b2c_bn_train_forward(dt, _lay(layout), n, c, h * w, xd.data_ptr(), gd.data_ptr(), bd.data_ptr(),
                                      rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, int(fuse_relu), y.data_ptr(),
                                      sm.data_ptr(), si.data_ptr(), scratch.data_ptr(), scratch.numel() * 8, stream()))
    _lib.check(L.b2c_bn_train_backward(dt, _lay(layout), n, c, h * w, xd.data_ptr(), dyd.data_ptr(),
                                       y.data_ptr() if fuse_relu and mask_from in ("both", "y") else None,
                                       bd.data_ptr() if fuse_relu and mask_from in ("both", "beta") else None,
                                       gd.data_ptr(), sm.data_ptr(),
                                       si.data_ptr(), dg.data_ptr(), db.data_ptr(), dx.data_ptr(),
                                       scratch.data_ptr(), scratch.numel() * 8, stream()))
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (y, rm, rv, dg, db, dx)]


def _assert_close(got, ref, dtype, what):
    tol = dict(rtol=3e-5, atol=3e-6) if np.dtype(dtype) == np.float32 else dict(rtol=1e-10, atol=1e-11)
    np.testing.assert_allclose(got, ref, err_msg=what, **tol)


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_batch_norm_relu_pool_golden(layout, dtype):
    ref = np.load(os.path.join(GOLD, "aux_ref.npz"))
    L = _lib.lib()
    tag = f"{layout}_{dtype}"
    x, dy = ref[f"bn_{tag}_x"], ref[f"bn_{tag}_dy"]
    gamma, beta = ref[f"bn_{tag}_gamma"], ref[f"bn_{tag}_beta"]
    y, rm, rv, dg, db, dx = _bn_train(x, dy, gamma, beta, layout)
    for name, got in (("y", y), ("running_mean", rm), ("running_var", rv), ("dgamma", dg), ("dbeta", db), ("dx", dx)):
        _assert_close(got, ref[f"bn_{tag}_{name}"], dtype, f"bn {name}")
    dt = _lib.dtype_code(dtype)
    n, h, w, c = _nchw_dims(x, layout)
    # inference with the statistics the reference used
    inv_std = ref[f"bn_{tag}_inv_std"]
    xd = dev(x)
    yd = torch.empty_like(xd)
    vecs = [dev(v) for v in (ref[f"bn_{tag}_running_mean"], inv_std, gamma, beta)]
    _lib.check(L.b2c_bn_inference(dt, _lay(layout), n, c, h * w, xd.data_ptr(), *[v.data_ptr() for v in vecs], 0,
                                  yd.data_ptr(), stream()))
    _assert_close(yd.cpu().numpy(), ref[f"bn_{tag}_y_eval"], dtype, "bn eval")
    # ReLU
    ry, rdx = torch.empty_like(xd), torch.empty_like(xd)
    dyd = dev(dy)
    _lib.check(L.b2c_relu_forward(dt, xd.numel(), xd.data_ptr(), ry.data_ptr(), stream()))
    _lib.check(L.b2c_relu_backward(dt, xd.numel(), dyd.data_ptr(), ry.data_ptr(), rdx.data_ptr(), stream()))
    assert np.array_equal(ry.cpu().numpy(), ref[f"relu_{tag}_y"])
    assert np.array_equal(rdx.cpu().numpy(), ref[f"relu_{tag}_dx"])
    # pooling
    for pname, is_max, args in (("mp3", 1, (3, 3, 1, 1, 2, 2, 1, 1)), ("mp2", 1, (2, 2, 0, 0, 2, 2, 1, 1)),
                                ("ap3", 0, (3, 3, 1, 1, 2, 2, 1, 1)), ("gap", 0, (h, w, 0, 0, 1, 1, 1, 1))):
        py_ref, pdy, pdx_ref = ref[f"{pname}_{tag}_y"], ref[f"{pname}_{tag}_dy"], ref[f"{pname}_{tag}_dx"]
        py = torch.empty(py_ref.shape, dtype=xd.dtype, device=DEV)
        idx = torch.empty(py_ref.shape, dtype=torch.int32, device=DEV)
        pdx = torch.empty_like(xd)
        pdyd = dev(pdy)
        _lib.check(L.b2c_pool_forward(dt, _lay(layout), is_max, n, h, w, c, *args, xd.data_ptr(), py.data_ptr(),
                                      idx.data_ptr(), stream()))
        _lib.check(L.b2c_pool_backward(dt, _lay(layout), is_max, n, h, w, c, *args, pdyd.data_ptr(), idx.data_ptr(),
                                       pdx.data_ptr(), stream()))
        _assert_close(py.cpu().numpy(), py_ref, dtype, pname + " y")
        _assert_close(pdx.cpu().numpy(), pdx_ref, dtype, pname + " dx")


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_batch_norm_at_resnet_sizes_and_fused_relu(layout):
    rng = np.random.Generator(np.random.PCG64(11))
    n, h, w, c = 8, 28, 28, 128
    shape = (n, h, w, c) if layout == "NHWC" else (n, c, h, w)
    x = (rng.standard_normal(shape) * 1.5 + 0.3).astype(np.float32)
    dy = rng.standard_normal(shape).astype(np.float32)
    gamma, beta = rng.standard_normal(c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
    z = np.zeros(c, np.float32)
    y_ref, cache, rm_ref, rv_ref = ao.bn_train_forward(x.astype(np.float64), gamma, beta, z, z, 0.9, 1e-5, layout)
    dg_ref, db_ref, dx_ref = ao.bn_train_backward(dy.astype(np.float64), cache, gamma, layout)
    y, rm, rv, dg, db, dx = _bn_train(x, dy, gamma, beta, layout)
    for nm, got, want in (("y", y, y_ref), ("rm", rm, rm_ref), ("rv", rv, rv_ref), ("dgamma", dg, dg_ref),
                          ("dbeta", db, db_ref), ("dx", dx, dx_ref)):
        assert_parity(got, want, np.float32, f"bn {layout} {nm}")
    # BN with the ReLU folded in == BN followed by ReLU, forward and backward
    ry_ref, mask = ao.relu_forward(y_ref)
    dg2, db2, dx2 = ao.bn_train_backward(ao.relu_backward(dy.astype(np.float64), mask), cache, gamma, layout)
    y, _, _, dg, db, dx = _bn_train(x, dy, gamma, beta, layout, fuse_relu=True)
    for nm, got, want in (("y", y, ry_ref), ("dgamma", dg, dg2), ("dbeta", db, db2), ("dx", dx, dx2)):
        assert_parity(got, want, np.float32, f"bn+relu {layout} {nm}")
    if layout == "NHWC":
        # the ReLU mask recomputed from x (beta given) is the mask read from y, bit for bit
        a = _bn_train(x, dy, gamma, beta, layout, fuse_relu=True, mask_from="y")
        b = _bn_train(x, dy, gamma, beta, layout, fuse_relu=True, mask_from="beta")
        for nm, u, v in zip(("y", "rm", "rv", "dgamma", "dbeta", "dx"), a, b):
            assert np.array_equal(u, v), f"mask from y vs from beta: {nm}"


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_softmax_cross_entropy_accuracy_sgd(dtype):
    ref = np.load(os.path.join(GOLD, "aux_ref.npz"))
    L = _lib.lib()
    dt = _lib.dtype_code(dtype)
    logits, labels = ref[f"sm_{dtype}_logits"], ref[f"sm_{dtype}_labels"]
    b, ncls = logits.shape
    xd = dev(logits)
    probs, dprobs, dlogits = torch.empty_like(xd), torch.empty_like(xd), torch.empty_like(xd)
    row_loss = torch.empty(b, dtype=xd.dtype, device=DEV)
    hit = torch.empty(b, dtype=torch.int32, device=DEV)
    lab = dev(labels.astype(np.int32))
    _lib.check(L.b2c_softmax_forward(dt, b, ncls, xd.data_ptr(), probs.data_ptr(), stream()))
    _lib.check(L.b2c_cce_forward_backward(dt, b, ncls, probs.data_ptr(), lab.data_ptr(), 2 * b, 1e-8,
                                          row_loss.data_ptr(), hit.data_ptr(), dprobs.data_ptr(), stream()))
    _lib.check(L.b2c_softmax_backward(dt, b, ncls, dprobs.data_ptr(), probs.data_ptr(), dlogits.data_ptr(), stream()))
    torch.cuda.synchronize()
    _assert_close(probs.cpu().numpy(), ref[f"sm_{dtype}_probs"], dtype, "probs")
    _assert_close(-row_loss.cpu().numpy().sum() / b, ref[f"sm_{dtype}_loss"], dtype, "loss")
    _assert_close(dprobs.cpu().numpy(), ref[f"sm_{dtype}_dprobs"], dtype, "dprobs")
    _assert_close(dlogits.cpu().numpy(), ref[f"sm_{dtype}_dlogits"], dtype, "dlogits")
    assert abs(hit.cpu().numpy().sum() * 100.0 / b - float(ref[f"sm_{dtype}_acc"])) < 1e-4
    w = dev(ref[f"sgd_{dtype}_w0"])
    v = torch.zeros_like(w)
    for step in range(2):
        dw = dev(ref[f"sgd_{dtype}_dw{step}"])
        _lib.check(L.b2c_sgd_update(dt, w.numel(), w.data_ptr(), dw.data_ptr(), v.data_ptr(), 0.01, 0.9, 1e-4, 0, stream()))
        _assert_close(w.cpu().numpy(), ref[f"sgd_{dtype}_w{step + 1}"], dtype, f"sgd step {step}")


def test_softmax_cce_at_imagenet_width_and_residual_sum():
    L = _lib.lib()
    rng = np.random.Generator(np.random.PCG64(12))
    b, ncls = 64, 1000
    logits = (rng.standard_normal((b, ncls)) * 4).astype(np.float32)
    labels = rng.integers(0, ncls, b).astype(np.int32)
    y_targ = np.zeros((b, ncls), np.float64)
    y_targ[np.arange(b), labels] = 1
    p_ref = ao.softmax_forward(logits.astype(np.float64))
    loss_ref, dp_ref = ao.categorical_cross_entropy(p_ref, y_targ, 8 * b)
    dl_ref = ao.softmax_backward(dp_ref, p_ref)
    xd, lab = dev(logits), dev(labels)
    probs, dprobs, dlogits = torch.empty_like(xd), torch.empty_like(xd), torch.empty_like(xd)
    row_loss = torch.empty(b, device=DEV)
    hit = torch.empty(b, dtype=torch.int32, device=DEV)
    _lib.check(L.b2c_softmax_forward(0, b, ncls, xd.data_ptr(), probs.data_ptr(), stream()))
    _lib.check(L.b2c_cce_forward_backward(0, b, ncls, probs.data_ptr(), lab.data_ptr(), 8 * b, 1e-8, row_loss.data_ptr(),
                                          hit.data_ptr(), dprobs.data_ptr(), stream()))
    _lib.check(L.b2c_softmax_backward(0, b, ncls, dprobs.data_ptr(), probs.data_ptr(), dlogits.data_ptr(), stream()))
    assert_parity(probs.cpu().numpy(), p_ref, np.float32, "probs")
    assert abs(-row_loss.double().sum().item() / b - loss_ref) <= 1e-5 * abs(loss_ref)
    assert_parity(dlogits.cpu().numpy(), dl_ref, np.float32, "dlogits")
    assert hit.sum().item() == int((np.argmax(p_ref, axis=1) == labels).sum())
    a, o = rng.standard_normal(100003).astype(np.float32), rng.standard_normal(100003).astype(np.float32)
    ad, od = dev(a), dev(o)
    _lib.check(L.b2c_add_inplace(0, ad.numel(), ad.data_ptr(), od.data_ptr(), stream()))
    assert np.array_equal(ad.cpu().numpy(), a + o)
    a4, o4 = rng.standard_normal(1 << 20).astype(np.float32), rng.standard_normal(1 << 20).astype(np.float32)
    ad, od = dev(a4), dev(o4)
    _lib.check(L.b2c_add_inplace(0, ad.numel(), ad.data_ptr(), od.data_ptr(), stream()))
    assert np.array_equal(ad.cpu().numpy(), a4 + o4)


@pytest.mark.parametrize("case", [(3, 5, 55, 55, 3, 3, 0, 0, 2, 2), (2, 7, 13, 13, 3, 3, 0, 0, 2, 2), (2, 3, 90, 91, 2, 3, 1, 0, 2, 1),
                                  (1, 2, 100, 100, 3, 3, 1, 1, 2, 2)])
def test_nchw_pooling_planes_exact(case):
    """NCHW float32 pooling at AlexNet's shapes and around the limits of the shared-memory plane kernel (several
    planes per block with a ragged last block; one plane per block; a plane too large for it): values and argmax
    indices equal the oracle's exactly (max), averages to float32 rounding."""
    n, c, h, w, kh, kw, vpad, hpad, vstr, hstr = case
    rng = np.random.Generator(np.random.PCG64(h * 1000 + w))
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    L = _lib.lib()
    xd = dev(x)
    y_ref, idx_ref = ao.max_pool_forward(x, kh, kw, vpad, hpad, vstr, hstr, layout="NCHW")
    a_ref = ao.avg_pool_forward(x, kh, kw, vpad, hpad, vstr, hstr, layout="NCHW")
    a_ref = a_ref[0] if isinstance(a_ref, tuple) else a_ref
    y = torch.empty(y_ref.shape, dtype=torch.float32, device=DEV)
    idx = torch.empty(y_ref.shape, dtype=torch.int32, device=DEV)
    _lib.check(L.b2c_pool_forward(_lib.F32, _lib.LAYOUT_NCHW, 1, n, h, w, c, kh, kw, vpad, hpad, vstr, hstr, 1, 1,
                                  xd.data_ptr(), y.data_ptr(), idx.data_ptr(), stream()))
    assert np.array_equal(y.cpu().numpy(), y_ref)
    assert np.array_equal(idx.cpu().numpy(), idx_ref)
    _lib.check(L.b2c_pool_forward(_lib.F32, _lib.LAYOUT_NCHW, 0, n, h, w, c, kh, kw, vpad, hpad, vstr, hstr, 1, 1,
                                  xd.data_ptr(), y.data_ptr(), None, stream()))
    assert_parity(y.cpu().numpy(), a_ref, np.float32, "average pool NCHW")
