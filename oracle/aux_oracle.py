"""CPU checker for the layers either side of the convolution in a training step --
TEST INFRASTRUCTURE ONLY (see conv_oracle.py for the rules on who may import this).

NumPy restatements of the reference's CPU batch normalisation, ReLU, pooling, softmax,
categorical cross-entropy, accuracy and SGD, each citing the reference lines it follows.
Parity status: pinned against ``tests/golden/aux_ref.npz`` (outputs of the reference classes).
All functions take ``layout`` "NHWC" or "NCHW" where a channel axis matters.
"""
from __future__ import annotations

import numpy as np

NHWC, NCHW = "NHWC", "NCHW"


def _caxis(layout):
    return 3 if layout == NHWC else 1


def _to_rows(x, layout):
    """(N,H,W,C) or (N,C,H,W) -> (N*H*W, C), channels last (batch_normalization_cpu.py:54-57)."""
    if x.ndim == 2:
        return x
    if layout == NCHW:
        x = x.transpose(0, 2, 3, 1)
    return np.ascontiguousarray(x).reshape(-1, x.shape[-1])


def _from_rows(r, like_shape, layout):
    if len(like_shape) == 2:
        return r
    if layout == NCHW:
        n, c, h, w = like_shape
        return np.ascontiguousarray(r.reshape(n, h, w, c).transpose(0, 3, 1, 2))
    return r.reshape(like_shape)


def bn_train_forward(x, gamma, beta, running_mean, running_var, momentum=0.9, eps=1e-5, layout=NHWC):
    """Training-mode batch norm: batch mean and biased variance over N*H*W, then the running
    averages (pydtnn/backends/cpu/layers/batch_normalization_cpu.py:59-76).
    Returns y, cache(std, xn), new_running_mean, new_running_var."""
    r = _to_rows(x, layout)
    mu = np.mean(r, axis=0)
    xc = r - mu
    var = np.mean(xc ** 2, axis=0)
    std = np.sqrt(var + eps)
    xn = xc / std
    y = gamma * xn + beta
    rm = momentum * running_mean + (1.0 - momentum) * mu
    rv = momentum * running_var + (1.0 - momentum) * var
    return _from_rows(y.astype(x.dtype), x.shape, layout), (std, xn), rm.astype(x.dtype), rv.astype(x.dtype)


def bn_train_backward(dy, cache, gamma, layout=NHWC, need_dx=True):
    """dgamma, dbeta, dx (batch_normalization_cpu.py:108-129 and
    pydtnn/cython_modules/bn_training_cython.pyx:224-227)."""
    std, xn = cache
    r = _to_rows(dy, layout)
    n = r.shape[0]
    dgamma = np.sum(r * xn, axis=0)
    dbeta = np.sum(r, axis=0)
    dx = None
    if need_dx:
        dxr = (gamma / (std * n)) * (n * r - xn * dgamma - dbeta)
        dx = _from_rows(dxr.astype(dy.dtype), dy.shape, layout)
    return dgamma, dbeta, dx


def bn_inference(x, running_mean, inv_std, gamma, beta, layout=NHWC):
    """((x-mean)*inv_std)*gamma+beta (pydtnn/cython_modules/bn_inference_cython.pyx:71-72)."""
    r = _to_rows(x, layout)
    y = ((r - running_mean) * inv_std) * gamma + beta
    return _from_rows(y.astype(x.dtype), x.shape, layout)


def relu_forward(x):
    """y = max(x,0), mask = x>0 (pydtnn/cython_modules/relu_cython.pyx:53-60)."""
    mask = x > 0
    return np.where(mask, x, x.dtype.type(0)), mask


def relu_backward(dy, mask):
    """pydtnn/backends/cpu/activations/relu_cpu.py:38-40."""
    return dy * mask


def _pool_geometry(h, w, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil):
    ho = (h + 2 * vpad - vdil * (kh - 1) - 1) // vstr + 1
    wo = (w + 2 * hpad - hdil * (kw - 1) - 1) // hstr + 1
    return ho, wo


def _as_nhwc(x, layout):
    return x if layout == NHWC else np.ascontiguousarray(x.transpose(0, 2, 3, 1))


def _as_layout(x_nhwc, layout):
    return x_nhwc if layout == NHWC else np.ascontiguousarray(x_nhwc.transpose(0, 3, 1, 2))


def max_pool_forward(x, kh, kw, vpad, hpad, vstr, hstr, vdil=1, hdil=1, layout=NHWC):
    """Max over the in-bounds taps only; the first maximum wins; idx = ii*kw + jj
    (pydtnn/cython_modules/max_pool_2d_nhwc_cython.pyx:96-113). Returns y, idx_max (int32)."""
    xh = _as_nhwc(x, layout)
    n, h, w, c = xh.shape
    ho, wo = _pool_geometry(h, w, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil)
    y = np.full((n, ho, wo, c), np.finfo(x.dtype).min, x.dtype)
    idx = np.zeros((n, ho, wo, c), np.int32)
    for ii in range(kh):
        for jj in range(kw):
            for xx in range(ho):
                x_x = vstr * xx + vdil * ii - vpad
                if not (0 <= x_x < h):
                    continue
                for yy in range(wo):
                    x_y = hstr * yy + hdil * jj - hpad
                    if not (0 <= x_y < w):
                        continue
                    val = xh[:, x_x, x_y, :]
                    better = val > y[:, xx, yy, :]
                    y[:, xx, yy, :] = np.where(better, val, y[:, xx, yy, :])
                    idx[:, xx, yy, :] = np.where(better, ii * kw + jj, idx[:, xx, yy, :])
    return _as_layout(y, layout), _as_layout(idx, layout)


def max_pool_backward(dy, idx_max, x_shape, kh, kw, vpad, hpad, vstr, hstr, vdil=1, hdil=1, layout=NHWC):
    """Route dy to the recorded tap (max_pool_2d_nhwc_cython.pyx:203-212; the reference
    decodes the tap as (idx // kh, idx % kw), identical to (idx // kw, idx % kw) for the
    square windows every shipped model uses)."""
    dyh, idh = _as_nhwc(dy, layout), _as_nhwc(idx_max, layout)
    if layout == NCHW:
        n, c, h, w = x_shape
    else:
        n, h, w, c = x_shape
    dx = np.zeros((n, h, w, c), dy.dtype)
    _, ho, wo, _ = dyh.shape
    for xx in range(ho):
        for yy in range(wo):
            ii, jj = idh[:, xx, yy, :] // kh, idh[:, xx, yy, :] % kw
            x_x = vstr * xx + vdil * ii - vpad
            x_y = hstr * yy + hdil * jj - hpad
            ok = (x_x >= 0) & (x_x < h) & (x_y >= 0) & (x_y < w)
            nn, cc = np.nonzero(ok)
            np.add.at(dx, (nn, x_x[nn, cc], x_y[nn, cc], cc), dyh[nn, xx, yy, cc])
    return _as_layout(dx, layout)


def avg_pool_forward(x, kh, kw, vpad, hpad, vstr, hstr, vdil=1, hdil=1, layout=NHWC):
    """Mean over the in-bounds taps, divisor = number of in-bounds taps
    (pydtnn/cython_modules/average_pool_2d_nhwc_cython.pyx:93-111)."""
    xh = _as_nhwc(x, layout)
    n, h, w, c = xh.shape
    ho, wo = _pool_geometry(h, w, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil)
    acc = np.zeros((n, ho, wo, c), x.dtype)
    items = np.zeros((ho, wo), np.int64)
    for ii in range(kh):
        for jj in range(kw):
            for xx in range(ho):
                x_x = vstr * xx + vdil * ii - vpad
                if not (0 <= x_x < h):
                    continue
                for yy in range(wo):
                    x_y = hstr * yy + hdil * jj - hpad
                    if 0 <= x_y < w:
                        acc[:, xx, yy, :] = acc[:, xx, yy, :] + xh[:, x_x, x_y, :]
                        items[xx, yy] += 1
    y = acc / items[None, :, :, None].astype(x.dtype)
    return _as_layout(y.astype(x.dtype), layout)


def avg_pool_backward(dy, x_shape, kh, kw, vpad, hpad, vstr, hstr, vdil=1, hdil=1, layout=NHWC):
    """Spread dy/items over the in-bounds taps (average_pool_2d_nhwc_cython.pyx:207-227)."""
    dyh = _as_nhwc(dy, layout)
    if layout == NCHW:
        n, c, h, w = x_shape
    else:
        n, h, w, c = x_shape
    _, ho, wo, _ = dyh.shape
    dx = np.zeros((n, h, w, c), dy.dtype)
    for xx in range(ho):
        for yy in range(wo):
            taps = [(vstr * xx + vdil * ii - vpad, hstr * yy + hdil * jj - hpad)
                    for ii in range(kh) for jj in range(kw)]
            taps = [(a, b) for a, b in taps if 0 <= a < h and 0 <= b < w]
            avg = dyh[:, xx, yy, :] / dy.dtype.type(len(taps))
            for a, b in taps:
                dx[:, a, b, :] += avg
    return _as_layout(dx, layout)


def softmax_forward(x):
    """pydtnn/backends/cpu/activations/softmax_cpu.py:32-35."""
    y = np.exp(x - np.max(x, axis=1, keepdims=True))
    y /= np.sum(y, axis=1, keepdims=True)
    return y


def softmax_backward(dy, y):
    """pydtnn/backends/cpu/activations/softmax_cpu.py:37-39."""
    return y * (dy - (dy * y).sum(axis=1, keepdims=True))


def categorical_cross_entropy(y_pred, y_targ, global_batch_size, eps=1e-8):
    """loss (mean over the local batch) and d(loss)/d(y_pred) already divided by the GLOBAL
    batch (pydtnn/backends/cpu/losses/categorical_cross_entropy_cpu.py:27-35)."""
    y_pred = np.clip(y_pred, a_min=eps, a_max=(1 - eps))
    b_range = np.arange(y_pred.shape[0])
    amax = np.argmax(y_targ, axis=1)
    loss = -np.sum(np.log(y_pred[b_range, amax])) / y_pred.shape[0]
    dx = np.copy(y_targ)
    dx[b_range, amax] /= (-y_pred[b_range, amax] * global_batch_size)
    return loss, dx


def categorical_accuracy(y_pred, y_targ):
    """Percent of rows whose arg-max hits the label
    (pydtnn/backends/cpu/metrics/categorical_accuracy_cpu.py:27-29)."""
    b = y_targ.shape[0]
    return np.sum(y_targ[np.arange(b), np.argmax(y_pred, axis=1)]) * 100 / b


def sgd_update(w, dw, velocity, lr, momentum=0.9, nesterov=False, decay=0.0):
    """v = m*v + dw ; w -= lr*(decay*w + v)  (Nesterov: w -= lr*(decay*w + dw + m*v))
    (pydtnn/backends/cpu/optimizers/sgd_cpu.py:28-41). Returns new (w, velocity)."""
    velocity = momentum * velocity + dw
    if nesterov:
        w = w - lr * (decay * w + dw + momentum * velocity)
    else:
        w = w - lr * (decay * w + velocity)
    return w.astype(dw.dtype), velocity.astype(dw.dtype)
