"""Convolution forward that also takes the batch sums of its output, and the batch norm that consumes them
(b2c_conv_fprop_stats + b2c_bn_train_forward_prestats), through the C ABI: the convolution output must be bit-identical
to b2c_conv_fprop, and the batch-norm results must match both the separate-pass entry point and the CPU oracle chain
conv -> training-mode batch norm (the un-fused definition, pydtnn/backends/cpu/layers/batch_normalization_cpu.py:65-76).  GPU."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import aux_oracle as ao
from oracle import conv_oracle as co
from pydtnn_b200 import _lib
from tests.gpu_util import DEV, assert_parity, dev, make_desc, stream, w_from_cpu_layout, workspace

pytestmark = pytest.mark.gpu

# (n, h, w, ci, co, k, stride, pad): tile counts below, equal to and far above the SM count, a ragged last tile,
# 64- and 128-wide column tiles, the balanced mode (14x14x256 3x3 at batch 64) and a few-channel stem
SHAPES = [(3, 10, 10, 32, 64, 3, 1, 1), (4, 16, 16, 64, 256, 1, 1, 0), (8, 28, 28, 128, 128, 3, 2, 1),
          (64, 14, 14, 256, 256, 3, 1, 1), (16, 56, 56, 64, 256, 1, 1, 0), (2, 9, 9, 32, 2048, 1, 1, 0),
          (4, 40, 40, 3, 64, 7, 2, 3),
          # sums kept per CTA over many tiles (more row tiles than SMs), a half-empty column tile, ragged rows, six column
          # tiles (a grid of 144 CTAs); the batch norm's fast path takes channel counts 4..128, 256 and multiples of 256
          (3, 91, 91, 64, 32, 1, 1, 0), (2, 29, 31, 96, 128, 1, 1, 0), (2, 40, 40, 128, 768, 1, 1, 0),
          # long K with whole tiles: the chunked drain's per-CTA sums (25 row tiles x 2 column tiles)
          (4, 28, 28, 256, 256, 3, 1, 1),
          # eight k-blocks: the streaming epilogue with four drain warps; 32 k-blocks of a 1x1 filter
          (4, 14, 14, 256, 128, 1, 1, 0), (4, 14, 14, 1024, 256, 1, 1, 0)]


def _conv_and_bn(g, x, w_krsc, b, gamma, beta, fused, relu, addend):
    L = _lib.lib()
    desc = make_desc(g, "NHWC", np.float32, "KRSC")
    ws = workspace(desc)
    xd, wd, bd, gd, bed = dev(x), dev(w_krsc), dev(b), dev(gamma), dev(beta)
    y = torch.full((g.n, g.ho, g.wo, g.co), float("nan"), device=DEV)
    out = torch.full_like(y, float("nan"))
    rm, rv = torch.full((g.co,), 0.25, device=DEV), torch.full((g.co,), 0.75, device=DEV)
    sm, si = torch.empty(g.co, device=DEV), torch.empty(g.co, device=DEV)
    ad = dev(addend) if addend is not None else None
    scratch = torch.empty(1200 * g.co, dtype=torch.float64, device=DEV)
    if fused:
        nbytes = L.b2c_conv_stats_bytes(ctypes.byref(desc))
        assert nbytes > 0
        stats = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=DEV)       # garbage: nothing may rely on zeros
        _lib.check(L.b2c_conv_fprop_stats(ctypes.byref(desc), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), y.data_ptr(),
                                          stats.data_ptr(), nbytes, ws.data_ptr(), ws.numel(), stream()))
        _lib.check(L.b2c_bn_train_forward_prestats(g.n, g.co, g.ho * g.wo, y.data_ptr(), stats.data_ptr(), nbytes, gd.data_ptr(),
                                                   bed.data_ptr(), rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, int(relu),
                                                   ad.data_ptr() if ad is not None else None, out.data_ptr(), sm.data_ptr(),
                                                   si.data_ptr(), scratch.data_ptr(), scratch.numel() * 8, stream()))
    else:
        _lib.check(L.b2c_conv_fprop(ctypes.byref(desc), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), None, 0, y.data_ptr(),
                                    ws.data_ptr(), ws.numel(), stream()))
        if ad is None:
            _lib.check(L.b2c_bn_train_forward(_lib.F32, _lib.LAYOUT_NHWC, g.n, g.co, g.ho * g.wo, y.data_ptr(), gd.data_ptr(),
                                              bed.data_ptr(), rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, int(relu), out.data_ptr(),
                                              sm.data_ptr(), si.data_ptr(), scratch.data_ptr(), scratch.numel() * 8, stream()))
        else:
            _lib.check(L.b2c_bn_train_forward_residual(_lib.F32, _lib.LAYOUT_NHWC, g.n, g.co, g.ho * g.wo, y.data_ptr(), gd.data_ptr(),
                                                       bed.data_ptr(), rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, ad.data_ptr(), int(relu),
                                                       out.data_ptr(), sm.data_ptr(), si.data_ptr(), scratch.data_ptr(),
                                                       scratch.numel() * 8, stream()))
    torch.cuda.synchronize()
    _lib.check(L.b2c_check_device_status(None))
    return [t.cpu().numpy() for t in (y, out, sm, si, rm, rv)]


@pytest.mark.parametrize("shape", SHAPES)
def test_conv_with_batch_sums_feeds_the_batch_norm(shape):
    n, h, w_, ci, cout, k, stride, pad = shape
    g = co.Geom(n, h, w_, ci, cout, k, k, pad, pad, stride, stride)
    rng = np.random.Generator(np.random.PCG64(hash(shape) & 0xFFFF))
    x = rng.standard_normal((g.n, g.h, g.w, g.ci)).astype(np.float32)
    w = (rng.standard_normal((g.ci, g.kh, g.kw, g.co)) * np.sqrt(2.0 / g.k)).astype(np.float32)
    b = rng.standard_normal((g.co,)).astype(np.float32)
    gamma, beta = rng.standard_normal(g.co).astype(np.float32), rng.standard_normal(g.co).astype(np.float32)
    w_krsc = w_from_cpu_layout(w, "NHWC", "KRSC")
    for relu, with_addend in ((False, False), (True, False), (True, True)):
        addend = rng.standard_normal((g.n, g.ho, g.wo, g.co)).astype(np.float32) if with_addend else None
        got = _conv_and_bn(g, x, w_krsc, b, gamma, beta, True, relu, addend)
        want = _conv_and_bn(g, x, w_krsc, b, gamma, beta, False, relu, addend)
        assert np.array_equal(got[0], want[0]), "the convolution output must not change"
        for name, a, r in zip(("bn out", "save_mean", "save_inv_std", "running_mean", "running_var"), got[1:], want[1:]):
            assert_parity(a, r, np.float32, f"{shape} relu={relu} addend={with_addend} {name} vs separate pass")
        if g.flops <= 3e9 and not with_addend:
            # the un-fused chain on the CPU oracle
            y_ref = co.conv2d_forward(x, w, b, g, "NHWC")
            bn_ref, (std, _), rm_ref, rv_ref = ao.bn_train_forward(y_ref.astype(np.float64), gamma.astype(np.float64), beta.astype(np.float64),
                                                                   np.full(g.co, 0.25), np.full(g.co, 0.75), 0.9, 1e-5, "NHWC")
            if relu:
                bn_ref = np.maximum(bn_ref, 0)
            assert_parity(got[0], y_ref, np.float32, f"{shape} y vs oracle")
            # the normalised output divides by the batch deviation: the float32 convolution error (1e-6) is amplified by
            # |y - mean| / std only, so the float32 bar still holds
            assert_parity(got[1], bn_ref, np.float32, f"{shape} bn vs oracle")
            assert_parity(got[4], rm_ref, np.float32, f"{shape} running_mean vs oracle")
            assert_parity(got[5], rv_ref, np.float32, f"{shape} running_var vs oracle")


def test_batch_sums_are_bitwise_repeatable():
    """The sums are accumulated by fixed owners in a fixed order: two runs give the same bits."""
    g = co.Geom(64, 14, 14, 256, 256, 3, 3, 1, 1, 1, 1)
    rng = np.random.Generator(np.random.PCG64(3))
    x = rng.standard_normal((g.n, g.h, g.w, g.ci)).astype(np.float32)
    w = (rng.standard_normal((g.co, g.kh, g.kw, g.ci)) * np.sqrt(2.0 / g.k)).astype(np.float32)
    b = rng.standard_normal((g.co,)).astype(np.float32)
    gamma, beta = np.ones(g.co, np.float32), np.zeros(g.co, np.float32)
    a = _conv_and_bn(g, x, w, b, gamma, beta, True, False, None)
    c = _conv_and_bn(g, x, w, b, gamma, beta, True, False, None)
    for u, v in zip(a, c):
        assert np.array_equal(u, v)


def test_shapes_outside_the_path_are_refused():
    L = _lib.lib()
    g = co.Geom(2, 8, 8, 32, 64, 3, 3, 1, 1, 1, 1)
    for layout, dtype in (("NCHW", np.float32), ("NHWC", np.float64)):
        desc = make_desc(g, layout, dtype, "KRSC" if layout == "NHWC" else "KCRS")
        assert L.b2c_conv_stats_bytes(ctypes.byref(desc)) == 0
    desc = make_desc(g, "NHWC", np.float32, "KRSC", engine=_lib.ENGINE_FMA)
    assert L.b2c_conv_stats_bytes(ctypes.byref(desc)) == 0
    t = torch.zeros(64, device=DEV)
    rc = L.b2c_conv_fprop_stats(ctypes.byref(desc), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), t.data_ptr(), 256, t.data_ptr(), 256, stream())
    assert rc == -6
