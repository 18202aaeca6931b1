"""A seeded sample of the shape sweep (H=W in {7,14,28,56,112}, Ci/Co in {64,128,256,512}, 1x1/3x3/5x5/7x7,
stride 1/2, 'same' padding; float32 and float64, NHWC and NCHW; fprop, dgrad, wgrad) against the CPU
oracle, at a batch the oracle finishes quickly.  GPU."""
import itertools
import random

import numpy as np
import pytest

from oracle import conv_oracle as co
from tests.gpu_util import assert_parity, run_conv

pytestmark = pytest.mark.gpu

_ALL = list(itertools.product((7, 14, 28, 56, 112), (64, 128, 256, 512), (64, 128, 256, 512), (1, 3, 5, 7), (1, 2)))
_rng = random.Random(20240)
_SAMPLE = _rng.sample(_ALL, 28)


def _cost(hw, ci, cout, k, s):
    return (hw // s) ** 2 * ci * cout * k * k


@pytest.mark.parametrize("hw,ci,cout,k,stride", _SAMPLE)
def test_sweep_point(hw, ci, cout, k, stride):
    # batch 2, or 1 for the heaviest points, keeps the CPU oracle to a few seconds per point
    n = 1 if _cost(hw, ci, cout, k, stride) > 3e9 else 2
    if _cost(hw, ci, cout, k, stride) * n > 1.5e10:
        pytest.skip("oracle too slow for this point; covered by the adjoint-property test at full size")
    pad = (k - 1) // 2
    g = co.Geom(n, hw, hw, ci, cout, k, k, pad, pad, stride, stride)
    seed = hash((hw, ci, cout, k, stride)) & 0xFFFF
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((g.n, g.h, g.w, g.ci)).astype(np.float32)
    w = (rng.standard_normal((g.ci, g.kh, g.kw, g.co)) * np.sqrt(2.0 / g.k)).astype(np.float32)
    b = rng.standard_normal((g.co,)).astype(np.float32)
    dy = rng.standard_normal((g.n, g.ho, g.wo, g.co)).astype(np.float32)
    combos = [("NHWC", np.float32)]
    if seed % 3 == 0:
        combos.append(("NCHW", np.float32))
    if seed % 4 == 0 and _cost(hw, ci, cout, k, stride) < 1e9:
        combos.append(("NHWC", np.float64))
    for layout, dtype in combos:
        xl, wl, dyl = x.astype(dtype), w.astype(dtype), dy.astype(dtype)
        if layout == "NCHW":
            xl = np.ascontiguousarray(xl.transpose(0, 3, 1, 2))
            wl = np.ascontiguousarray(wl.transpose(3, 0, 1, 2))
            dyl = np.ascontiguousarray(dyl.transpose(0, 3, 1, 2))
        keep = {}
        y = co.conv2d_forward(xl, wl, b.astype(dtype), g, layout, keep=keep)
        dw, db, dx = co.conv2d_backward(xl, dyl, wl, g, layout, keep=keep)
        out = run_conv(g, layout, np.dtype(dtype), xl, wl, b.astype(dtype), dyl,
                       w_layout="KRSC" if layout == "NHWC" else "KCRS")
        for nm, ref in (("y", y), ("dw", dw), ("db", db), ("dx", dx)):
            assert_parity(out[nm], ref, dtype, f"{g} {layout} {np.dtype(dtype).name} {nm}")
