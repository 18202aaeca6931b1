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


def _device_passes(g, layout, tdt, x, w, b, dy):
    """fprop, wgrad and dgrad of device tensors through the C ABI; returns device tensors."""
    import ctypes
    import torch
    from pydtnn_b200 import _lib
    from tests.gpu_util import make_desc, stream, workspace
    L = _lib.lib()
    desc = make_desc(g, layout, np.float32 if tdt == torch.float32 else np.float64, "KRSC" if layout == "NHWC" else "KCRS")
    ws = workspace(desc)
    y = torch.full_like(dy, float("nan"))
    dw, db, dx = torch.full_like(w, float("nan")), torch.full_like(b, float("nan")), torch.full_like(x, float("nan"))
    _lib.check(L.b2c_conv_fprop(ctypes.byref(desc), x.data_ptr(), w.data_ptr(), b.data_ptr(), None, 0, y.data_ptr(),
                                ws.data_ptr(), ws.numel(), stream()))
    _lib.check(L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                ws.data_ptr(), ws.numel(), stream()))
    _lib.check(L.b2c_conv_dgrad(ctypes.byref(desc), dy.data_ptr(), w.data_ptr(), dx.data_ptr(), ws.data_ptr(),
                                ws.numel(), stream()))
    return {"y": y, "dw": dw, "db": db, "dx": dx}


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("hw", [7, 14, 28, 56, 112])
def test_every_sweep_geometry_float32_against_the_float64_engine(hw, layout):
    """All 128 geometries of one image size (channels x kernel x stride), batch 2, on the device only: the float32
    result (tensor-core engine wherever it takes the shape) against the float64 FMA engine on the same inputs.
    The float64 engine is checked against the CPU oracle to 1e-12 on the sampled points above and on the golden
    vectors, so agreement to the float32 bar here carries the parity to every geometry of the sweep."""
    import torch
    from tests.gpu_util import DEV
    gen = torch.Generator(device=DEV).manual_seed(1000 + hw)
    worst = {}
    for ci, cout, k, stride in itertools.product((64, 128, 256, 512), (64, 128, 256, 512), (1, 3, 5, 7), (1, 2)):
        pad = (k - 1) // 2
        g = co.Geom(2, hw, hw, ci, cout, k, k, pad, pad, stride, stride)
        xs, ys = ((g.n, g.h, g.w, g.ci), (g.n, g.ho, g.wo, g.co)) if layout == "NHWC" else ((g.n, g.ci, g.h, g.w), (g.n, g.co, g.ho, g.wo))
        wsh = (g.co, g.kh, g.kw, g.ci) if layout == "NHWC" else (g.co, g.ci, g.kh, g.kw)
        x = torch.randn(xs, device=DEV, generator=gen)
        w = torch.randn(wsh, device=DEV, generator=gen) * float(np.sqrt(2.0 / g.k))
        b = torch.randn((g.co,), device=DEV, generator=gen)
        dy = torch.randn(ys, device=DEV, generator=gen)
        got = _device_passes(g, layout, torch.float32, x, w, b, dy)
        ref = _device_passes(g, layout, torch.float64, x.double(), w.double(), b.double(), dy.double())
        torch.cuda.synchronize()
        for nm in ("y", "dw", "db", "dx"):
            a, r = got[nm].double(), ref[nm]
            assert bool(torch.isfinite(a).all()), f"{g} {layout} {nm}: non-finite values"
            rel = float((a - r).norm() / r.norm().clamp_min(1e-300))
            mabs = float((a - r).abs().max() / r.abs().max().clamp_min(1e-300))
            assert rel <= 1e-5, f"{g} {layout} {nm}: rel-L2 {rel:.3e} > 1e-5"
            assert mabs <= 1e-4, f"{g} {layout} {nm}: max-abs {mabs:.3e} > 1e-4 of the largest value"
            worst[nm] = max(worst.get(nm, 0.0), rel)
    print(f"hw {hw} {layout}: worst rel-L2 {worst}")


# ---- every (kernel, stride, layout, dtype) combination of the sweep against the CPU oracle -------------------
_COMBOS = []
_crng = random.Random(777)
for _k, _s, _layout, _dt in itertools.product((1, 3, 5, 7), (1, 2), ("NHWC", "NCHW"), ("float32", "float64")):
    _hw = _crng.choice((7, 14, 28) if _k >= 5 else (7, 14, 28, 56))
    _ci, _co = _crng.choice((64, 128, 256)), _crng.choice((64, 128, 256))
    _COMBOS.append((_k, _s, _layout, _dt, _hw, _ci, _co))


@pytest.mark.parametrize("k,stride,layout,dtype,hw,ci,cout", _COMBOS)
def test_sweep_combination_against_oracle(k, stride, layout, dtype, hw, ci, cout):
    """One geometry per (kernel size, stride, layout, dtype) combination of the sweep, all four results against the
    CPU oracle at the stated bars, so that no combination is covered only by the float32-vs-float64-engine test."""
    dtype = np.dtype(dtype).type
    pad = (k - 1) // 2
    n = 1 if _cost(hw, ci, cout, k, stride) > 1.5e9 else 2
    g = co.Geom(n, hw, hw, ci, cout, k, k, pad, pad, stride, stride)
    rng = np.random.Generator(np.random.PCG64(hash((k, stride, hw, ci, cout)) & 0xFFFF))
    x = rng.standard_normal((g.n, g.h, g.w, g.ci)).astype(dtype)
    w = (rng.standard_normal((g.ci, g.kh, g.kw, g.co)) * np.sqrt(2.0 / g.k)).astype(dtype)
    b = rng.standard_normal((g.co,)).astype(dtype)
    dy = rng.standard_normal((g.n, g.ho, g.wo, g.co)).astype(dtype)
    if layout == "NCHW":
        x = np.ascontiguousarray(x.transpose(0, 3, 1, 2))
        w = np.ascontiguousarray(w.transpose(3, 0, 1, 2))
        dy = np.ascontiguousarray(dy.transpose(0, 3, 1, 2))
    keep = {}
    y = co.conv2d_forward(x, w, b, g, layout, keep=keep)
    dw, db, dx = co.conv2d_backward(x, dy, w, g, layout, keep=keep)
    out = run_conv(g, layout, np.dtype(dtype), x, w, b, dy, w_layout="KRSC" if layout == "NHWC" else "KCRS")
    for nm, ref in (("y", y), ("dw", dw), ("db", db), ("dx", dx)):
        assert_parity(out[nm], ref, dtype, f"{g} {layout} {np.dtype(dtype).name} {nm}")


# ---- the benchmark's own shapes at the benchmark's batch sizes ------------------------------------------------
def _resnet50_convs():
    """(h, ci, co, k, stride, pad) of every distinct Conv2D of ResNet-50 on 224x224 inputs
    (pydtnn/models/resnet50_imagenet.py:24-63: the stride sits on the 3x3 convolution)."""
    shapes = [(224, 3, 64, 7, 2, 3)]
    hw, cin = 56, 64
    for f, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for r in range(blocks):
            s = stride if r == 0 else 1
            shapes.append((hw, cin, f, 1, 1, 0))
            shapes.append((hw, f, f, 3, s, 1))
            shapes.append((hw // s, f, 4 * f, 1, 1, 0))
            if r == 0:
                shapes.append((hw, cin, 4 * f, 1, s, 0))
            hw, cin = hw // s, 4 * f
    return sorted(set(shapes))


def _vgg16_convs():
    shapes, hw, cin = [], 224, 3
    for f, convs in ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3)):
        for _ in range(convs):
            shapes.append((hw, cin, f, 3, 1, 1))
            cin = f
        hw //= 2
    return sorted(set(shapes))


_ALEXNET_CONVS = [(227, 3, 96, 11, 4, 0), (27, 96, 256, 5, 1, 2), (13, 256, 384, 3, 1, 1), (13, 384, 384, 3, 1, 1),
                  (13, 384, 256, 3, 1, 1)]
# not a network: short K loops (2 and 4 k-blocks per tile) on launches long enough to take split filter copies
# instead of the filter in place (more than 30000 tile x k-block units), a combination none of the networks has
_SHORT_K_LONG_LAUNCH = [(112, 64, 1024, 1, 1, 0), (112, 128, 640, 1, 1, 0)]
_NETWORKS = {"resnet50": (64, "NHWC", _resnet50_convs()), "vgg16": (32, "NHWC", _vgg16_convs()),
             "alexnet": (64, "NCHW", _ALEXNET_CONVS), "short_k_long_launch": (20, "NHWC", _SHORT_K_LONG_LAUNCH)}


@pytest.mark.parametrize("net", sorted(_NETWORKS))
def test_benchmark_shapes_at_full_batch_against_the_float64_engine(net):
    """Every distinct Conv2D shape of the three benchmark networks at the benchmark's own batch size (ResNet-50 at 64,
    VGG16 at 32, AlexNet at 64, its NCHW layout included): y, dw, db and dx of the float32 path AUTO picks against the
    float64 FMA engine on the same device tensors, at the float32 bar.  The float64 engine is within 1e-12 of the CPU
    oracle (sampled sweep points, golden vectors), so it referees sizes the oracle cannot finish in a test.
    Also pins the engine choice: every float32 NHWC pass with a multiple of 32 input channels, and the few-channel
    stems' fprop and wgrad, must run on the tensor-core engine."""
    import ctypes
    import torch
    from pydtnn_b200 import _lib
    from tests.gpu_util import DEV, make_desc
    batch, layout, shapes = _NETWORKS[net]
    L = _lib.lib()
    gen = torch.Generator(device=DEV).manual_seed(4242)
    worst = {}
    for hw, ci, cout, k, stride, pad in shapes:
        g = co.Geom(batch, hw, hw, ci, cout, k, k, pad, pad, stride, stride)
        desc = make_desc(g, layout, np.float32, "KRSC" if layout == "NHWC" else "KCRS")
        engines = [L.b2c_conv_engine_for(ctypes.byref(desc), p) for p in (_lib.PASS_FPROP, _lib.PASS_DGRAD, _lib.PASS_WGRAD)]
        if layout == "NCHW":         # channel-last copies are weighed against the FMA engine per pass; the forward pass always wins
            assert engines[0] == _lib.ENGINE_TENSOR, f"{net} {g}: fprop engine {engines[0]}, expected the tensor-core engine"
        elif ci % 32 == 0:
            assert engines == [_lib.ENGINE_TENSOR] * 3, \
                f"{net} {g}: engines {engines} (fprop, dgrad, wgrad), expected the tensor-core engine"
        else:
            assert engines[0] == _lib.ENGINE_TENSOR and engines[2] == _lib.ENGINE_TENSOR, f"{net} stem {g}: {engines}"
        xs, ys = ((g.n, g.h, g.w, g.ci), (g.n, g.ho, g.wo, g.co)) if layout == "NHWC" else ((g.n, g.ci, g.h, g.w), (g.n, g.co, g.ho, g.wo))
        wsh = (g.co, g.kh, g.kw, g.ci) if layout == "NHWC" else (g.co, g.ci, g.kh, g.kw)
        x = torch.randn(xs, device=DEV, generator=gen)
        w = torch.randn(wsh, device=DEV, generator=gen) * float(np.sqrt(2.0 / g.k))
        b = torch.randn((g.co,), device=DEV, generator=gen)
        dy = torch.randn(ys, device=DEV, generator=gen)
        got = _device_passes(g, layout, torch.float32, x, w, b, dy)
        ref = _device_passes(g, layout, torch.float64, x.double(), w.double(), b.double(), dy.double())
        torch.cuda.synchronize()
        for nm in ("y", "dw", "db", "dx"):
            a, r = got[nm].double(), ref[nm]
            assert bool(torch.isfinite(a).all()), f"{net} {g} {nm}: non-finite values"
            rel = float((a - r).norm() / r.norm().clamp_min(1e-300))
            mabs = float((a - r).abs().max() / r.abs().max().clamp_min(1e-300))
            assert rel <= 1e-5, f"{net} {g} {nm}: rel-L2 {rel:.3e} > 1e-5"
            assert mabs <= 1e-4, f"{net} {g} {nm}: max-abs {mabs:.3e} > 1e-4 of the largest value"
            worst[nm] = max(worst.get(nm, 0.0), rel)
        del x, w, b, dy, got, ref
        torch.cuda.empty_cache()
    _lib.check(L.b2c_check_device_status(None))
    print(f"{net} batch {batch} {layout}: worst rel-L2 {worst}")
