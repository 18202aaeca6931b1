"""Parity of the CUDA convolution / FC path with the CPU oracle and the reference's golden
vectors, through the C ABI.  Needs a GPU."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from pydtnn_b200 import _lib
from tests.gpu_util import (DEV, assert_parity, dev, make_desc, rel_l2, run_conv, stream, workspace)

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
ENGINES = {"auto": _lib.ENGINE_AUTO, "fma": _lib.ENGINE_FMA}


def _geom(arr):
    return co.Geom(*[int(v) for v in arr])


@pytest.mark.parametrize("engine", ["auto", "fma"])
@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_golden_vectors_from_the_reference(layout, dtype, engine):
    ref = np.load(os.path.join(GOLD, "conv_ref.npz"))
    for i in range(8):
        key = f"c{i}_{layout}_{dtype}"
        g = _geom(ref[key + "_geom"])
        x, w, b, dy = (ref[f"{key}_{n}"] for n in ("x", "w", "b", "dy"))
        for w_layout in (("CRSK", "KRSC") if layout == "NHWC" else ("KCRS",)):
            out = run_conv(g, layout, np.dtype(dtype), x, w, b, dy, w_layout=w_layout, engine=ENGINES[engine])
            for name in ("y", "dw", "db", "dx"):
                assert_parity(out[name], ref[f"{key}_{name}"], dtype, f"{key} {w_layout} {name}")


def test_known_answer_cases_are_exact():
    ka = np.load(os.path.join(GOLD, "conv_known_answer.npz"))
    for i in range(int(ka["count"])):
        x, w = ka[f"k{i}_x"], ka[f"k{i}_w"]
        vs, hs = [int(v) for v in ka[f"k{i}_stride"]]
        g = co.Geom(x.shape[0], x.shape[2], x.shape[3], x.shape[1], w.shape[0], w.shape[2], w.shape[3], 0, 0, vs, hs)
        y_ref = ka[f"k{i}_y"]
        out = run_conv(g, "NCHW", np.float32, x, w, np.zeros(1, np.float32), np.ones_like(y_ref))
        assert np.array_equal(out["y"], y_ref)
        assert np.array_equal(out["dw"], ka[f"k{i}_dw"])
        assert np.array_equal(out["dx"], ka[f"k{i}_dx"])


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_index_map_is_bit_exact(layout):
    ref = np.load(os.path.join(GOLD, "conv_ref.npz"))
    geoms = [_geom(ref[f"c{i}_{layout}_float32_geom"]) for i in range(8)]
    geoms.append(co.Geom(3, 17, 13, 5, 2, 3, 5, 2, 1, 2, 3, 2, 1))
    geoms.append(co.Geom(2, 32, 32, 16, 8, 3, 3, 1, 1, 1, 1, 1, 1))
    L = _lib.lib()
    for g in geoms:
        want = co.index_map_nhwc(g) if layout == "NHWC" else co.index_map_nchw(g)
        got = torch.full(want.shape, -7, dtype=torch.int64, device=DEV)
        desc = make_desc(g, layout, np.float32, "CRSK" if layout == "NHWC" else "KCRS")
        _lib.check(L.b2c_conv_index_map(ctypes.byref(desc), got.data_ptr(), stream()))
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), want), g


# shapes of the benchmark configurations at oracle-friendly batch sizes
PARITY_SHAPES = {
    "cfg1_3x3_64_64_n64": co.Geom(64, 32, 32, 64, 64, 3, 3, 1, 1, 1, 1),
    "resnet_stem_7x7s2": co.Geom(2, 224, 224, 3, 64, 7, 7, 3, 3, 2, 2),
    "resnet_1x1_64_256": co.Geom(4, 56, 56, 64, 256, 1, 1, 0, 0, 1, 1),
    "resnet_1x1_256_64": co.Geom(4, 56, 56, 256, 64, 1, 1, 0, 0, 1, 1),
    "resnet_3x3s2_128": co.Geom(4, 56, 56, 128, 128, 3, 3, 1, 1, 2, 2),
    "resnet_1x1s2_256_512": co.Geom(4, 56, 56, 256, 512, 1, 1, 0, 0, 2, 2),
    "resnet_3x3_512_7": co.Geom(8, 7, 7, 512, 512, 3, 3, 1, 1, 1, 1),
    "alexnet_conv1_11x11s4": co.Geom(2, 227, 227, 3, 96, 11, 11, 0, 0, 4, 4),
    "alexnet_conv2_5x5": co.Geom(2, 27, 27, 96, 256, 5, 5, 2, 2, 1, 1),
    "sweep_5x5s2_14": co.Geom(4, 14, 14, 64, 128, 5, 5, 2, 2, 2, 2),
    "sweep_7x7_28": co.Geom(2, 28, 28, 64, 64, 7, 7, 3, 3, 1, 1),
    "dilated_3x3": co.Geom(2, 20, 20, 16, 24, 3, 3, 2, 2, 1, 1, 2, 2),
    "ragged_everything": co.Geom(3, 13, 11, 7, 5, 3, 2, 1, 0, 2, 1, 1, 1),
    # strides that differ, extents the strides do not divide, a kernel narrower than the stride in one direction:
    # some residue classes of the input pixels have no tap at all (their gradient is zero)
    "stride_3x2_odd_extent": co.Geom(2, 17, 13, 8, 12, 2, 5, 1, 2, 3, 2),
    "single_pixel": co.Geom(1, 1, 1, 1, 1, 1, 1, 0, 0, 1, 1),
    "pad_larger_than_input": co.Geom(1, 2, 2, 3, 2, 3, 3, 2, 2, 1, 1),
    # tile counts that do not fill the CTA grid evenly: the tensor-core kernel balances (tile, k-block) units over
    # the CTAs and tiles are shared by 2 (first case) or about 6 (second case) consecutive CTAs
    "balanced_160_tiles_9_kblocks": co.Geom(5, 64, 64, 32, 128, 3, 3, 1, 1, 1, 1),
    "balanced_50_tiles_72_kblocks": co.Geom(16, 14, 14, 256, 256, 3, 3, 1, 1, 1, 1),
    # short K loops (1-4 k-blocks: eight drain warps, filter tiles resident in shared memory, a grid that is a multiple
    # of the column-tile count): a ragged last row tile, a half-empty last column tile (192 = 128 + 64), three and one
    # k-blocks, a 64-wide and a 96-wide output; more row tiles than SMs in the first (every CTA walks several tiles)
    "short_k_2kb_ragged_rows_192_cols": co.Geom(3, 91, 91, 64, 192, 1, 1, 0, 0, 1, 1),
    "short_k_3kb_96_cols": co.Geom(2, 29, 31, 96, 96, 1, 1, 0, 0, 1, 1),
    "short_k_1kb_64_cols": co.Geom(5, 20, 20, 32, 64, 1, 1, 0, 0, 1, 1),
    "short_k_4kb_5_column_tiles": co.Geom(2, 40, 40, 128, 640, 1, 1, 0, 0, 1, 1),
}


def _inputs(g, dtype, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((g.n, g.h, g.w, g.ci)).astype(dtype)
    w = (rng.standard_normal((g.ci, g.kh, g.kw, g.co)) * np.sqrt(2.0 / g.k)).astype(dtype)
    b = rng.standard_normal((g.co,)).astype(dtype)
    dy = rng.standard_normal((g.n, g.ho, g.wo, g.co)).astype(dtype)
    return x, w, b, dy


def _to_layout(x, w, dy, layout):
    if layout == "NHWC":
        return x, w, dy
    t = lambda a: np.ascontiguousarray(a.transpose(0, 3, 1, 2))
    return t(x), np.ascontiguousarray(w.transpose(3, 0, 1, 2)), t(dy)


@pytest.mark.parametrize("engine", ["auto", "fma"])
@pytest.mark.parametrize("name", list(PARITY_SHAPES))
def test_float32_nhwc_against_oracle(name, engine):
    g = PARITY_SHAPES[name]
    x, w, b, dy = _inputs(g, np.float32)
    keep = {}
    y = co.conv2d_forward(x, w, b, g, "NHWC", keep=keep)
    dw, db, dx = co.conv2d_backward(x, dy, w, g, "NHWC", keep=keep)
    out = run_conv(g, "NHWC", np.float32, x, w, b, dy, w_layout="KRSC", engine=ENGINES[engine])
    for nm, ref in (("y", y), ("dw", dw), ("db", db), ("dx", dx)):
        assert_parity(out[nm], ref, np.float32, f"{name} {nm}")


@pytest.mark.parametrize("w_layout", ["KRSC", "CRSK"])
@pytest.mark.parametrize("shape", [(4, 56, 56, 64, 256), (3, 27, 29, 32, 128), (2, 28, 28, 64, 160)])
def test_1x1_weight_gradient_without_bias_on_few_input_channels(shape, w_layout):
    """Without a bias gradient to take, a 1x1 weight gradient with at most 64 input channels runs with x and dy
    exchanged (co on the GEMM row axis) and writes dw through exchanged filter strides: same dw, both filter layouts,
    and the same as the plain form that a bias gradient request selects."""
    n, h, w_, ci, cout = shape
    g = co.Geom(n, h, w_, ci, cout, 1, 1, 0, 0, 1, 1)
    x, w, b, dy = _inputs(g, np.float32, seed=5)
    dw, db, _ = co.conv2d_backward(x, dy, w, g, "NHWC")
    exchanged = run_conv(g, "NHWC", np.float32, x, w, None, dy, w_layout=w_layout, passes=("wgrad",))
    plain = run_conv(g, "NHWC", np.float32, x, w, b, dy, w_layout=w_layout, passes=("wgrad",))
    assert exchanged["db"] is None
    assert_parity(exchanged["dw"], dw, np.float32, f"{shape} {w_layout} dw, exchanged operands")
    assert_parity(plain["dw"], dw, np.float32, f"{shape} {w_layout} dw")
    assert_parity(plain["db"], db, np.float32, f"{shape} {w_layout} db")


@pytest.mark.parametrize("layout,dtype", [("NCHW", "float32"), ("NHWC", "float64"), ("NCHW", "float64")])
@pytest.mark.parametrize("name", ["cfg1_3x3_64_64_n64", "resnet_3x3s2_128", "resnet_1x1_64_256", "sweep_5x5s2_14",
                                  "dilated_3x3", "ragged_everything", "alexnet_conv1_11x11s4", "resnet_1x1s2_256_512",
                                  "stride_3x2_odd_extent"])
def test_other_layouts_and_float64_against_oracle(name, layout, dtype):
    g = PARITY_SHAPES[name]
    if name == "cfg1_3x3_64_64_n64":
        g = co.Geom(16, *[getattr(g, f) for f in ("h", "w", "ci", "co", "kh", "kw", "vpad", "hpad", "vstr", "hstr")])
    x, w, b, dy = _inputs(g, np.dtype(dtype), seed=1)
    xl, wl, dyl = _to_layout(x, w, dy, layout)
    keep = {}
    y = co.conv2d_forward(xl, wl, b, g, layout, keep=keep)
    dw, db, dx = co.conv2d_backward(xl, dyl, wl, g, layout, keep=keep)
    out = run_conv(g, layout, np.dtype(dtype), xl, wl, b, dyl)
    for nm, ref in (("y", y), ("dw", dw), ("db", db), ("dx", dx)):
        assert_parity(out[nm], ref, dtype, f"{name} {layout} {dtype} {nm}")


# the fused epilogue on every drain path of the tensor-core kernel: the chunked drain (3x3, nine k-blocks), the
# streaming epilogue with eight drain warps and resident filter tiles (1x1 on 64 and on 128 channels: 128- and 64-wide
# column tiles), the streaming epilogue with four drain warps (1x1 on 256 channels, a partial last column tile)
_EPILOGUE_GEOMS = {"3x3_32_48": co.Geom(4, 14, 14, 32, 48, 3, 3, 1, 1, 1, 1),
                   "1x1_64_256": co.Geom(4, 28, 28, 64, 256, 1, 1, 0, 0, 1, 1),
                   "1x1_128_64": co.Geom(2, 28, 28, 128, 64, 1, 1, 0, 0, 1, 1),
                   "1x1_256_192": co.Geom(2, 14, 14, 256, 192, 1, 1, 0, 0, 1, 1)}


@pytest.mark.parametrize("mode", ["relu", "bn", "bn_relu", "nobias_bn_relu"])
@pytest.mark.parametrize("layout,geom", [("NHWC", k) for k in _EPILOGUE_GEOMS] + [("NCHW", "3x3_32_48")])
def test_fused_inference_epilogue(layout, geom, mode):
    g = _EPILOGUE_GEOMS[geom]
    x, w, b, dy = _inputs(g, np.float32, seed=2)
    xl, wl, _ = _to_layout(x, w, dy, layout)
    rng = np.random.Generator(np.random.PCG64(5))
    bn = dict(running_mean=rng.standard_normal(g.co).astype(np.float32),
              inv_std=(1.0 / np.sqrt(rng.uniform(0.5, 2.0, g.co) + 1e-5)).astype(np.float32),
              gamma=rng.standard_normal(g.co).astype(np.float32), beta=rng.standard_normal(g.co).astype(np.float32))
    use_bn = "bn" in mode
    use_relu = "relu" in mode
    bias = None if mode.startswith("nobias") else b
    ref = co.conv2d_fused_inference(xl, wl, bias, g, layout, bn if use_bn else None, use_relu)
    out = run_conv(g, layout, np.float32, xl, wl, bias, None, bn=bn if use_bn else None, relu=use_relu,
                   passes=("fprop",))
    assert_parity(out["y"], ref, np.float32, f"fused {mode} {layout} {geom}")


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_fc_against_reference_golden_and_oracle(dtype):
    L = _lib.lib()
    ref = np.load(os.path.join(GOLD, "fc_ref.npz"))
    cases = [tuple(ref[f"f{i}_{dtype}_{n}"] for n in ("x", "w", "b", "dy", "y", "dw", "db", "dx")) for i in range(3)]
    rng = np.random.Generator(np.random.PCG64(3))
    # tensor-core forward and input gradient; partial tiles and a ragged batch in the dense dw kernel; the last three take
    # the small-batch route (the weight matrix on the GEMM row axis): whole tiles, an input count that is not a multiple
    # of a k-block, an output count that is not a multiple of a tile, batches of 32 / 64 / 96
    for (bsz, fin, fout) in ((64, 2048, 1000), (32, 1000, 4096), (5, 7, 3), (21, 200, 132),
                             (64, 4096, 2048), (32, 2052, 4096), (96, 2048, 2080)):
        x = rng.standard_normal((bsz, fin)).astype(dtype)
        w = (rng.standard_normal((fin, fout)) / np.sqrt(fin)).astype(dtype)
        b = rng.standard_normal((fout,)).astype(dtype)
        dy = rng.standard_normal((bsz, fout)).astype(dtype)
        y = co.fc_forward(x, w, b)
        dw, db, dx = co.fc_backward(x, dy, w)
        cases.append((x, w, b, dy, y, dw, db, dx))
    dt = _lib.dtype_code(dtype)
    for x, w, b, dy, y, dw, db, dx in cases:
        bsz, fin = x.shape
        fout = w.shape[1]
        nbytes = L.b2c_fc_workspace_bytes(dt, bsz, fin, fout, 0)
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=DEV)
        xd, wd, bd, dyd = dev(x), dev(w), dev(b), dev(dy)
        yd, dwd, dbd, dxd = torch.empty_like(dyd), torch.empty_like(wd), torch.empty_like(bd), torch.empty_like(xd)
        _lib.check(L.b2c_fc_forward(dt, 0, bsz, fin, fout, xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), yd.data_ptr(),
                                    ws.data_ptr(), ws.numel(), stream()))
        _lib.check(L.b2c_fc_backward(dt, 0, bsz, fin, fout, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(), dwd.data_ptr(),
                                     dbd.data_ptr(), dxd.data_ptr(), ws.data_ptr(), ws.numel(), stream()))
        torch.cuda.synchronize()
        for nm, got, want in (("y", yd, y), ("dw", dwd, dw), ("db", dbd, db), ("dx", dxd, dx)):
            assert_parity(got.cpu().numpy(), want, dtype, f"fc {x.shape}x{w.shape} {nm}")


@pytest.mark.parametrize("engine", ["auto", "fma"])
@pytest.mark.parametrize("shape", [(64, 56, 56, 64, 64, 3, 1, 1), (64, 56, 56, 256, 64, 1, 0, 1),
                                   (64, 28, 28, 128, 128, 3, 1, 2), (64, 14, 14, 256, 1024, 1, 0, 1),
                                   # 196 and 100 output tiles on 148 SMs: the balanced (tile, k-block) split
                                   (64, 14, 14, 256, 256, 3, 1, 1), (64, 7, 7, 512, 512, 3, 1, 1),
                                   # the network stem: 3 channels, written-out im2row matrix
                                   (64, 224, 224, 3, 64, 7, 3, 2)])
def test_full_batch_properties(shape, engine):
    """At the benchmark's batch size the oracle is too slow, so check what holds at any size:
    the three passes are mutually adjoint, <fprop(x,w),dy> = <x,dgrad(dy,w)> = <w,wgrad(x,dy)>,
    the forward pass is linear in x, and a second run is bitwise identical (fixed summation order)."""
    n, h, w_, ci, cout, k, pad, stride = shape
    g = co.Geom(n, h, w_, ci, cout, k, k, pad, pad, stride, stride)
    L = _lib.lib()
    gen = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn((g.n, g.h, g.w, g.ci), device=DEV, generator=gen)
    x2 = torch.randn((g.n, g.h, g.w, g.ci), device=DEV, generator=gen)
    wt = torch.randn((g.co, g.kh, g.kw, g.ci), device=DEV, generator=gen) * (2.0 / g.k) ** 0.5
    dy = torch.randn((g.n, g.ho, g.wo, g.co), device=DEV, generator=gen)
    desc = make_desc(g, "NHWC", np.float32, "KRSC", ENGINES[engine])
    ws = workspace(desc)

    def fprop(inp):
        y = torch.empty((g.n, g.ho, g.wo, g.co), device=DEV)
        _lib.check(L.b2c_conv_fprop(ctypes.byref(desc), inp.data_ptr(), wt.data_ptr(), None, None, 0, y.data_ptr(),
                                    ws.data_ptr(), ws.numel(), stream()))
        return y

    y = fprop(x)
    dx = torch.empty_like(x)
    dw = torch.empty_like(wt)
    db = torch.empty((g.co,), device=DEV)
    _lib.check(L.b2c_conv_dgrad(ctypes.byref(desc), dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), ws.data_ptr(),
                                ws.numel(), stream()))
    _lib.check(L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                ws.data_ptr(), ws.numel(), stream()))
    dot = lambda a, b: float((a.double() * b.double()).sum())
    a, b_, c = dot(y, dy), dot(x, dx), dot(wt, dw)
    scale = float(y.double().norm() * dy.double().norm())
    assert abs(a - b_) <= 1e-5 * scale and abs(a - c) <= 1e-5 * scale, (a, b_, c, scale)
    assert rel_l2(db.cpu().numpy(), dy.double().sum(dim=(0, 1, 2)).cpu().numpy()) <= 1e-6
    y_lin = fprop(2.5 * x + x2)
    want = 2.5 * y.double() + fprop(x2).double()
    assert float((y_lin.double() - want).norm() / want.norm()) <= 1e-5
    assert torch.equal(fprop(x), y)
    dw2 = torch.empty_like(wt)
    _lib.check(L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw2.data_ptr(), None,
                                ws.data_ptr(), ws.numel(), stream()))
    assert torch.equal(dw, dw2)


def test_errors_are_status_codes_not_faults():
    L = _lib.lib()
    g = co.Geom(64, 32, 32, 64, 64, 3, 3, 1, 1, 1, 1)
    desc = make_desc(g, "NHWC", np.float32, "KRSC", _lib.ENGINE_FMA)
    x = torch.zeros((g.n, g.h, g.w, g.ci), device=DEV)
    wt = torch.zeros((g.co, 3, 3, g.ci), device=DEV)
    dy = torch.zeros((g.n, g.ho, g.wo, g.co), device=DEV)
    dw = torch.zeros_like(wt)
    # wgrad needs split-K scratch for this shape: refusing a missing / short workspace is a status
    assert L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw.data_ptr(), None, None, 0, stream()) == -4
    tiny = torch.empty(64, dtype=torch.uint8, device=DEV)
    assert L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw.data_ptr(), None, tiny.data_ptr(), 64,
                            stream()) == -4
    torch.cuda.synchronize()


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """Every in-kernel wait of the tensor-core engine is bounded. Nothing is broken here: a self-test kernel waits on
    a barrier nothing arrives at, for at most 20 M cycles (about 10 ms); the wait gives up, the kernel returns, the
    status word reports it once, and the next convolution runs as usual."""
    L = _lib.lib()
    L.b2c_check_device_status(None)                       # clear whatever an earlier test may have left
    _lib.check(L.b2c_selftest_bounded_wait(20_000_000, stream()))
    detail = ctypes.c_int(0)
    assert L.b2c_check_device_status(ctypes.byref(detail)) == -9          # B2C_ERR_DEVICE_TIMEOUT
    assert detail.value == 7
    assert L.b2c_check_device_status(ctypes.byref(detail)) == 0 and detail.value == 0     # read once, then cleared
    assert L.b2c_selftest_bounded_wait(0, stream()) == -2                 # limits outside 1..2e9 are refused
    g = PARITY_SHAPES["cfg1_3x3_64_64_n64"]
    x, w, b, dy = _inputs(g, np.float32)
    y = co.conv2d_forward(x, w, b, g, "NHWC", keep={})
    out = run_conv(g, "NHWC", np.float32, x, w, b, dy, w_layout="KRSC")
    assert_parity(out["y"], y, np.float32, "conv after a timed-out wait")
    assert L.b2c_check_device_status(None) == 0


@pytest.mark.parametrize("ci,passes", [(4, ("fprop", "wgrad", "dgrad")), (3, ("fprop", "wgrad")), (8, ("fprop", "wgrad", "dgrad"))])
def test_nchw_few_channels_on_the_tensor_engine(ci, passes):
    """NCHW tensors with at most 8 channels go through the thin layout copies (one thread per pixel) on their way to
    and from the channel-last kernels; the engine is forced so that the small shape does not fall to the FMA engine."""
    g = co.Geom(3, 21, 19, ci, 32, 3, 3, 1, 1, 1, 1)
    x, w, b, dy = _inputs(g, np.float32, seed=5)
    xl, wl, dyl = _to_layout(x, w, dy, "NCHW")
    keep = {}
    y = co.conv2d_forward(xl, wl, b, g, "NCHW", keep=keep)
    dw, db, dx = co.conv2d_backward(xl, dyl, wl, g, "NCHW", keep=keep)
    out = run_conv(g, "NCHW", np.float32, xl, wl, b, dyl, engine=_lib.ENGINE_TENSOR, passes=passes)
    refs = {"y": y, "dw": dw, "db": db, "dx": dx}
    for nm in ("y",) + (("dw", "db") if "wgrad" in passes else ()) + (("dx",) if "dgrad" in passes else ()):
        assert_parity(out[nm], refs[nm], np.float32, f"NCHW ci={ci} {nm}")


def test_balanced_mode_layer_next_to_a_kernel_that_holds_most_sms():
    """The balanced mode hands partial tiles between consecutive CTAs.  Its CTAs need not be resident together: here a
    long weight-gradient kernel (144 persistent CTAs, each owning its SM's shared memory) is started on a second stream
    and a balanced forward pass right behind it on the first, so only a few of the 148 CTAs can start until the other
    kernel ends.  The result must be bit-identical to the same pass run alone, and no bounded wait may run out."""
    L = _lib.lib()
    big = co.Geom(64, 56, 56, 256, 256, 3, 3, 1, 1, 1, 1)          # wgrad: 36 output tiles x 4 pixel ranges = 144 CTAs, about 1 ms
    bal = co.Geom(64, 14, 14, 256, 256, 3, 3, 1, 1, 1, 1)          # fprop: 196 tiles x 72 k-blocks on 148 CTAs -> balanced ranges
    gen = torch.Generator(device=DEV).manual_seed(77)
    dbig, dbal = make_desc(big, "NHWC", np.float32, "KRSC"), make_desc(bal, "NHWC", np.float32, "KRSC")
    xb = torch.randn((big.n, big.h, big.w, big.ci), device=DEV, generator=gen)
    dyb = torch.randn((big.n, big.ho, big.wo, big.co), device=DEV, generator=gen)
    dwb = torch.empty((big.co, 3, 3, big.ci), device=DEV)
    x = torch.randn((bal.n, bal.h, bal.w, bal.ci), device=DEV, generator=gen)
    w = torch.randn((bal.co, 3, 3, bal.ci), device=DEV, generator=gen) * 0.03
    y_alone, y_busy = torch.empty((bal.n, bal.ho, bal.wo, bal.co), device=DEV), torch.empty((bal.n, bal.ho, bal.wo, bal.co), device=DEV)
    ws_a, ws_b = workspace(dbal), workspace(dbig)
    main = torch.cuda.current_stream()
    other = torch.cuda.Stream()

    def fprop(out):
        _lib.check(L.b2c_conv_fprop(ctypes.byref(dbal), x.data_ptr(), w.data_ptr(), None, None, 0, out.data_ptr(), ws_a.data_ptr(),
                                    ws_a.numel(), main.cuda_stream))
    fprop(y_alone)
    torch.cuda.synchronize()
    for _ in range(3):                                             # a few rounds: the overlap depends on launch timing
        y_busy.fill_(float("nan"))
        torch.cuda.synchronize()
        _lib.check(L.b2c_conv_wgrad(ctypes.byref(dbig), xb.data_ptr(), dyb.data_ptr(), dwb.data_ptr(), None, ws_b.data_ptr(),
                                    ws_b.numel(), other.cuda_stream))
        fprop(y_busy)
        torch.cuda.synchronize()
        _lib.check(L.b2c_check_device_status(None))
        assert torch.equal(y_busy, y_alone)


def test_weight_gradient_from_the_forward_pass_lowered_input_is_bit_identical():
    """A few-channel layer (network stem) writes its im2row matrix into the workspace in the forward pass; with the same
    workspace untouched, b2c_conv_wgrad_lowered must give the bits of b2c_conv_wgrad (which lowers x again)."""
    L = _lib.lib()
    g = co.Geom(4, 40, 40, 3, 64, 7, 7, 3, 3, 2, 2)
    desc = make_desc(g, "NHWC", np.float32, "KRSC")
    assert L.b2c_conv_keeps_lowered_input(ctypes.byref(desc)) == 1
    gen = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn((g.n, g.h, g.w, g.ci), device=DEV, generator=gen)
    w = torch.randn((g.co, 7, 7, g.ci), device=DEV, generator=gen) * 0.1
    b = torch.randn((g.co,), device=DEV, generator=gen)
    dy = torch.randn((g.n, g.ho, g.wo, g.co), device=DEV, generator=gen)
    y = torch.empty_like(dy)
    ws = workspace(desc)
    out = {}
    for name in ("plain", "lowered"):
        dw, db = torch.full_like(w, float("nan")), torch.full_like(b, float("nan"))
        _lib.check(L.b2c_conv_fprop(ctypes.byref(desc), x.data_ptr(), w.data_ptr(), b.data_ptr(), None, 0, y.data_ptr(), ws.data_ptr(),
                                    ws.numel(), stream()))
        fn = L.b2c_conv_wgrad if name == "plain" else L.b2c_conv_wgrad_lowered
        _lib.check(fn(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), dw.data_ptr(), db.data_ptr(), ws.data_ptr(), ws.numel(), stream()))
        torch.cuda.synchronize()
        out[name] = (dw.cpu().numpy(), db.cpu().numpy())
    assert np.array_equal(out["plain"][0], out["lowered"][0]) and np.array_equal(out["plain"][1], out["lowered"][1])
    # layers with a multiple of 32 input channels never lower: the entry point refuses them
    g2 = co.Geom(2, 8, 8, 32, 32, 3, 3, 1, 1, 1, 1)
    d2 = make_desc(g2, "NHWC", np.float32, "KRSC")
    assert L.b2c_conv_keeps_lowered_input(ctypes.byref(d2)) == 0
    t = torch.zeros(64, device=DEV)
    assert L.b2c_conv_wgrad_lowered(ctypes.byref(d2), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 256, stream()) == -6
