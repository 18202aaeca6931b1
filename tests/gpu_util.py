"""Helpers for the GPU parity tests: call the C ABI with NumPy arrays (torch moves the bytes)."""
import ctypes

import numpy as np
import torch

from oracle import conv_oracle as co
from pydtnn_b200 import _lib

DEV = "cuda:0"
W_LAYOUTS = {"CRSK": _lib.W_CRSK, "KCRS": _lib.W_KCRS, "KRSC": _lib.W_KRSC}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def stream():
    return torch.cuda.current_stream().cuda_stream


def make_desc(g: co.Geom, layout, dtype, w_layout, engine=_lib.ENGINE_AUTO):
    return _lib.ConvDesc(_lib.LAYOUT_NHWC if layout == "NHWC" else _lib.LAYOUT_NCHW, _lib.dtype_code(dtype),
                         W_LAYOUTS[w_layout], engine, g.n, g.h, g.w, g.ci, g.co, g.kh, g.kw, g.vpad, g.hpad,
                         g.vstr, g.hstr, g.vdil, g.hdil)


def workspace(desc):
    L = _lib.lib()
    n = max(L.b2c_conv_workspace_bytes(ctypes.byref(desc), p) for p in range(3))
    return torch.empty(max(int(n), 256), dtype=torch.uint8, device=DEV)


def w_from_cpu_layout(w, layout, w_layout):
    """Oracle filter layout (NHWC: (ci,kh,kw,co); NCHW: (co,ci,kh,kw)) -> requested layout."""
    if layout == "NHWC":
        crsk = w
    else:
        crsk = w.transpose(1, 2, 3, 0)
    if w_layout == "CRSK":
        return np.ascontiguousarray(crsk)
    if w_layout == "KCRS":
        return np.ascontiguousarray(crsk.transpose(3, 0, 1, 2))
    return np.ascontiguousarray(crsk.transpose(3, 1, 2, 0))


def w_to_cpu_layout(wl, layout, w_layout):
    if w_layout == "CRSK":
        crsk = wl
    elif w_layout == "KCRS":
        crsk = wl.transpose(1, 2, 3, 0)
    else:
        crsk = wl.transpose(3, 1, 2, 0)
    return np.ascontiguousarray(crsk if layout == "NHWC" else crsk.transpose(3, 0, 1, 2))


def run_conv(g, layout, dtype, x, w_cpu, b, dy, w_layout=None, engine=_lib.ENGINE_AUTO, need_dx=True, bn=None,
             relu=False, passes=("fprop", "wgrad", "dgrad")):
    """Run the passes through the C ABI. ``w_cpu`` is in the oracle's filter layout; results come back
    in the oracle's layouts: dict(y, dw, db, dx)."""
    L = _lib.lib()
    w_layout = w_layout or ("CRSK" if layout == "NHWC" else "KCRS")
    desc = make_desc(g, layout, dtype, w_layout, engine)
    ws = workspace(desc)
    xd, wd = dev(x.astype(dtype)), dev(w_from_cpu_layout(w_cpu.astype(dtype), layout, w_layout))
    bd = dev(b.astype(dtype)) if b is not None else None
    out = {}
    yshape = (g.n, g.ho, g.wo, g.co) if layout == "NHWC" else (g.n, g.co, g.ho, g.wo)
    if "fprop" in passes:
        yd = torch.full(yshape, float("nan"), dtype=xd.dtype, device=DEV)
        bnp = None
        keepalive = []
        if bn is not None:
            vecs = [dev(bn[k].astype(dtype)) for k in ("running_mean", "inv_std", "gamma", "beta")]
            keepalive += vecs
            bnp = ctypes.byref(_lib.BnParams(*[v.data_ptr() for v in vecs]))
        _lib.check(L.b2c_conv_fprop(ctypes.byref(desc), xd.data_ptr(), wd.data_ptr(),
                                    bd.data_ptr() if bd is not None else None, bnp, int(relu), yd.data_ptr(),
                                    ws.data_ptr(), ws.numel(), stream()))
        out["y"] = yd.cpu().numpy()
    if dy is not None:
        dyd = dev(dy.astype(dtype))
        if "wgrad" in passes:
            dwd = torch.full(wd.shape, float("nan"), dtype=xd.dtype, device=DEV)
            dbd = torch.full((g.co,), float("nan"), dtype=xd.dtype, device=DEV) if b is not None else None
            _lib.check(L.b2c_conv_wgrad(ctypes.byref(desc), xd.data_ptr(), dyd.data_ptr(), dwd.data_ptr(),
                                        dbd.data_ptr() if dbd is not None else None, ws.data_ptr(), ws.numel(), stream()))
            out["dw"] = w_to_cpu_layout(dwd.cpu().numpy(), layout, w_layout)
            out["db"] = dbd.cpu().numpy() if dbd is not None else None
        if need_dx and "dgrad" in passes:
            dxd = torch.full(xd.shape, float("nan"), dtype=xd.dtype, device=DEV)
            _lib.check(L.b2c_conv_dgrad(ctypes.byref(desc), dyd.data_ptr(), wd.data_ptr(), dxd.data_ptr(),
                                        ws.data_ptr(), ws.numel(), stream()))
            out["dx"] = dxd.cpu().numpy()
    torch.cuda.synchronize()
    return out


def rel_l2(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    den = np.linalg.norm(ref)
    return np.linalg.norm(got - ref) / (den if den > 0 else 1.0)


def assert_parity(got, ref, dtype, what=""):
    """The stated bar: float32 rel-L2 <= 1e-5 and max-abs <= 1e-4 * max|ref|; float64 <= 1e-12."""
    got64, ref64 = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got64.shape == ref64.shape, f"{what}: shape {got64.shape} vs {ref64.shape}"
    assert np.all(np.isfinite(got64)), f"{what}: non-finite values (unwritten output?)"
    r = rel_l2(got64, ref64)
    scale = max(np.max(np.abs(ref64)), 1e-30)
    mabs = np.max(np.abs(got64 - ref64))
    if np.dtype(dtype) == np.float32:
        assert r <= 1e-5, f"{what}: rel-L2 {r:.3e} > 1e-5"
        assert mabs <= 1e-4 * scale, f"{what}: max-abs {mabs:.3e} > 1e-4*{scale:.3e}"
    else:
        assert r <= 1e-12, f"{what}: rel-L2 {r:.3e} > 1e-12"
        assert mabs <= 1e-11 * scale, f"{what}: max-abs {mabs:.3e}"
