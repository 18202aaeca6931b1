"""The allocation-free batch-norm entry point against the regular one, through the C ABI.

``b2c_bn_train_forward_static`` serves hosts that pre-allocate all device memory into their own pool
and then forbid allocation, and that have no scratch buffer to lend: its reduction scratch is a fixed
array inside the library.  The test calls it twice in a row (the array keeps the first call's
contents) and compares every output with ``b2c_bn_train_forward`` on the same inputs, within the
float32 / float64 tolerances the other parity tests use.  It also checks the size limit.
Collected last on purpose, so a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

from pydtnn_b200 import _lib
from tests.gpu_util import DEV, assert_parity, dev, stream

pytestmark = pytest.mark.gpu


def _run(fn_static, x, gamma, beta, layout, relu, dtype):
    L = _lib.lib()
    dt = _lib.dtype_code(dtype)
    lay = _lib.LAYOUT_NHWC if layout == "NHWC" else _lib.LAYOUT_NCHW
    if layout == "NHWC":
        n, h, w, c = x.shape
    else:
        n, c, h, w = x.shape
    xd, gd, bd = dev(x), dev(gamma), dev(beta)
    rm = torch.full((c,), 0.25, dtype=xd.dtype, device=DEV)
    rv = torch.full((c,), 0.75, dtype=xd.dtype, device=DEV)
    y = torch.full_like(xd, float("nan"))
    sm, si = torch.empty_like(rm), torch.empty_like(rm)
    if fn_static:
        rc = L.b2c_bn_train_forward_static(dt, lay, n, c, h * w, xd.data_ptr(), gd.data_ptr(), bd.data_ptr(),
                                           rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, int(relu), y.data_ptr(),
                                           sm.data_ptr(), si.data_ptr(), stream())
    else:
        scratch = torch.empty(1200 * c, dtype=torch.float64, device=DEV)
        rc = L.b2c_bn_train_forward(dt, lay, n, c, h * w, xd.data_ptr(), gd.data_ptr(), bd.data_ptr(), rm.data_ptr(),
                                    rv.data_ptr(), 0.9, 1e-5, int(relu), y.data_ptr(), sm.data_ptr(), si.data_ptr(),
                                    scratch.data_ptr(), scratch.numel() * 8, stream())
    _lib.check(rc)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (y, sm, si, rm, rv)]


@pytest.mark.parametrize("layout,dtype,shape", [("NHWC", "float32", (8, 28, 28, 128)), ("NHWC", "float32", (4, 7, 7, 2048)),
                                                ("NCHW", "float32", (4, 24, 9, 9)), ("NHWC", "float64", (4, 6, 6, 20)),
                                                # 2048 channels on the generic reduction: 64 chunks x 2 x 2048 doubles, the whole array
                                                ("NCHW", "float32", (2, 2048, 8, 8)), ("NHWC", "float64", (2, 8, 8, 2048))])
def test_static_scratch_entry_point_matches_regular_one_twice(layout, dtype, shape):
    rng = np.random.Generator(np.random.PCG64(21))
    c = shape[3] if layout == "NHWC" else shape[1]
    for call in range(2):                       # second call runs on top of the first call's leftovers
        x = (rng.standard_normal(shape) * (1.0 + call) + 0.5 * call).astype(dtype)
        gamma, beta = rng.standard_normal(c).astype(dtype), rng.standard_normal(c).astype(dtype)
        want = _run(False, x, gamma, beta, layout, relu=bool(call), dtype=dtype)
        got = _run(True, x, gamma, beta, layout, relu=bool(call), dtype=dtype)
        for name, g, w in zip(("y", "save_mean", "save_inv_std", "running_mean", "running_var"), got, want):
            assert_parity(g, w, dtype, f"call {call} {name}")


def test_static_scratch_entry_point_against_the_cpu_oracle():
    """One direct comparison with the CPU restatement of the reference's batch norm (not only with the regular
    entry point): y, the running averages and the saved mean."""
    from oracle import aux_oracle as ao
    rng = np.random.Generator(np.random.PCG64(5))
    shape, c = (8, 14, 14, 64), 64
    x = rng.standard_normal(shape).astype(np.float32) * 2.0 + 0.3
    gamma, beta = rng.standard_normal(c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
    y, sm, si, rm, rv = _run(True, x, gamma, beta, "NHWC", relu=False, dtype="float32")
    y_ref, (std, _), rm_ref, rv_ref = ao.bn_train_forward(x.astype(np.float64), gamma.astype(np.float64), beta.astype(np.float64),
                                                          np.full(c, 0.25), np.full(c, 0.75), 0.9, 1e-5, "NHWC")
    assert_parity(y, y_ref, np.float32, "y")
    assert_parity(rm, rm_ref, np.float32, "running_mean")
    assert_parity(rv, rv_ref, np.float32, "running_var")
    assert_parity(si, 1.0 / std, np.float32, "save_inv_std")
    assert_parity(sm, x.astype(np.float64).reshape(-1, c).mean(axis=0), np.float32, "save_mean")


def test_static_scratch_entry_point_allocates_nothing():
    """The property the entry point exists for: with every tensor in place and the first call done, further calls
    leave the device's free memory exactly where it was (cudaMemGetInfo before and after)."""
    L = _lib.lib()
    n, h, w, c = 8, 28, 28, 256
    x = torch.randn((n, h, w, c), device=DEV)
    y = torch.empty_like(x)
    gamma, beta = torch.ones(c, device=DEV), torch.zeros(c, device=DEV)
    rm, rv, sm, si = (torch.zeros(c, device=DEV) for _ in range(4))

    def call():
        _lib.check(L.b2c_bn_train_forward_static(_lib.F32, _lib.LAYOUT_NHWC, n, c, h * w, x.data_ptr(), gamma.data_ptr(),
                                                 beta.data_ptr(), rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, 1, y.data_ptr(),
                                                 sm.data_ptr(), si.data_ptr(), stream()))
    call()                                      # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)


def test_static_scratch_entry_point_rejects_sizes_beyond_its_array():
    L = _lib.lib()
    c = 2049
    x = torch.zeros((1, 1, 1, c), device=DEV)
    v = torch.zeros((c,), device=DEV)
    rc = L.b2c_bn_train_forward_static(0, 0, 1, c, 1, x.data_ptr(), v.data_ptr(), v.data_ptr(), v.data_ptr(), v.data_ptr(),
                                       0.9, 1e-5, 0, x.data_ptr(), v.data_ptr(), v.data_ptr(), stream())
    assert rc == -8
    assert b"capacity" in L.b2c_status_string(rc)
    with pytest.raises(_lib.B2CError):
        _lib.check(rc)
