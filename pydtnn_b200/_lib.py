"""ctypes binding of ``libb2c.so`` (the C ABI declared in ``include/b2c.h``).

There is no fallback: if the shared library is missing or a call returns a negative status an
exception is raised, mirroring how the reference's cuDNN/NCCL wrappers raise on a non-zero
status (pydtnn/backends/gpu/libs/libcudnn.py:306-323).
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_int, c_int32, c_int64, c_size_t, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb2c.so")

LAYOUT_NHWC, LAYOUT_NCHW = 0, 1
F32, F64 = 0, 1
W_CRSK, W_KCRS, W_KRSC = 0, 1, 2
PASS_FPROP, PASS_DGRAD, PASS_WGRAD = 0, 1, 2
ENGINE_AUTO, ENGINE_FMA, ENGINE_TENSOR = 0, 1, 2


class B2CError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        super().__init__(f"b2c status {status}: {detail}")


class ConvDesc(Structure):
    _fields_ = [(k, c_int32) for k in ("layout", "dtype", "w_layout", "engine", "n", "h", "w", "ci", "co", "kh",
                                       "kw", "vpad", "hpad", "vstr", "hstr", "vdil", "hdil")]


class BnParams(Structure):
    _fields_ = [("mean", c_void_p), ("inv_std", c_void_p), ("gamma", c_void_p), ("beta", c_void_p)]


# name -> (restype, argtypes); every symbol include/b2c.h declares
PROTOTYPES = {
    "b2c_status_string": (c_char_p, [c_int]),
    "b2c_last_cuda_error": (c_char_p, []),
    "b2c_version": (c_int, []),
    "b2c_launch_count": (ctypes.c_uint64, []),
    "b2c_check_device_status": (c_int, [POINTER(c_int)]),
    "b2c_conv_workspace_bytes": (c_size_t, [POINTER(ConvDesc), c_int]),
    "b2c_conv_engine_for": (c_int, [POINTER(ConvDesc), c_int]),
    "b2c_conv_fprop": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, POINTER(BnParams), c_int, c_void_p,
                               c_void_p, c_size_t, c_void_p]),
    "b2c_conv_stats_bytes": (c_size_t, [POINTER(ConvDesc)]),
    "b2c_conv_fprop_stats": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                     c_void_p, c_size_t, c_void_p]),
    "b2c_bn_train_forward_prestats": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_double, c_double, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b2c_conv_dgrad": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b2c_conv_wgrad": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                               c_void_p]),
    "b2c_conv_keeps_lowered_input": (c_int, [POINTER(ConvDesc)]),
    "b2c_conv_wgrad_lowered": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                       c_void_p]),
    "b2c_conv_index_map": (c_int, [POINTER(ConvDesc), c_void_p, c_void_p]),
    "b2c_fc_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "b2c_fc_forward": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_size_t, c_void_p]),
    "b2c_fc_backward": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_size_t, c_void_p]),
    "b2c_bn_train_forward": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_double, c_double, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_size_t, c_void_p]),
    "b2c_bn_train_forward_static": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_double, c_double, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_bn_train_forward_residual": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_double, c_double, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_size_t, c_void_p]),
    "b2c_bn_train_backward": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b2c_bn_inference": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, c_void_p, c_void_p]),
    "b2c_relu_forward": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "b2c_relu_backward": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_add_inplace": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "b2c_selftest_bounded_wait": (c_int, [c_int64, c_void_p]),
    "b2c_add_relu": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_add_relu_backward": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_pool_forward": (c_int, [c_int] * 15 + [c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_pool_backward": (c_int, [c_int] * 15 + [c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_softmax_forward": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b2c_softmax_backward": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_cce_forward_backward": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_double, c_void_p, c_void_p,
                                         c_void_p, c_void_p]),
    "b2c_cce_totals": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2c_bn_inv_std": (c_int, [c_int, c_int, c_void_p, c_double, c_void_p, c_void_p]),
    "b2c_probe_fma": (c_int, [c_int, c_int, c_int, c_void_p, POINTER(c_double), c_void_p]),
    "b2c_sgd_update": (c_int, [c_int, c_int64, c_void_p, c_void_p, c_void_p, c_double, c_double, c_double, c_int,
                               c_void_p]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built (run ``__graft_entry__.build()``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B2CError(-100, f"{LIB_PATH} is missing: build the CUDA extension first "
                                 f"(python pydtnn_b200/csrc/build.py); there is no CPU fallback")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status):
    """Raise B2CError for a negative status (the library's error convention)."""
    if status < 0:
        L = lib()
        msg = L.b2c_status_string(status).decode()
        if status == -7:
            msg += " -- " + L.b2c_last_cuda_error().decode()
        raise B2CError(status, msg)
    return status


def dtype_code(np_dtype):
    import numpy as np
    return {np.dtype(np.float32): F32, np.dtype(np.float64): F64}[np.dtype(np_dtype)]
