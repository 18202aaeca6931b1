"""Where the warp roles of the tensor-core convolution kernel spend their time, for one layer shape.

    python pydtnn_b200/csrc/build.py --variant profile
    python pydtnn_b200/csrc/role_profile.py n,h,w,ci,co,k,stride,pad [fprop|dgrad|wgrad|fprop+stats] ...

Loads ``pydtnn_b200/libb2c_profile.so`` (not the product library), runs the pass a few times and prints, per role
of CTA 0, the share of the call's wall time spent in each state.  Development aid; needs a GPU."""
import ctypes
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

SLOTS = {0: "producer: waits for a free stage", 14: "producer: issues TMA", 1: "MMA: waits for a drained accumulator",
         3: "MMA: waits for the transform", 4: "MMA: issues", 5: "transform: waits for TMA data", 6: "transform: works",
         7: "drain: waits for a finished chunk", 8: "drain: tensor-memory loads, adds, epilogue arithmetic",
         10: "drain: waits for a free staging slab", 9: "drain: staging writes, fence, store issue (or the scattered-store epilogue)",
         11: "drain: batch statistics"}


def main():
    import torch
    from pydtnn_b200 import _lib
    _lib.LIB_PATH = os.path.join(ROOT, "pydtnn_b200", "libb2c_profile.so")
    L = _lib.lib()
    L.b2c_debug_prof.argtypes = [ctypes.c_void_p, ctypes.c_int]
    args = sys.argv[1:]
    if not args:
        raise SystemExit(__doc__)
    jobs = []
    while args:
        shape = tuple(int(v) for v in args.pop(0).split(","))
        what = args.pop(0) if args and "," not in args[0] else "fprop"
        jobs.append((shape, what))
    st = torch.cuda.current_stream().cuda_stream
    for (n, h, w, ci, co, k, stride, pad), what in jobs:
        ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        d = _lib.ConvDesc(0, 0, _lib.W_KRSC, 0, n, h, w, ci, co, k, k, pad, pad, stride, stride, 1, 1)
        nb = max(L.b2c_conv_workspace_bytes(ctypes.byref(d), q) for q in range(3))
        ws = torch.empty(max(nb, 256), dtype=torch.uint8, device="cuda")
        x, wt = torch.randn((n, h, w, ci), device="cuda"), torch.randn((co, k, k, ci), device="cuda")
        y, dw = torch.randn((n, ho, wo, co), device="cuda"), torch.empty((co, k, k, ci), device="cuda")
        sb = L.b2c_conv_stats_bytes(ctypes.byref(d))
        stats = torch.empty(max(sb, 16), dtype=torch.uint8, device="cuda")

        def call():
            if what == "fprop":
                return L.b2c_conv_fprop(ctypes.byref(d), x.data_ptr(), wt.data_ptr(), None, None, 0, y.data_ptr(), ws.data_ptr(), ws.numel(), st)
            if what == "fprop+stats":
                return L.b2c_conv_fprop_stats(ctypes.byref(d), x.data_ptr(), wt.data_ptr(), None, y.data_ptr(), stats.data_ptr(), sb,
                                              ws.data_ptr(), ws.numel(), st)
            if what == "dgrad":
                return L.b2c_conv_dgrad(ctypes.byref(d), y.data_ptr(), wt.data_ptr(), x.data_ptr(), ws.data_ptr(), ws.numel(), st)
            return L.b2c_conv_wgrad(ctypes.byref(d), x.data_ptr(), y.data_ptr(), dw.data_ptr(), None, ws.data_ptr(), ws.numel(), st)
        for _ in range(2):
            _lib.check(call())
        buf = (ctypes.c_longlong * 32)()
        L.b2c_debug_prof(buf, 1)
        iters = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        L.b2c_debug_prof(buf, 1)
        mhz = torch.cuda.clock_rate() if hasattr(torch.cuda, "clock_rate") else 1965     # SM clock in MHz
        cyc = ms * 1e-3 * mhz * 1e6
        print(f"{(n, h, w, ci, co, k, stride, pad)} {what}: {ms * 1e3:.1f} us per call")
        for slot, name in SLOTS.items():
            print(f"    {100.0 * buf[slot] / iters / cyc:5.1f} %  {name}")


if __name__ == "__main__":
    main()
