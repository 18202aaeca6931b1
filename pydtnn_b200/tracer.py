"""Step tracer: the reference's model-level event taxonomy on the device timeline.

The reference marks each layer's forward, backward, gradient all-reduce, wait and update with
``emit_event(PYDTNN_MDL_EVENT, layer.id * PYDTNN_MDL_EVENTS + <kind>)`` / ``emit_event(PYDTNN_MDL_EVENT, 0)``
(pydtnn/model.py:468-517, event numbers pydtnn/tracers/events.py:25-32) and its ``SimpleTracer`` sums host
times per event into a CSV (pydtnn/tracers/simple_tracer.py:66-83). Here an event is a pair of CUDA events on
the launching stream (device time of the kernels between them) plus an NVTX range, so the same events show up in
a timeline viewer; ``write_output`` produces the reference's CSV columns.

Tracing serialises kernels at every event (an event between two kernels stops the second from starting while
the first drains), so a traced step is a little slower than an untraced one.
"""
from collections import defaultdict

PYDTNN_MDL_EVENT = 60000001
PYDTNN_MDL_EVENTS = 5
(PYDTNN_MDL_FORWARD, PYDTNN_MDL_BACKWARD, PYDTNN_MDL_ALLREDUCE_DW, PYDTNN_MDL_WAIT_DW,
 PYDTNN_MDL_UPDATE_DW) = range(1, PYDTNN_MDL_EVENTS + 1)
_KIND_NAMES = {PYDTNN_MDL_FORWARD: "forward", PYDTNN_MDL_BACKWARD: "backward", PYDTNN_MDL_ALLREDUCE_DW: "allreduce_dw",
               PYDTNN_MDL_WAIT_DW: "wait_dw", PYDTNN_MDL_UPDATE_DW: "update_dw"}
HEADER = "Event type;Event value;Event name;Calls;Total time;Median of times\n"

# Per-operation events (pydtnn/tracers/events.py:33-70): one number per kind of operation inside a layer's hook; the
# event value is layer.id * PYDTNN_OPS_EVENTS + kind, as for the model-level events.  The names keep the reference's
# spelling although no cuDNN / cuBLAS is called here: FORWARD_CUDNN is the convolution forward pass (bias added in
# its epilogue, so FORWARD_CUDNN_SUM_BIASES never fires on its own), BACKWARD_CUDNN_DW the weight gradient (the bias
# gradient rides in the same kernel: BACKWARD_CUDNN_DB never fires on its own), BACKWARD_CUDNN_DX the input gradient;
# the CUBLAS names are the FC layer's three GEMMs.
PYDTNN_OPS_EVENT = 60000002
_OPS_NAMES = ("ALLREDUCE_DW BACKWARD_CONVGEMM BACKWARD_CUBLAS_MATMUL_DW BACKWARD_CUBLAS_MATMUL_DX BACKWARD_CUBLAS_MATVEC_DB "
              "BACKWARD_CUDNN_DB BACKWARD_CUDNN_DW BACKWARD_CUDNN_DX BACKWARD_DECONV_GEMM BACKWARD_ELTW_SUM BACKWARD_IM2COL "
              "BACKWARD_RESHAPE_DW BACKWARD_RESHAPE_DX BACKWARD_SPLIT BACKWARD_SUM_BIASES BACKWARD_TRANSPOSE_DY "
              "BACKWARD_TRANSPOSE_W COMP_DW_MATMUL COMP_DX_COL2IM COMP_DX_MATMUL FORWARD_DEPTHWISE_CONV "
              "FORWARD_POINTWISE_CONV FORWARD_CONCAT FORWARD_CONVGEMM FORWARD_CONVWINOGRAD FORWARD_CUBLAS_MATMUL "
              "FORWARD_CUDNN FORWARD_CUDNN_SUM_BIASES FORWARD_ELTW_SUM FORWARD_IM2COL FORWARD_MATMUL FORWARD_REPLICATE "
              "FORWARD_RESHAPE_W FORWARD_RESHAPE_Y FORWARD_SUM_BIASES FORWARD_TRANSPOSE_Y").split()
PYDTNN_OPS_EVENTS = len(_OPS_NAMES)
for _i, _n in enumerate(_OPS_NAMES, start=1):
    globals()["PYDTNN_OPS_" + _n] = _i
_OPS_KIND_NAMES = {i: n.lower() for i, n in enumerate(_OPS_NAMES, start=1)}


def ops_event_value(layer_id, kind):
    return layer_id * PYDTNN_OPS_EVENTS + kind


def event_value(layer_id, kind):
    return layer_id * PYDTNN_MDL_EVENTS + kind


def event_name(layer_name, kind):
    return f"{layer_name}_{_KIND_NAMES[kind]}"


class StepTracer:
    """Collects (event value, name, start, end) records; ``timer`` makes the start/end marks and ``elapsed``
    turns a pair into seconds (CUDA events by default; injectable for tests without a GPU)."""

    def __init__(self, timer=None, elapsed=None, nvtx=None):
        self.enabled = False
        self.ops = False
        self.records = []
        self.names = {}
        if timer is None:
            import torch

            def timer():
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                return e

            def elapsed(a, b):
                return a.elapsed_time(b) * 1e-3
            nvtx = torch.cuda.nvtx
        self._timer, self._elapsed, self._nvtx = timer, elapsed, nvtx

    def enable_tracing(self, ops=False):
        self.enabled = True
        self.ops = bool(ops)

    def disable_tracing(self):
        self.enabled = False

    def region(self, layer, kind):
        """Context manager around one event of one layer (a no-op object when tracing is off)."""
        return _Region(self, layer, kind) if self.enabled else _NULL

    def op_region(self, layer, kind):
        """The same for one operation inside a layer's hook (PYDTNN_OPS_*); off unless ``enable_tracing(ops=True)``."""
        return _Region(self, layer, kind, ops=True) if self.enabled and self.ops else _NULL

    def summary(self):
        """{event value: (name, calls, total seconds, median seconds)}; synchronises the device."""
        return self._summary(lambda key: not isinstance(key, tuple))

    def ops_summary(self):
        """The per-operation events: {event value: (name, calls, total seconds, median seconds)}."""
        return {k[1]: v for k, v in self._summary(lambda key: isinstance(key, tuple)).items()}

    def _summary(self, keep):
        times = defaultdict(list)
        for value, start, end in self.records:
            if keep(value):
                times[value].append(self._elapsed(start, end))
        out = {}
        for value, t in times.items():
            t.sort()
            out[value] = (self.names[value], len(t), sum(t), t[len(t) // 2])
        return out

    def write_output(self, filename):
        with open(filename, "w") as f:
            f.write(HEADER)
            for value, (name, calls, total, median) in sorted(self.summary().items()):
                f.write(f"Model;{value};{name};{calls};{total};{median}\n")
            for value, (name, calls, total, median) in sorted(self.ops_summary().items()):
                f.write(f"Operations;{value};{name};{calls};{total};{median}\n")


class _Region:
    def __init__(self, tracer, layer, kind, ops=False):
        self.t = tracer
        if ops:
            self.value = ("ops", ops_event_value(layer.id, kind))      # kept apart from the model-level numbers
            self.name = f"{layer.canonical_name_with_id}_{_OPS_KIND_NAMES[kind]}"
        else:
            self.value = event_value(layer.id, kind)
            self.name = event_name(layer.canonical_name_with_id, kind)

    def __enter__(self):
        if self.t._nvtx is not None:
            self.t._nvtx.range_push(self.name)
        self.start = self.t._timer()

    def __exit__(self, *exc):
        self.t.records.append((self.value, self.start, self.t._timer()))
        self.t.names[self.value] = self.name
        if self.t._nvtx is not None:
            self.t._nvtx.range_pop()
        return False


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NULL = _Null()
