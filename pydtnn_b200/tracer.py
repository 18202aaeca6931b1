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


def event_value(layer_id, kind):
    return layer_id * PYDTNN_MDL_EVENTS + kind


def event_name(layer_name, kind):
    return f"{layer_name}_{_KIND_NAMES[kind]}"


class StepTracer:
    """Collects (event value, name, start, end) records; ``timer`` makes the start/end marks and ``elapsed``
    turns a pair into seconds (CUDA events by default; injectable for tests without a GPU)."""

    def __init__(self, timer=None, elapsed=None, nvtx=None):
        self.enabled = False
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

    def enable_tracing(self):
        self.enabled = True

    def disable_tracing(self):
        self.enabled = False

    def region(self, layer, kind):
        """Context manager around one event of one layer (a no-op object when tracing is off)."""
        return _Region(self, layer, kind) if self.enabled else _NULL

    def summary(self):
        """{event value: (name, calls, total seconds, median seconds)}; synchronises the device."""
        times = defaultdict(list)
        for value, start, end in self.records:
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


class _Region:
    def __init__(self, tracer, layer, kind):
        self.t, self.value = tracer, event_value(layer.id, kind)
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
