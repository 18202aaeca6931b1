"""Step tracer without a GPU: event numbering of the reference (pydtnn/tracers/events.py:25-32, pydtnn/model.py:468)
and the CSV layout of its SimpleTracer (pydtnn/tracers/simple_tracer.py:70-83), with an injected clock."""
import itertools

from pydtnn_b200 import tracer as tr


class _L:
    def __init__(self, lid, name):
        self.id, self.canonical_name_with_id = lid, f"{lid}_{name}"


def test_event_values_follow_the_reference_numbering():
    assert tr.PYDTNN_MDL_EVENT == 60000001 and tr.PYDTNN_MDL_EVENTS == 5
    assert (tr.PYDTNN_MDL_FORWARD, tr.PYDTNN_MDL_BACKWARD, tr.PYDTNN_MDL_ALLREDUCE_DW, tr.PYDTNN_MDL_WAIT_DW,
            tr.PYDTNN_MDL_UPDATE_DW) == (1, 2, 3, 4, 5)
    assert tr.event_value(7, tr.PYDTNN_MDL_BACKWARD) == 37


def test_regions_are_summed_per_event_and_written_as_the_reference_csv(tmp_path):
    clock = itertools.count()
    t = tr.StepTracer(timer=lambda: next(clock), elapsed=lambda a, b: float(b - a), nvtx=None)
    conv, fc = _L(1, "Conv2D"), _L(2, "FC")
    with t.region(conv, tr.PYDTNN_MDL_FORWARD):       # tracing is off: nothing is recorded
        pass
    assert t.records == []
    t.enable_tracing()
    for _ in range(3):
        with t.region(conv, tr.PYDTNN_MDL_FORWARD):
            next(clock)
        with t.region(fc, tr.PYDTNN_MDL_FORWARD):
            pass
    with t.region(conv, tr.PYDTNN_MDL_BACKWARD):
        pass
    s = t.summary()
    assert s[6] == ("1_Conv2D_forward", 3, 6.0, 2.0)
    assert s[11] == ("2_FC_forward", 3, 3.0, 1.0)
    assert s[7][0:2] == ("1_Conv2D_backward", 1)
    out = tmp_path / "trace.csv"
    t.write_output(out)
    lines = out.read_text().splitlines()
    assert lines[0] == "Event type;Event value;Event name;Calls;Total time;Median of times"
    assert lines[1].startswith("Model;6;1_Conv2D_forward;3;6.0;2.0")
    assert len(lines) == 4
