"""Trace controller (reference tests: crates/sparkflash-trace unit tests for controller/scope/export)."""
import gzip
import json

import pytest

from sparkflash_b200.utils.trace import ALL, BIT, SCOPES, TraceController, percentile


def test_arm_tick_and_filters():
    t = TraceController()
    assert len(SCOPES) == 16 and t.active_mask() == 0
    m = t.parse_scopes("moe, attention|seam")
    assert m == (1 << BIT["moe"]) | (1 << BIT["attention"]) | (1 << BIT["seam"]) and t.parse_scopes("all") == ALL
    with pytest.raises(ValueError):
        t.parse_scopes("nope")
    t.arm(m, 2)
    with t.span("moe", "gate_up", layer=3):
        pass
    with t.span("head", "lm_head"):        # not armed: no event
        pass
    t.tick_step(); assert t.active("moe")
    t.tick_step(); assert not t.active("moe") and t.status()["steps_left"] == 0
    assert [e[1] for e in t.events] == ["gate_up"]
    t.arm(ALL, 5); t.set_request_filter(["r1"])
    assert t.is_request_traced("r1") and not t.is_request_traced("r2")
    t.set_request_filter(None); assert t.is_request_traced("r2")


def test_export_and_summary(tmp_path):
    t = TraceController()
    t.arm(ALL, 100)
    for i in range(10):
        with t.span("decode", "step", i=i):
            pass
    dev = [{"t_ns": 1000, "scope": "moe", "tag": 7, "phase": 0, "smid": 3, "aux": 0},
           {"t_ns": 4000, "scope": "moe", "tag": 7, "phase": 1, "smid": 3, "aux": 0},
           {"t_ns": 5000, "scope": "seam", "tag": 1, "phase": 2, "smid": 0, "aux": 0}]
    doc = t.export_chrome(dev)
    xs = [e for e in doc["traceEvents"] if e["pid"] == 1]
    assert xs[0]["ph"] == "X" and abs(xs[0]["dur"] - 3.0) < 1e-9 and xs[1]["ph"] == "i"
    s = t.summary()["decode/step"]
    assert s["count"] == 10 and s["p50_us"] <= s["p99_us"]
    p = tmp_path / "t.json.gz"
    t.write(str(p))
    assert len(json.loads(gzip.open(p).read())["traceEvents"]) == 10
    assert percentile([1.0, 2.0, 3.0, 4.0], 50) == 2.5 and percentile([], 99) == 0.0


@pytest.mark.gpu
def test_device_ring_records_ordered_global_timer_events():
    import torch
    t = TraceController()
    t.attach_device_ring(256)
    t.arm(t.parse_scopes("moe"), 10)
    x = torch.zeros(1 << 20, device="cuda")
    for i in range(4):
        t.mark("moe", i, 0)
        x.add_(1.0)
        t.mark("moe", i, 1)
        t.mark("seam", i, 2)        # not armed: dropped on the device
    torch.cuda.synchronize()
    ev = t.drain_device()
    assert len(ev) == 8 and [e["phase"] for e in ev] == [0, 1] * 4
    ts = [e["t_ns"] for e in ev]
    assert ts == sorted(ts) and ts[-1] > ts[0]
    assert t.drain_device() == []
    doc = t.export_chrome(ev)
    assert sum(1 for e in doc["traceEvents"] if e["ph"] == "X") == 4
