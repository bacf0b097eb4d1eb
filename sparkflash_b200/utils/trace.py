"""Scope-mask tracing: a controller that arms named scopes for a number of engine steps, CPU spans, GPU
events from a host-mapped ring stamped with the device's global timer, Chrome-trace export and per-scope
percentiles.  Reference: crates/sparkflash-trace/src/controller.rs:55-264 (arm / tick_step / request filter),
scope.rs:28-224 (16 named scopes), export.rs:30-225 (Chrome JSON, p50/p99).
"""
from __future__ import annotations

import contextlib
import ctypes
import gzip
import json
import threading
import time
from ctypes import c_void_p

SCOPES = ["step", "sched", "prefill", "decode", "attention", "moe", "seam", "collective", "head", "sample", "draft",
          "kv", "engram", "vision", "io", "api"]
BIT = {n: i for i, n in enumerate(SCOPES)}
ALL = (1 << len(SCOPES)) - 1


class TraceController:
    def __init__(self, capacity: int = 1 << 16):
        self._lock = threading.Lock()
        self.mask = 0
        self.steps_left = 0
        self.request_filter: set[str] | None = None
        self.events: list[tuple] = []          # (scope, name, t0_ns, t1_ns, tid, args)
        self.capacity = capacity
        self._ring = None                      # (host_ptr, dev_ptr, capacity) once a device ring is attached
        self._ring_read = 0
        self._t_base: tuple[int, int] | None = None   # (host ns, device ns) pairing for the export

    # ---- control ------------------------------------------------------------------------------------
    @staticmethod
    def parse_scopes(text) -> int:
        if isinstance(text, int):
            return text & ALL
        m = 0
        for part in str(text).replace("|", ",").split(","):
            part = part.strip()
            if not part:
                continue
            if part == "all":
                m |= ALL
            elif part in BIT:
                m |= 1 << BIT[part]
            elif part.isdigit() or part.startswith("0x"):
                m |= int(part, 0) & ALL
            else:
                raise ValueError(f"unknown trace scope {part!r}; known: {SCOPES}")
        return m

    def arm(self, mask: int, steps: int) -> None:
        with self._lock:
            self.mask, self.steps_left = mask & ALL, max(0, steps)
            self._mirror()

    def tick_step(self) -> None:
        """Called once per engine step: disarms when the armed step count runs out."""
        with self._lock:
            if self.steps_left > 0:
                self.steps_left -= 1
                if self.steps_left == 0:
                    self.mask = 0
                    self._mirror()

    def active_mask(self) -> int:
        return self.mask

    def active(self, scope: str) -> bool:
        return bool((self.mask >> BIT[scope]) & 1)

    def set_request_filter(self, request_ids: list[str] | None) -> None:
        self.request_filter = set(request_ids) if request_ids else None

    def is_request_traced(self, request_id: str) -> bool:
        return self.mask != 0 and (self.request_filter is None or request_id in self.request_filter)

    def status(self) -> dict:
        return {"mask": self.mask, "scopes": [s for s in SCOPES if self.active(s)], "steps_left": self.steps_left,
                "events": len(self.events), "device_ring": self._ring is not None}

    # ---- CPU events ---------------------------------------------------------------------------------------
    @contextlib.contextmanager
    def span(self, scope: str, name: str, **args):
        if not self.active(scope):
            yield
            return
        t0 = time.monotonic_ns()
        try:
            yield
        finally:
            self._push((scope, name, t0, time.monotonic_ns(), threading.get_ident() & 0xFFFF, args))

    def instant(self, scope: str, name: str, **args) -> None:
        if self.active(scope):
            t = time.monotonic_ns()
            self._push((scope, name, t, t, threading.get_ident() & 0xFFFF, args))

    def _push(self, ev) -> None:
        with self._lock:
            if len(self.events) >= self.capacity:
                del self.events[:self.capacity // 2]
            self.events.append(ev)

    # ---- device ring ----------------------------------------------------------------------------------------
    def attach_device_ring(self, capacity: int = 1 << 14) -> None:
        from .. import _lib
        L = _lib.cuda()
        host, dev = c_void_p(), c_void_p()
        rc = L.sfb_trace_ring_create(ctypes.c_longlong(capacity), ctypes.byref(host), ctypes.byref(dev))
        if rc:
            raise RuntimeError(f"trace ring allocation failed: cuda error {rc}")
        self._ring = (host.value, dev.value, capacity)
        self._mirror()

    def _mirror(self) -> None:
        if self._ring is not None:
            ctypes.c_uint64.from_address(self._ring[0]).value = self.mask

    def mark(self, scope: str, tag: int, phase: int, aux: int = 0, stream: int = 0) -> None:
        """Enqueue a device-side event (phase 0 begin, 1 end, 2 instant) on ``stream``."""
        if self._ring is None or not self.active(scope):
            return
        from .. import _lib
        _lib.cuda().sfb_trace_mark(c_void_p(self._ring[1]), ctypes.c_uint(BIT[scope]), ctypes.c_uint(tag), ctypes.c_uint(phase),
                                   ctypes.c_uint64(aux), c_void_p(stream))

    def drain_device(self) -> list[dict]:
        """Events pushed since the last drain (synchronise the stream first)."""
        if self._ring is None:
            return []
        host, _, cap = self._ring
        head = ctypes.c_uint64.from_address(host + 8).value
        out = []
        start = max(self._ring_read, head - cap)
        for i in range(start, head):
            base = host + 64 + (i % cap) * 32
            t = ctypes.c_uint64.from_address(base).value
            scope_bit, tag, phase, smid = (ctypes.c_uint32.from_address(base + 8 + 4 * k).value for k in range(4))
            out.append({"t_ns": t, "scope": SCOPES[scope_bit] if scope_bit < len(SCOPES) else str(scope_bit), "tag": tag,
                        "phase": phase, "smid": smid, "aux": ctypes.c_uint64.from_address(base + 24).value})
        self._ring_read = head
        return out

    # ---- export -------------------------------------------------------------------------------------------------
    def export_chrome(self, device_events: list[dict] | None = None) -> dict:
        ev = []
        with self._lock:
            cpu = list(self.events)
        for scope, name, t0, t1, tid, args in cpu:
            ev.append({"name": name, "cat": scope, "ph": "X", "ts": t0 / 1e3, "dur": max(0.001, (t1 - t0) / 1e3), "pid": 0, "tid": tid, "args": args})
        dev = device_events if device_events is not None else self.drain_device()
        open_ev: dict[tuple, int] = {}
        for d in dev:
            key = (d["scope"], d["tag"])
            if d["phase"] == 0:
                open_ev[key] = d["t_ns"]
            elif d["phase"] == 1 and key in open_ev:
                t0 = open_ev.pop(key)
                ev.append({"name": f"{d['scope']}:{d['tag']}", "cat": d["scope"], "ph": "X", "ts": t0 / 1e3, "dur": max(0.001, (d["t_ns"] - t0) / 1e3), "pid": 1, "tid": 0, "args": {"smid": d["smid"]}})
            else:
                ev.append({"name": f"{d['scope']}:{d['tag']}", "cat": d["scope"], "ph": "i", "s": "t", "ts": d["t_ns"] / 1e3, "pid": 1, "tid": 0})
        return {"traceEvents": ev, "displayTimeUnit": "ns", "metadata": {"scopes": SCOPES}}

    def write(self, path: str) -> None:
        data = json.dumps(self.export_chrome()).encode()
        if path.endswith(".gz"):
            with gzip.open(path, "wb") as f:
                f.write(data)
        else:
            with open(path, "wb") as f:
                f.write(data)

    def summary(self) -> dict:
        """Per (scope, name): count, p50, p99, total - in microseconds."""
        groups: dict[tuple, list[float]] = {}
        with self._lock:
            for scope, name, t0, t1, _, _ in self.events:
                groups.setdefault((scope, name), []).append((t1 - t0) / 1e3)
        out = {}
        for (scope, name), xs in groups.items():
            xs.sort()
            out[f"{scope}/{name}"] = {"count": len(xs), "p50_us": percentile(xs, 50), "p99_us": percentile(xs, 99), "total_us": sum(xs)}
        return out


def percentile(sorted_xs: list[float], p: float) -> float:
    if not sorted_xs:
        return 0.0
    k = (len(sorted_xs) - 1) * p / 100.0
    lo, hi = int(k), min(int(k) + 1, len(sorted_xs) - 1)
    return sorted_xs[lo] + (sorted_xs[hi] - sorted_xs[lo]) * (k - lo)
