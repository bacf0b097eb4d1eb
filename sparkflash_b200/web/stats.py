"""Serving telemetry with a bounded history.

A sampler thread outside the inference path reads the server's ``/v1/cluster/stats`` once per interval and folds the
answer into an in-memory ring.  A graph asks for a window and a number of points; the ring is down-sampled by bucket
means, so a day's view is a few hundred points.  A JSON snapshot is written only while the server is idle (nothing
running or waiting) and at most once per flush interval: serving never waits for this module's disk writes.

Reference behaviour: crates/sparkflash-web/src/stats.rs (sampler, ring, down-sampling, idle-only persistence).
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from collections import deque
from pathlib import Path
from typing import Callable

FIELDS = ("running", "waiting", "tokens_total", "requests_total", "tok_s", "kv_used", "step_ms")


def http_source(url: str) -> Callable[[], dict]:
    def read() -> dict:
        with urllib.request.urlopen(url.rstrip("/") + "/v1/cluster/stats", timeout=2) as r:
            return json.loads(r.read())
    return read


def flatten(raw: dict) -> dict:
    """The counters a graph needs from a cluster-stats answer (absent ones read 0)."""
    sched = raw.get("scheduler", raw)
    return {"running": float(sched.get("running", raw.get("running", 0)) or 0), "waiting": float(sched.get("waiting", raw.get("waiting", 0)) or 0),
            "tokens_total": float(raw.get("generated_tokens", raw.get("tokens_total", 0)) or 0),
            "requests_total": float(raw.get("requests_finished", raw.get("requests_total", 0)) or 0),
            "kv_used": float(raw.get("kv_pages_used", raw.get("kv_used", 0)) or 0), "step_ms": float(raw.get("step_ms_p50", raw.get("step_ms", 0)) or 0)}


class History:
    def __init__(self, interval_s: float = 2.0, history_s: float = 86400.0, flush_s: float = 300.0, path: str | Path | None = None,
                 clock: Callable[[], float] = time.time):
        self.interval_s, self.flush_s, self.clock = interval_s, flush_s, clock
        self.ring: deque = deque(maxlen=max(2, int(history_s / max(interval_s, 1e-3))))
        self.path = Path(path) if path else None
        self.errors = 0
        self.last_error: str | None = None
        self._last_flush = 0.0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        if self.path and self.path.is_file():
            try:
                for row in json.loads(self.path.read_text()).get("samples", []):
                    self.ring.append(row)
            except (json.JSONDecodeError, OSError):
                pass

    # ---- sampling ------------------------------------------------------------------------------------------------
    def add(self, raw: dict) -> dict:
        s = flatten(raw)
        s["t"] = self.clock()
        with self._lock:
            prev = self.ring[-1] if self.ring else None
            dt = s["t"] - prev["t"] if prev else 0.0
            # the rate comes from the counter, so a sample missed in between loses nothing; a counter that went
            # backwards means the server restarted
            s["tok_s"] = max(0.0, s["tokens_total"] - prev["tokens_total"]) / dt if prev and dt > 0 and s["tokens_total"] >= prev["tokens_total"] else 0.0
            self.ring.append(s)
        self._maybe_flush(s)
        return s

    def sample(self, source: Callable[[], dict]) -> dict | None:
        try:
            return self.add(source())
        except Exception as e:                                     # noqa: BLE001 - the server being down is a normal state
            self.errors += 1
            self.last_error = f"{type(e).__name__}: {e}"
            return None

    def start(self, source: Callable[[], dict]) -> "History":
        def loop():
            while not self._stop.wait(self.interval_s):
                self.sample(source)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)

    # ---- persistence ---------------------------------------------------------------------------------------------
    def _maybe_flush(self, s: dict) -> None:
        if not self.path or s["running"] or s["waiting"] or s["t"] - self._last_flush < self.flush_s:
            return
        self._last_flush = s["t"]
        with self._lock:
            rows = list(self.ring)
        tmp = self.path.with_name(self.path.name + ".tmp")
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp.write_text(json.dumps({"samples": rows}))
        tmp.replace(self.path)

    # ---- queries -------------------------------------------------------------------------------------------------
    def window(self, seconds: float, points: int = 300) -> list[dict]:
        """Samples of the last ``seconds``, reduced to at most ``points`` buckets (mean of gauges and rates, last value
        of counters)."""
        now = self.clock()
        with self._lock:
            rows = [r for r in self.ring if r["t"] >= now - seconds]
        if len(rows) <= points or points < 1:
            return rows
        out = []
        per = len(rows) / points
        for b in range(points):
            chunk = rows[int(b * per):max(int((b + 1) * per), int(b * per) + 1)]
            agg = {"t": chunk[-1]["t"]}
            for f in FIELDS:
                agg[f] = chunk[-1][f] if f.endswith("_total") else sum(c[f] for c in chunk) / len(chunk)
            out.append(agg)
        return out

    def summary(self, seconds: float = 60.0) -> dict:
        rows = self.window(seconds, points=0)
        if not rows:
            return {"samples": 0, "errors": self.errors, "last_error": self.last_error}
        return {"samples": len(rows), "tok_s_mean": sum(r["tok_s"] for r in rows) / len(rows), "tok_s_peak": max(r["tok_s"] for r in rows),
                "running_peak": max(r["running"] for r in rows), "waiting_peak": max(r["waiting"] for r in rows), "errors": self.errors,
                "last_error": self.last_error}
