"""Captured launch segments with an identity check.

A rows step of a given shape is captured once into a CUDA graph and replayed.  Replay is only valid while the step
would launch exactly what was captured; a configuration change between capture and replay (another arm, a toggled
feature, a different segment count) would silently replay stale work.  ``LaunchLog`` records the sequence of kernel
launches as the wrappers issue them; a ``Segment`` keeps the digest of the sequence it was captured from and
``matches`` compares a fresh recording against it.

Reference: crates/sparkflash-deepseek-forward/src/tp4_graph.rs (CUDA-graph capture of launch-only segments, replay only
when the recorded launch list is identical), crates/sparkflash-runtime (fused segments).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass


class LaunchLog:
    """Ordered record of launches.  ``ops.native`` appends (name,) tuples through ``note`` while a log is installed."""

    def __init__(self):
        self.items: list[str] = []

    def note(self, name: str) -> None:
        self.items.append(name)

    def digest(self) -> str:
        h = hashlib.sha256()
        for it in self.items:
            h.update(it.encode()); h.update(b"\0")
        return h.hexdigest()[:16]

    def __len__(self) -> int:
        return len(self.items)


_current: LaunchLog | None = None


def install(log: LaunchLog | None) -> LaunchLog | None:
    """Make ``log`` the recorder of the launch wrappers (None = stop recording); returns the previous one."""
    global _current
    prev, _current = _current, log
    return prev


def note(name: str) -> None:
    if _current is not None:
        _current.note(name)


class recording:
    """``with recording() as log:`` records every launch issued inside the block."""

    def __enter__(self) -> LaunchLog:
        self.log = LaunchLog()
        self.prev = install(self.log)
        return self.log

    def __exit__(self, *exc) -> None:
        install(self.prev)


@dataclass
class Segment:
    key: tuple
    digest: str
    launches: int
    graph: object = None

    def matches(self, log: LaunchLog) -> bool:
        return log.digest() == self.digest and len(log) == self.launches


class SegmentCache:
    """Segments by key; ``check`` raises when a fresh recording of the same key differs from the captured one."""

    def __init__(self):
        self.segments: dict[tuple, Segment] = {}

    def put(self, key: tuple, log: LaunchLog, graph=None) -> Segment:
        seg = Segment(key, log.digest(), len(log), graph)
        self.segments[key] = seg
        return seg

    def check(self, key: tuple, log: LaunchLog) -> None:
        seg = self.segments.get(key)
        if seg is None:
            raise KeyError(f"no captured segment for {key}")
        if not seg.matches(log):
            raise RuntimeError(f"launch list of {key} changed since capture: {seg.launches} launches / {seg.digest} captured, "
                               f"{len(log)} / {log.digest()} now")
