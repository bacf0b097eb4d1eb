"""In-step agreement of a serving group.

Every rank runs the same deterministic step from the same tick.  ``GroupLanes`` gives each rank a running digest of
what it executed (tick number, rows, lanes, positions, sampled tokens); the leader compares the digests the followers
report and declares the group out of step on the first difference - the fail-stop signal for "one rank took another
branch", which no collective would catch by itself.

Reference: crates/sparkflash-runtime group lanes (GroupLanes::in_step, group_out_of_step;
docs/engine/03-runtime.md:309-327).
"""
from __future__ import annotations

import hashlib
import struct


class GroupOutOfStep(RuntimeError):
    pass


class GroupLanes:
    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.tick = 0
        self._h = hashlib.sha256()
        self._reports: dict[int, dict[int, str]] = {}      # tick -> rank -> digest

    def record(self, rows, lanes, positions, tokens_out=()) -> str:
        """Fold one executed step into this rank's running digest; returns the digest after the step."""
        self.tick += 1
        self._h.update(struct.pack("<qI", self.tick, len(rows)))
        for seq in (rows, lanes, positions, tokens_out):
            self._h.update(struct.pack(f"<{len(seq)}q", *[int(x) for x in seq]))
        return self.digest()

    def digest(self) -> str:
        return self._h.copy().hexdigest()[:16]

    # ---- leader side ---------------------------------------------------------------------------------
    def report(self, rank: int, tick: int, digest: str) -> None:
        self._reports.setdefault(tick, {})[rank] = digest
        for t in [t for t in self._reports if t < tick - 64]:
            del self._reports[t]

    def in_step(self, tick: int) -> bool | None:
        """True when every rank reported the same digest for ``tick``; None while reports are missing."""
        got = self._reports.get(tick, {})
        if len(got) < self.world:
            return None
        return len(set(got.values())) == 1

    def check(self, tick: int) -> None:
        ok = self.in_step(tick)
        if ok is False:
            got = self._reports[tick]
            raise GroupOutOfStep(f"group out of step at tick {tick}: " + ", ".join(f"rank {r}={d}" for r, d in sorted(got.items())))
