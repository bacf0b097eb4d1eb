"""Per-step ledger: what a step is allowed to do, counted while it runs, checked when it ends.

A serving step has a fixed shape: so many kernel launches, so many collectives, so many host<->device crossings.
When a change sneaks a synchronising copy or a stray collective into the hot loop, the count moves; the ledger turns
that into an error at the end of the step instead of a slow regression found weeks later.  The engine calls
``count`` from its launch / copy / collective sites; ``Budget`` is derived from the model shape.

Reference: crates/sparkflash-deepseek-forward/src/device_counters.rs (allowed host<->device crossings per step; a step
whose count differs is refused), layer_device.rs:1344,1365 (collective count checked inside the engine),
scripts/check-collective-count.py, crates/sparkflash-runtime (ledger).
"""
from __future__ import annotations

from dataclasses import dataclass, field

KINDS = ("launch", "collective", "h2d", "d2h", "host_sync", "alloc")


class LedgerError(RuntimeError):
    pass


@dataclass(frozen=True)
class Budget:
    """Upper bounds per step (None = unbounded) and exact counts where the design fixes them."""
    max_launches: int | None = None
    collectives: int | None = None         # exact
    max_h2d: int | None = None
    max_d2h: int | None = None
    max_host_sync: int | None = None
    max_alloc: int | None = 0              # a steady-state step allocates nothing

    @staticmethod
    def for_rows_step(n_layers: int, world: int, fused: bool, sampled: bool = True, launches_per_layer: int = 24) -> "Budget":
        """Two reductions per layer, plus the exchange of the vocabulary-slice winners when the step is sampled; none on
        one rank.  Five input copies (tokens, lanes, positions, temperatures, seeds) and one result copy per step."""
        coll = 0 if world == 1 else 2 * n_layers + (1 if sampled else 0)
        return Budget(max_launches=launches_per_layer * n_layers + 32, collectives=coll, max_h2d=8, max_d2h=1 if sampled else 0,
                      max_host_sync=1)


@dataclass
class StepLedger:
    budget: Budget = field(default_factory=Budget)
    counts: dict = field(default_factory=lambda: {k: 0 for k in KINDS})
    steps: int = 0
    history: list = field(default_factory=list)      # last few steps' counts, for /v1/cluster/stats
    keep: int = 16

    def begin(self) -> None:
        for k in KINDS:
            self.counts[k] = 0

    def count(self, kind: str, n: int = 1) -> None:
        if kind not in self.counts:
            raise KeyError(kind)
        self.counts[kind] += n

    def end(self, strict: bool = True) -> dict:
        """Close the step: returns its counts; raises LedgerError when a count breaks the budget and ``strict``."""
        c, b = dict(self.counts), self.budget
        problems = []
        if b.collectives is not None and c["collective"] != b.collectives:
            problems.append(f"collectives {c['collective']} != {b.collectives}")
        for kind, cap in (("launch", b.max_launches), ("h2d", b.max_h2d), ("d2h", b.max_d2h), ("host_sync", b.max_host_sync),
                          ("alloc", b.max_alloc)):
            if cap is not None and c[kind] > cap:
                problems.append(f"{kind} {c[kind]} > {cap}")
        self.steps += 1
        self.history.append(c)
        del self.history[:-self.keep]
        if problems and strict:
            raise LedgerError("step breaks its budget: " + "; ".join(problems))
        c["problems"] = problems
        return c

    def snapshot(self) -> dict:
        return {"steps": self.steps, "last": self.history[-1] if self.history else None}
