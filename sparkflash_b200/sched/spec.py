"""Speculative-decoding policy: step-cost model, per-sequence draft depth, shared verify-step row allocation, draft
passes (C++ core in csrc/host_spec.cpp).

A decode tick with S decoding sequences runs one verify step of ``S + sum(k_s)`` rows: every sequence's anchor row plus
the k_s drafts kept for it.  Rows cost time (``StepCost``: two linear bands fitted to measured step times), drafts gain
tokens only while every shallower draft of the same sequence is accepted, so the policy adds drafts in order of
expected gain while the step's expected tokens per millisecond still rises.

Reference: crates/sparkflash-deepseek-forward/src/tp4_forward/spec.rs:1673 (STEP_COST), :1818 (depth policy),
batch.rs:2260-2485,2624 (shared speculative step, anchors first), draft.rs:904 (draft passes of at most 16 sequences),
docs/performance.md:303-307 (25.5 + 2.68 rows | 41.8 + 1.71 rows ms on the reference's hardware).
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_double, c_float, c_int, c_uint32, c_uint64
from dataclasses import dataclass

from .. import _lib

_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_spec_cost.restype = c_double
        L.sfb_spec_cost.argtypes = [c_double, c_double, c_double, c_double, c_int, c_int]
        L.sfb_spec_fit.argtypes = [ctypes.c_void_p, ctypes.c_void_p, c_int, c_int, ctypes.c_void_p]
        L.sfb_spec_allocate.argtypes = [c_int, ctypes.c_void_p, ctypes.c_void_p, c_int, c_int, c_double, c_double, c_double, c_double,
                                        c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.sfb_spec_draft_passes.argtypes = [c_int, c_int, ctypes.c_void_p, c_int]
        L.sfb_spec_accept.argtypes = [ctypes.c_void_p, ctypes.c_void_p, c_int]
        L.sfb_philox4x32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.sfb_philox_uniform.restype = c_double
        L.sfb_philox_uniform.argtypes = [c_uint64, c_uint64, c_uint64]
        _declared = True
    return L


@dataclass
class StepCost:
    """cost(rows) in ms: a0 + b0 rows up to ``band`` rows, a1 + b1 rows above.  The defaults are one B200 running the
    reduced single-GPU configuration (7.3 ms for one row, 15 ms for five rows, 20.5 ms for sixteen)."""
    a0: float = 5.4
    b0: float = 1.92
    a1: float = 13.2
    b1: float = 0.46
    band: int = 5

    def __call__(self, rows: int) -> float:
        return _L().sfb_spec_cost(self.a0, self.b0, self.a1, self.b1, self.band, rows)

    @classmethod
    def fit(cls, rows: list[int], ms: list[float], band: int) -> "StepCost":
        n = len(rows)
        out = (c_double * 4)()
        rc = _L().sfb_spec_fit((c_int * n)(*rows), (c_double * n)(*ms), n, band, out)
        if rc != 0:
            raise ValueError("need at least two distinct row counts to fit a step-cost band")
        return cls(out[0], out[1], out[2], out[3], band)


def calibrate(conf_logit: float, temperature: float = 1.0, bias: float = 0.0) -> float:
    """Acceptance probability of a draft from the drafter's raw confidence logit."""
    z = (conf_logit + bias) / max(temperature, 1e-6)
    return 1.0 / (1.0 + math.exp(-z)) if z > -60 else 0.0


@dataclass
class Allocation:
    keep: list[int]              # drafts kept per sequence
    rows: int                    # anchors + drafts
    expected_tokens: float
    cost_ms: float

    @property
    def tokens_per_ms(self) -> float:
        return self.expected_tokens / self.cost_ms if self.cost_ms > 0 else 0.0


class SpecPolicy:
    def __init__(self, cost: StepCost | None = None, max_rows: int = 64, max_depth: int = 8, passes_of: int = 16):
        self.cost, self.max_rows, self.max_depth, self.passes_of = cost or StepCost(), max_rows, max_depth, passes_of

    def allocate(self, probs: list[list[float]]) -> Allocation:
        """``probs[s]`` = acceptance probabilities of sequence s's drafts, shallowest first."""
        S, D = len(probs), self.max_depth
        depth = (c_int * max(S, 1))(*[min(len(p), D) for p in probs])
        flat = (c_float * max(S * D, 1))()
        for s, p in enumerate(probs):
            for j, v in enumerate(p[:D]):
                flat[s * D + j] = v
        keep = (c_int * max(S, 1))()
        tok, ms = c_double(0.0), c_double(0.0)
        c = self.cost
        rows = _L().sfb_spec_allocate(S, depth, flat, D, self.max_rows, c.a0, c.b0, c.a1, c.b1, c.band, keep, ctypes.byref(tok),
                                      ctypes.byref(ms))
        if rows < 0:
            raise ValueError(f"{S} decoding sequences do not fit a step of {self.max_rows} rows")
        return Allocation(list(keep[:S]), rows, tok.value, ms.value)

    def draft_passes(self, n_seq: int) -> list[range]:
        """Sequences that need a draft block, in passes of at most ``passes_of``."""
        mp = n_seq // max(1, self.passes_of) + 2
        start = (c_int * (mp + 1))()
        p = _L().sfb_spec_draft_passes(n_seq, self.passes_of, start, mp)
        return [range(start[i], start[i + 1]) for i in range(p)]


def accept(drafts: list[int], sampled: list[int]) -> int:
    """Number of drafts the verifier reproduced (``sampled[i]`` = the token chosen at verify row i; the bonus token is
    ``sampled[accepted]``)."""
    k = min(len(drafts), len(sampled))
    return _L().sfb_spec_accept((ctypes.c_int32 * max(k, 1))(*drafts[:k]), (ctypes.c_int32 * max(k, 1))(*sampled[:k]), k)


def philox4x32(counter: tuple[int, int, int, int], key: tuple[int, int]) -> tuple[int, int, int, int]:
    out = (c_uint32 * 4)()
    _L().sfb_philox4x32((c_uint32 * 4)(*counter), (c_uint32 * 2)(*key), out)
    return tuple(out)


def philox_uniform(seed: int, stream: int, index: int) -> float:
    return _L().sfb_philox_uniform(seed & (2 ** 64 - 1), stream & (2 ** 64 - 1), index & (2 ** 64 - 1))
