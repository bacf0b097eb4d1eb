"""Python face of the C++ scheduler core (csrc/host_sched.cpp) and the KV planning structures
(csrc/host_radix.cpp)."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_int64, c_void_p
from dataclasses import dataclass

from .. import _lib

_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_sched_create.restype = c_void_p
        L.sfb_sched_create.argtypes = [c_int] * 8 + [c_int64]
        L.sfb_sched_destroy.argtypes = [c_void_p]
        L.sfb_sched_set_ring_slack.argtypes = [c_void_p, c_int64]
        L.sfb_sched_set_decoder_tail.argtypes = [c_void_p, c_int]
        L.sfb_sched_submit.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int]
        L.sfb_sched_cancel.argtypes = [c_void_p, c_int64]
        L.sfb_sched_set_drafts.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int]
        L.sfb_sched_tick.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
        L.sfb_sched_commit.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_int]
        L.sfb_sched_release.argtypes = [c_void_p, c_int64]
        L.sfb_sched_stats.argtypes = [c_void_p, c_void_p]
        L.sfb_sched_seq_info.argtypes = [c_void_p, c_int64, c_void_p]
        L.sfb_radix_create.restype = c_void_p
        L.sfb_radix_destroy.argtypes = [c_void_p]
        L.sfb_radix_match.argtypes = [c_void_p, c_void_p, c_int]; L.sfb_radix_match.restype = c_int64
        L.sfb_radix_insert.argtypes = [c_void_p, c_void_p, c_int]
        L.sfb_radix_pin.argtypes = [c_void_p, c_void_p, c_int, c_int]
        L.sfb_radix_evict.argtypes = [c_void_p, c_int64]; L.sfb_radix_evict.restype = c_int64
        L.sfb_radix_tokens.argtypes = [c_void_p]; L.sfb_radix_tokens.restype = c_int64
        L.sfb_radix_stats.argtypes = [c_void_p, c_void_p]
        L.sfb_pager_create.restype = c_void_p; L.sfb_pager_create.argtypes = [c_int]
        for f in ("sfb_pager_destroy",):
            getattr(L, f).argtypes = [c_void_p]
        L.sfb_pager_alloc.argtypes = [c_void_p]
        L.sfb_pager_share.argtypes = [c_void_p, c_int]
        L.sfb_pager_release.argtypes = [c_void_p, c_int]
        L.sfb_pager_free_count.argtypes = [c_void_p]
        _declared = True
    return L


def _i32(seq):
    arr = (c_int32 * len(seq))(*seq)
    return arr


@dataclass
class PlanRow:
    seq: int
    lane: int
    pos: int
    token: int
    kind: int  # 0 prefill, 1 decode anchor, 2 draft row, 3 prefill row that runs the cache-owning layers only

PHASE_IDLE, PHASE_PREFILL, PHASE_DECODE = 0, 1, 2
STATE_NAMES = ["waiting", "prefill", "decode", "finished", "preempted"]


class Scheduler:
    def __init__(self, max_lanes=32, queue_depth=64, max_rows=64, prefill_chunk=4096, prefill_chunk_busy=2048,
                 prefix_reuse_min=256, max_context=1048576, spec_depth=5, lane_row_budget=-1):
        self.max_rows = max_rows
        self._h = c_void_p(_L().sfb_sched_create(max_lanes, queue_depth, max_rows, prefill_chunk, prefill_chunk_busy,
                                                 prefix_reuse_min, max_context, spec_depth, lane_row_budget))
        self._buf = (c_int64 * (5 * max(max_rows, prefill_chunk)))()
        self._cap = max(max_rows, prefill_chunk)

    def __del__(self):
        try:
            _L().sfb_sched_destroy(self._h)
        except Exception:
            pass

    def set_ring_slack(self, rows: int) -> None:
        _L().sfb_sched_set_ring_slack(self._h, rows)

    def set_decoder_tail(self, rows: int) -> None:
        """Prompt rows more than ``rows`` before the prompt's end are planned as kind-3 chunks (cache-owning layers only)."""
        _L().sfb_sched_set_decoder_tail(self._h, rows)

    def submit(self, seq_id: int, prompt: list[int], max_new: int) -> int:
        return _L().sfb_sched_submit(self._h, seq_id, _i32(prompt), len(prompt), max_new)

    def cancel(self, seq_id: int) -> int:
        return _L().sfb_sched_cancel(self._h, seq_id)

    def set_drafts(self, seq_id: int, tokens: list[int], conf: list[float]) -> int:
        return _L().sfb_sched_set_drafts(self._h, seq_id, _i32(tokens), (c_float * len(conf))(*conf), len(tokens))

    def tick(self, max_out: int | None = None) -> tuple[int, list[PlanRow]]:
        phase = c_int(0)
        n = _L().sfb_sched_tick(self._h, self._buf, min(self._cap, max_out or self._cap), ctypes.byref(phase))
        b = self._buf
        rows = [PlanRow(b[5 * i], b[5 * i + 1], b[5 * i + 2], b[5 * i + 3], b[5 * i + 4]) for i in range(n)]
        return phase.value, rows

    def commit(self, seq_id: int, rows_done: int, new_tokens: list[int], eos_id: int) -> int:
        return _L().sfb_sched_commit(self._h, seq_id, rows_done, _i32(new_tokens), len(new_tokens), eos_id)

    def release(self, seq_id: int) -> int:
        return _L().sfb_sched_release(self._h, seq_id)

    def stats(self) -> dict:
        out = (c_int64 * 8)()
        _L().sfb_sched_stats(self._h, out)
        keys = ["running", "waiting", "free_lanes", "rejected", "preemptions", "prefix_hits", "prefix_rows", "tick"]
        return dict(zip(keys, list(out)))

    def info(self, seq_id: int) -> dict | None:
        out = (c_int64 * 4)()
        if _L().sfb_sched_seq_info(self._h, seq_id, out):
            return None
        return {"state": STATE_NAMES[out[0]], "lane": out[1], "computed": out[2], "generated": out[3]}


class RadixCache:
    def __init__(self):
        self._h = c_void_p(_L().sfb_radix_create())

    def __del__(self):
        try:
            _L().sfb_radix_destroy(self._h)
        except Exception:
            pass

    def match(self, tokens) -> int:
        return int(_L().sfb_radix_match(self._h, _i32(tokens), len(tokens)))

    def insert(self, tokens) -> None:
        _L().sfb_radix_insert(self._h, _i32(tokens), len(tokens))

    def pin(self, tokens, delta=1) -> None:
        _L().sfb_radix_pin(self._h, _i32(tokens), len(tokens), delta)

    def evict(self, target_tokens: int) -> int:
        return int(_L().sfb_radix_evict(self._h, target_tokens))

    @property
    def tokens(self) -> int:
        return int(_L().sfb_radix_tokens(self._h))


class Pager:
    def __init__(self, n_pages: int):
        self._h = c_void_p(_L().sfb_pager_create(n_pages))

    def __del__(self):
        try:
            _L().sfb_pager_destroy(self._h)
        except Exception:
            pass

    def alloc(self) -> int:
        return _L().sfb_pager_alloc(self._h)

    def share(self, page: int) -> int:
        return _L().sfb_pager_share(self._h, page)

    def release(self, page: int) -> int:
        return _L().sfb_pager_release(self._h, page)

    @property
    def free(self) -> int:
        return _L().sfb_pager_free_count(self._h)
