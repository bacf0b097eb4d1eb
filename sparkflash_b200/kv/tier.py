"""Second tier for sequence caches: a finished or preempted sequence's KV leaves its lane for pinned host memory and comes
back into any free lane later.

A lane's state up to position p is small (window ring tail + compressed entries + index keys of the cache-owning
layers: under 1 KB per token), so parking it costs one device->host copy per layer and un-parking one copy back; the
sequence then continues from position p without recomputing its prefix.  The tier is keyed by the token prefix (the
radix tree of csrc/host_radix.cpp finds the longest parked prefix of a new prompt), bounded in bytes, and evicts least
recently used entries.

What is saved per layer: the last ``window`` slots of the FP8 window ring (codes + scales) at their ring positions, the
compressor's pending inputs for ratio-2 layers, and rows [0, p // ratio] of the compressed KV and index-key caches of
the layers that own them.

Reference: crates/sparkflash-kv/src/{tier,swa,device_store,cache}.rs (tiering, sliding-window tail replay, device store),
docs/architecture/08-kv-footprint.md.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field

import torch


@dataclass
class ParkedSequence:
    tokens: tuple[int, ...]
    positions: int                      # tokens[0:positions] are cached
    layers: dict = field(default_factory=dict)
    nbytes: int = 0


def _host(t: torch.Tensor) -> torch.Tensor:
    h = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.device.type == "cuda")
    h.copy_(t, non_blocking=True)
    return h


class KVTier:
    def __init__(self, kv, budget_bytes: int = 8 << 30):
        """``kv``: the engine's KVCache (models/deepseek_v41/engine.py)."""
        self.kv, self.budget = kv, budget_bytes
        self.entries: "OrderedDict[tuple, ParkedSequence]" = OrderedDict()
        self.bytes = 0
        self.parked = self.restored = self.evicted = 0

    # ---- park ------------------------------------------------------------------------------------------
    def park(self, lane: int, tokens: list[int], positions: int) -> ParkedSequence:
        kv, cfg = self.kv, self.kv.cfg
        ring, window = kv.ring, cfg.window
        first = max(0, positions - window)
        slots = torch.tensor([p % ring for p in range(first, positions)], dtype=torch.int64, device=next(iter(kv.win_q.values())).device)
        ent = ParkedSequence(tuple(tokens[:positions]), positions)
        for l, wq in kv.win_q.items():
            rec = {"win_q": _host(wq[lane].index_select(0, slots)), "win_s": _host(kv.win_s[l][lane].index_select(0, slots))}
            if l in kv.cin:
                rec["cin"] = _host(kv.cin[l][lane].index_select(0, slots))
            if l in kv.ckv_q:
                n = positions // cfg.ratio(l) + 1
                for name in ("ckv_q", "ckv_s", "ik_q", "ik_s"):
                    rec[name] = _host(getattr(kv, name)[l][lane, :n])
            ent.layers[l] = rec
            ent.nbytes += sum(t.numel() * t.element_size() for t in rec.values())
        if torch.cuda.is_available() and slots.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self._insert(ent)
        self.parked += 1
        return ent

    def _insert(self, ent: ParkedSequence) -> None:
        old = self.entries.pop(ent.tokens, None)
        if old is not None:
            self.bytes -= old.nbytes
        self.entries[ent.tokens] = ent
        self.bytes += ent.nbytes
        while self.bytes > self.budget and len(self.entries) > 1:
            _, victim = self.entries.popitem(last=False)
            self.bytes -= victim.nbytes
            self.evicted += 1

    # ---- find / restore -----------------------------------------------------------------------------------
    def longest_prefix(self, prompt: list[int]) -> ParkedSequence | None:
        """The parked sequence that is the longest whole prefix of ``prompt`` (a parked sequence is usable only as a
        whole: its window tail belongs to its last position)."""
        best = None
        for key, ent in self.entries.items():
            n = len(key)
            if n <= len(prompt) and (best is None or n > best.positions) and tuple(prompt[:n]) == key:
                best = ent
        return best

    def restore(self, ent: ParkedSequence, lane: int) -> int:
        """Copy a parked sequence into ``lane``; returns the number of positions that are now cached there."""
        kv, cfg = self.kv, self.kv.cfg
        ring, window = kv.ring, cfg.window
        positions = ent.positions
        first = max(0, positions - window)
        dev = next(iter(kv.win_q.values())).device
        slots = torch.tensor([p % ring for p in range(first, positions)], dtype=torch.int64, device=dev)
        if hasattr(kv, "ensure"):
            kv.ensure([lane], [max(0, positions - 1)])
        for l, rec in ent.layers.items():
            kv.win_q[l][lane].index_copy_(0, slots, rec["win_q"].to(dev, non_blocking=True))
            kv.win_s[l][lane].index_copy_(0, slots, rec["win_s"].to(dev, non_blocking=True))
            if "cin" in rec:
                kv.cin[l][lane].index_copy_(0, slots, rec["cin"].to(dev, non_blocking=True))
            if "ckv_q" in rec:
                n = rec["ckv_q"].shape[0]
                for name in ("ckv_q", "ckv_s", "ik_q", "ik_s"):
                    getattr(kv, name)[l][lane, :n].copy_(rec[name].to(dev, non_blocking=True))
        self.entries.move_to_end(ent.tokens)
        self.restored += 1
        return positions

    def stats(self) -> dict:
        return {"entries": len(self.entries), "bytes": self.bytes, "parked": self.parked, "restored": self.restored, "evicted": self.evicted}
