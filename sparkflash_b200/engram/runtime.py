"""Engram inside the serving engine: per-lane compressed-token history and hashing on the host, row gather, key/value
projection and the gated residual write on the device, before the blocks of the Engram layers.
Reference: crates/sparkflash-deepseek-forward/src/tp4_forward/spec.rs:134-265 (lookup wired into the step),
docs/architecture/04-engram.md sections 5-7.  The tables are replicated (or sharded with ``world`` > 1 through
``EngramShard``'s range logic; partial lookups are then summed by the caller)."""
from __future__ import annotations

from ctypes import c_float, c_int

import numpy as np
import torch

from .. import _lib
from ..ops import native as N
from .layout import DEAD, EngramLayout
from .store import EngramShard, pack_table


class EngramRuntime:
    def __init__(self, cfg, layout: EngramLayout, shards: list[EngramShard], wkv: list, gate_w: list[torch.Tensor], token_map: np.ndarray | None = None,
                 sharded: bool = False):
        self.cfg, self.layout, self.shards, self.wkv, self.gate_w = cfg, layout, shards, wkv, gate_w
        self.sharded = sharded        # every rank holds a row range: the ranks' partial lookups are summed (rows outside a shard read as zeros)
        cv = cfg.engram_compressed_vocab
        self.token_map = token_map if token_map is not None else (np.arange(cfg.vocab_size, dtype=np.int64) % cv)
        self.pad = int(self.token_map[cfg.pad_id])
        self.hist: dict[int, np.ndarray] = {}
        self.lookups = 0

    @classmethod
    def from_checkpoint(cls, ck: dict, cfg, device="cuda", rank: int = 0, world: int = 1, table_dir: str | None = None,
                        page_rows: int = 64, cache_pages: int = 4096) -> "EngramRuntime":
        """``ck``: the quantised checkpoint dict (``engram.{l}.embed.weight|scale``, ``engram.{l}.wkv.weight|scale``, ``engram.{l}.gate_w``).
        ``world`` > 1: every rank keeps the row range ``store.shard_range`` gives it and the engine sums the ranks' lookups.
        ``table_dir``: the tables stay in the packed files written by ``store.pack`` (one rank: ``...-rank0-of-1.bin``) and are
        read through the page cache (engram/paged.py) instead of being held in memory."""
        from ..models.deepseek_v41 import tc as TC
        from ..models.deepseek_v41.prepare import _prep_sf_block32
        lay = EngramLayout.build(cfg.engram_layers, cfg.engram_max_ngram, cfg.engram_n_heads, cfg.engram_vocab, cfg.engram_compressed_vocab)
        shards, wkv, gw = [], [], []
        for j, l in enumerate(cfg.engram_layers):
            w, s = ck[f"engram.{l}.embed.weight"], ck[f"engram.{l}.embed.scale"]
            if table_dir is not None:
                import os
                from .paged import PagedShard, PagedTable
                path = os.path.join(table_dir, f"engram-L{l}-rank0-of-1.bin")
                shards.append(PagedShard(PagedTable(path, w.shape[0], page_rows, cache_pages, pin=torch.device(device).type == "cuda"), device))
            else:
                shards.append(EngramShard(pack_table(w, s, rank, world), w.shape[0], rank, world, device))
            q, sf = ck[f"engram.{l}.wkv.weight"].contiguous().to(device), _prep_sf_block32(ck[f"engram.{l}.wkv.scale"], ck[f"engram.{l}.wkv.weight"].shape[0]).to(device)
            wkv.append((q, sf, TC._matrix(q, sf, q.shape[0], q.shape[1], False, None)))
            gw.append(ck[f"engram.{l}.gate_w"].to(torch.float32).contiguous().to(device))
        return cls(cfg, lay, shards, wkv, gw, sharded=world > 1 and table_dir is None)

    def prefetch(self, tokens, lane: int, first_pos: int) -> int:
        """Read ahead for tokens that will be computed soon (a prompt's remaining chunks, a draft block): their row ids depend
        only on the token ids, so the pages can be on their way while the GPU runs the current step.  The lane's history
        is not changed.  Returns the number of pages queued (0 for resident shards)."""
        if not any(hasattr(s, "prefetch") for s in self.shards):
            return 0
        h = self.hist.get(lane)
        base = np.full((first_pos + len(tokens),), DEAD, dtype=np.int64)
        if h is not None:
            k = min(first_pos, h.shape[0])
            base[:k] = h[:k]
        for i, t in enumerate(tokens):
            base[first_pos + i] = self.token_map[t] if 0 <= t < self.token_map.shape[0] else DEAD
        pos = list(range(first_pos, first_pos + len(tokens)))
        queued = 0
        for j, sh in enumerate(self.shards):
            if hasattr(sh, "prefetch"):
                queued += sh.prefetch(torch.from_numpy(self.layout.hash_ids(j, base, pos, self.pad)))
        return queued

    def ids_for_step(self, tokens, lanes, positions) -> np.ndarray:
        """Row ids [n_engram_layers, n, cols] for the rows of one step; the lanes' histories are updated first."""
        n = len(tokens)
        for t, ln, p in zip(tokens, lanes, positions):
            h = self.hist.get(ln)
            if h is None or p >= h.shape[0]:
                grown = np.full((max(1024, 2 * (p + 1)),), DEAD, dtype=np.int64)
                if h is not None:
                    grown[:h.shape[0]] = h
                self.hist[ln] = h = grown
            h[p] = self.token_map[t] if 0 <= t < self.token_map.shape[0] else DEAD
        out = np.zeros((len(self.cfg.engram_layers), n, self.layout.cols), dtype=np.int64)
        for ln in sorted(set(lanes)):
            idx = [i for i, l_ in enumerate(lanes) if l_ == ln]
            pos = [positions[i] for i in idx]
            for j in range(out.shape[0]):
                out[j, idx] = self.layout.hash_ids(j, self.hist[ln], pos, self.pad)
        self.lookups += n * out.shape[0] * self.layout.cols
        return out


def gate_bf16(h: torch.Tensor, kv: torch.Tensor, w: torch.Tensor, image_mask: torch.Tensor | None, n: int, eps: float) -> None:
    hc, d = h.shape[1], h.shape[2]
    N._check(_lib.cuda().sfb_engram_gate_bf16(N._p(h), N._p(kv), N._p(w), N._p(image_mask), c_int(n), c_int(hc), c_int(d), c_float(eps), N._stream()),
             "engram_gate_bf16")
