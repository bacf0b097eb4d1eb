"""Engram table on storage: paged reads with a cache and read-ahead (C++ core: csrc/host_engram_paged.cpp).

``PagedTable`` serves the rows of one layer's packed table file (``engram.store.pack``) without holding the table in
memory.  ``gather(ids)`` returns the packed rows in a pinned host buffer, ready for one host->device copy;
``prefetch(ids)`` asks the background reader for the pages of rows that a coming step will need.  ``PagedShard`` gives
it the interface of ``EngramShard`` (``gather(ids, out)`` -> bf16 rows on the device), so the serving engine takes either.

Placement on B200: with eight ranks a row-range shard (23.6 GiB) lives in HBM (``EngramShard``); with one or two ranks
the reduced expert pool already fills the GPU and the tables stay on NVMe behind this reader.

Reference: crates/sparkflash-engram/src/{paged,store}.rs, crates/sparkflash-deepseek-forward/src/tp4_forward/spec.rs:134-265
(Engram reader inside the serve loop, read-ahead for the next positions).
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_uint64, c_void_p

import torch

from .. import _lib
from .store import STRIDE, gather_reference

_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_epaged_open.restype = c_void_p
        L.sfb_epaged_open.argtypes = [c_char_p, c_int64, c_int, c_int, c_int]
        L.sfb_epaged_close.argtypes = [c_void_p]
        L.sfb_epaged_gather.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
        L.sfb_epaged_prefetch.argtypes = [c_void_p, c_void_p, c_int]
        L.sfb_epaged_drain.argtypes = [c_void_p]
        L.sfb_epaged_stats.argtypes = [c_void_p, c_void_p]
        _declared = True
    return L


class PagedTable:
    def __init__(self, path: str, rows: int, page_rows: int = 64, cache_pages: int = 4096, stride: int = STRIDE, pin: bool = False):
        self.rows, self.stride, self.page_rows = rows, stride, page_rows
        self._h = _L().sfb_epaged_open(path.encode(), rows, stride, page_rows, cache_pages)
        if not self._h:
            raise OSError(f"cannot open {path} as a packed table of {rows} rows x {stride} bytes")
        self._pin = pin
        self._buf: torch.Tensor | None = None

    def _buffer(self, n: int) -> torch.Tensor:
        if self._buf is None or self._buf.shape[0] < n:
            b = torch.empty((max(n, 256), self.stride), dtype=torch.uint8)
            self._buf = b.pin_memory() if self._pin else b
        return self._buf[:n]

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        """Packed rows uint8 [ids.numel(), stride] for int64 ids (any shape); ids outside the table give zero rows.
        The returned tensor is a view of an internal buffer that the next call reuses."""
        flat = ids.reshape(-1).to(torch.int64).contiguous().cpu()
        out = self._buffer(flat.numel())
        if _L().sfb_epaged_gather(self._h, c_void_p(flat.data_ptr()), flat.numel(), c_void_p(out.data_ptr())) != 0:
            raise OSError("reading the packed table failed")
        return out

    def prefetch(self, ids: torch.Tensor) -> int:
        flat = ids.reshape(-1).to(torch.int64).contiguous().cpu()
        return _L().sfb_epaged_prefetch(self._h, c_void_p(flat.data_ptr()), flat.numel())

    def drain(self) -> None:
        _L().sfb_epaged_drain(self._h)

    def stats(self) -> dict:
        out = (c_uint64 * 8)()
        _L().sfb_epaged_stats(self._h, out)
        keys = ("hits", "misses", "prefetched_pages", "evictions", "bytes_read", "resident_pages", "waits", "queued")
        d = dict(zip(keys, [int(x) for x in out]))
        look = d["hits"] + d["misses"]
        d["hit_rate"] = d["hits"] / look if look else 0.0
        return d

    def close(self) -> None:
        if self._h:
            _L().sfb_epaged_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PagedShard:
    """``EngramShard``'s interface over a table that stays on storage: the step's rows are read through the page cache
    into pinned memory, copied to the device once, and decoded there."""

    def __init__(self, table: PagedTable, device="cuda"):
        self.table, self.device = table, torch.device(device)
        self.first, self.per, self.width = 0, table.rows, 256
        self.lookups = 0

    def gather(self, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        n, cols = ids.shape
        self.lookups += n * cols
        packed = self.table.gather(ids)                              # [n*cols, stride] host
        if out is None:
            out = torch.empty((n, cols * self.width), dtype=torch.bfloat16, device=self.device)
        if self.device.type == "cuda":
            from ..ops import native as N
            dev_rows = packed.to(self.device, non_blocking=True)
            seq = torch.arange(n * cols, dtype=torch.int64, device=self.device).reshape(n, cols)
            rc = _lib.cuda().sfb_engram_gather(c_void_p(dev_rows.data_ptr()), ctypes.c_longlong(0), ctypes.c_longlong(n * cols),
                                               c_int(self.table.stride), N._p(seq), c_int(n), c_int(cols), c_int(self.width), N._p(out),
                                               N._stream())
            N._check(rc, "engram_gather")
            return out
        seq = torch.arange(n * cols, dtype=torch.int64).reshape(n, cols)
        out.copy_(gather_reference(packed.clone(), 0, seq).to(torch.bfloat16))
        return out

    def prefetch(self, ids: torch.Tensor) -> int:
        return self.table.prefetch(ids)
