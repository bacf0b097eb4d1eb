"""Lane memory for the position-addressed KV regions: reserved address space per lane, 2 MiB chunks mapped as a
sequence grows, given back when it ends (csrc/k_lanes.cu).  ``LaneRegion.tensor`` is a torch view of the whole
[lanes, rows, width] array through ``__cuda_array_interface__``; rows beyond a lane's backed prefix own no
memory and must not be touched.  Reference: crates/sparkflash-kernels/src/lane_memory.rs:93-586,
crates/sparkflash-deepseek-forward/src/tp4_forward/lanes.rs (32 lanes, 1M context, lazy backing, LRU give-back).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import torch

from .. import _lib

_declared = False


def _L():
    global _declared
    L = _lib.cuda()
    if not _declared:
        L.sfb_lanepool_granularity.restype = c_longlong
        L.sfb_laneregion_base.restype = ctypes.c_ulonglong
        for f in ("sfb_laneregion_span", "sfb_laneregion_mapped"):
            getattr(L, f).restype = c_longlong
        L.sfb_laneregion_backed.restype = c_longlong
        _declared = True
    return L


class LaneBudgetExceeded(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc == 2:
        raise LaneBudgetExceeded(f"{what}: chunk budget exhausted")
    if rc:
        raise RuntimeError(f"{what} failed: status {rc}" + (f" (CUresult {rc - 100})" if rc >= 100 else ""))


class LanePool:
    def __init__(self, budget_bytes: int, device: int | None = None):
        dev = torch.cuda.current_device() if device is None else device
        h = c_void_p()
        _check(_L().sfb_lanepool_create(c_int(dev), c_longlong(budget_bytes), ctypes.byref(h)), "lane pool")
        self._h, self.device = h, dev
        self.granularity = int(_L().sfb_lanepool_granularity(self._h))
        self.regions: list[LaneRegion] = []

    def stats(self) -> dict:
        out = (c_longlong * 3)()
        _L().sfb_lanepool_stats(self._h, out)
        return {"created": out[0], "spare": out[1], "budget": out[2], "granularity": self.granularity}

    def trim(self, max_chunks: int = 1 << 30) -> int:
        return _L().sfb_lanepool_trim(self._h, c_int(min(max_chunks, 2 ** 31 - 1)))

    def close(self) -> None:
        for r in self.regions:
            r.close()
        self.regions = []
        if self._h:
            _L().sfb_lanepool_destroy(self._h)
            self._h = None


class _Iface:
    def __init__(self, ptr, shape, strides, typestr):
        self.__cuda_array_interface__ = {"shape": shape, "strides": strides, "typestr": typestr, "data": (ptr, False), "version": 3}


class LaneRegion:
    """[lanes, rows, width] uint8, lane stride = span bytes (rows is rounded up so that a lane fills whole chunks)."""

    def __init__(self, pool: LanePool, lanes: int, rows: int, width: int):
        self.pool, self.lanes, self.width = pool, lanes, width
        g = pool.granularity
        span = -(-rows * width // g) * g
        while span % width:          # keep the array dense: a lane must hold a whole number of rows
            span += g
        h = c_void_p()
        _check(_L().sfb_laneregion_create(pool._h, c_int(lanes), c_longlong(span), ctypes.byref(h)), "lane region")
        self._h = h
        self.span = int(_L().sfb_laneregion_span(self._h))
        self.rows = self.span // width
        self.base = int(_L().sfb_laneregion_base(self._h))
        self._keep = _Iface(self.base, (lanes, self.rows, width), None, "|u1")
        self.tensor = torch.as_tensor(self._keep, device=torch.device("cuda", pool.device))
        pool.regions.append(self)

    def ensure_rows(self, lane: int, rows: int) -> None:
        _check(_L().sfb_laneregion_ensure(self._h, c_int(lane), c_longlong(min(rows, self.rows) * self.width)), "lane ensure")

    def backed_rows(self, lane: int) -> int:
        return int(_L().sfb_laneregion_backed(self._h, c_int(lane))) // self.width

    def release(self, lane: int, from_row: int = 0) -> None:
        _check(_L().sfb_laneregion_release(self._h, c_int(lane), c_longlong(from_row * self.width)), "lane release")

    def copy_prefix(self, src: int, dst: int, rows: int) -> None:
        _check(_L().sfb_laneregion_copy_prefix(self._h, c_int(src), c_int(dst), c_longlong(rows * self.width),
                                               c_void_p(torch.cuda.current_stream().cuda_stream)), "lane copy_prefix")

    @property
    def mapped_bytes(self) -> int:
        return int(_L().sfb_laneregion_mapped(self._h))

    def close(self) -> None:
        if self._h:
            self.tensor = None
            _L().sfb_laneregion_destroy(self._h)
            self._h = None
