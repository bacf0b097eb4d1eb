"""Guard bands around device buffers: a stand-in for a memory checker where none can be run.

``with guarded() as arena:`` makes every ``torch.zeros / empty / full / ones`` on a CUDA device inside the block return a
view into a larger allocation with a 256-byte band of a fixed pattern before and after it (the view keeps 256-byte
alignment, so TMA maps and vector accesses are unaffected).  ``arena.check()`` reads the bands back and names every
allocation whose band changed, with the source line that made it: a kernel that wrote a few bytes past (or before) one
of its buffers is caught at the next check instead of corrupting a neighbour silently.  ``Engine.with_guards(...)`` builds
an engine this way and ``Engine.check_status()`` then checks the bands too; ``SFB_DEBUG_BOUNDS=1`` makes the serving
launcher and the tests' engine fixture do so.

Reference behaviour: the reference's debug builds with redzones around step buffers and its compute-sanitizer CI lane
(scripts/probes, ci/): the same class of defect, found without the tool.
"""
from __future__ import annotations

import contextlib
import traceback
from dataclasses import dataclass

import torch

GUARD = 256
PATTERN = 0xA5


@dataclass
class _Rec:
    raw: torch.Tensor
    nbytes: int
    where: str
    shape: tuple


class GuardArena:
    def __init__(self):
        self.records: list[_Rec] = []
        self._depth = 0

    def alloc(self, shape, dtype, device, fill=None) -> torch.Tensor:
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = n * esz
        body = (nbytes + GUARD - 1) // GUARD * GUARD
        raw = _REAL["empty"](GUARD + body + GUARD, dtype=torch.uint8, device=device)
        raw[:GUARD] = PATTERN
        raw[GUARD + nbytes:] = PATTERN
        view = raw[GUARD:GUARD + nbytes].view(dtype).view(shape)
        if fill is not None:
            view.fill_(fill)
        where = "?"
        for fr in reversed(traceback.extract_stack(limit=12)[:-2]):
            if "canary.py" not in fr.filename:
                where = f"{fr.filename.rsplit('/', 1)[-1]}:{fr.lineno}"
                break
        self.records.append(_Rec(raw, nbytes, where, shape))
        return view

    def check(self) -> list[str]:
        """Every allocation whose band before or after it no longer holds the pattern."""
        torch.cuda.synchronize()
        bad = []
        for r in self.records:
            head_ok = bool((r.raw[:GUARD] == PATTERN).all())
            tail_ok = bool((r.raw[GUARD + r.nbytes:] == PATTERN).all())
            if not (head_ok and tail_ok):
                side = "before" if not head_ok else "after"
                if not head_ok and not tail_ok:
                    side = "before and after"
                bad.append(f"{r.where}: buffer {r.shape} ({r.nbytes} bytes) was written {side} its bounds")
        return bad

    @contextlib.contextmanager
    def active(self):
        """Guard the allocations made inside the block (buffers an engine creates on first use)."""
        with _patched(self):
            yield self


_REAL = {"zeros": torch.zeros, "empty": torch.empty, "full": torch.full, "ones": torch.ones}


def _is_cuda(device) -> bool:
    if device is None:
        return False
    return torch.device(device).type == "cuda"


@contextlib.contextmanager
def _patched(arena: GuardArena):
    if arena._depth:
        arena._depth += 1
        try:
            yield
        finally:
            arena._depth -= 1
        return

    def zeros(*size, dtype=None, device=None, **kw):
        if not _is_cuda(device) or kw:
            return _REAL["zeros"](*size, dtype=dtype, device=device, **kw)
        shape = size[0] if len(size) == 1 and not isinstance(size[0], int) else size
        return arena.alloc(shape, dtype or torch.get_default_dtype(), device, 0)

    def ones(*size, dtype=None, device=None, **kw):
        if not _is_cuda(device) or kw:
            return _REAL["ones"](*size, dtype=dtype, device=device, **kw)
        shape = size[0] if len(size) == 1 and not isinstance(size[0], int) else size
        return arena.alloc(shape, dtype or torch.get_default_dtype(), device, 1)

    def empty(*size, dtype=None, device=None, **kw):
        if not _is_cuda(device) or kw:
            return _REAL["empty"](*size, dtype=dtype, device=device, **kw)
        shape = size[0] if len(size) == 1 and not isinstance(size[0], int) else size
        return arena.alloc(shape, dtype or torch.get_default_dtype(), device, None)

    def full(size, fill_value, dtype=None, device=None, **kw):
        if not _is_cuda(device) or kw or dtype is None:
            return _REAL["full"](size, fill_value, dtype=dtype, device=device, **kw)
        return arena.alloc(size, dtype, device, fill_value)

    arena._depth = 1
    torch.zeros, torch.empty, torch.full, torch.ones = zeros, empty, full, ones
    try:
        yield
    finally:
        torch.zeros, torch.empty, torch.full, torch.ones = _REAL["zeros"], _REAL["empty"], _REAL["full"], _REAL["ones"]
        arena._depth = 0


@contextlib.contextmanager
def guarded():
    arena = GuardArena()
    with _patched(arena):
        yield arena
