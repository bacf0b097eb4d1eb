"""Symmetric heap: the same byte layout allocated on every rank and mapped by every rank (CUDA IPC inside one
box; traffic goes over NVLink through NVSwitch).  ``SymmHeap.local_group`` builds W heaps inside one process on
one GPU so that multi-rank protocols can be run in lockstep without several GPUs.  Reference behaviour replaced:
crates/sparkflash-comm/src/rdma/write_exchange.rs (registered exchange regions), oneshot/ (peer-mapped buffers).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int64, c_void_p

from .. import _lib
from ..ops import native as N


class SymmHeap:
    def __init__(self, rank: int, world: int, nbytes: int):
        self.rank, self.world, self.nbytes = rank, world, (nbytes + 255) // 256 * 256
        self.bases: list[int] = []
        self._owned: int | None = None
        self._opened: list[int] = []

    def _alloc(self) -> int:
        p = c_void_p()
        N._check(_lib.cuda().sfb_symm_alloc(ctypes.byref(p), c_int64(self.nbytes)), "symm_alloc")
        return p.value

    def attach(self) -> "SymmHeap":
        """Allocate, exchange IPC handles through torch.distributed, map every peer."""
        import torch.distributed as dist
        L = _lib.cuda()
        self._owned = self._alloc()
        handle = ctypes.create_string_buffer(64)
        N._check(L.sfb_ipc_get_handle(c_void_p(self._owned), handle), "ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw))
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self._owned)
            else:
                q = c_void_p()
                N._check(L.sfb_ipc_open_handle(ctypes.create_string_buffer(h, 64), ctypes.byref(q)), "ipc_open_handle")
                self.bases.append(q.value)
                self._opened.append(q.value)
        dist.barrier()
        return self

    @classmethod
    def local_group(cls, world: int, nbytes: int) -> list["SymmHeap"]:
        heaps = [cls(r, world, nbytes) for r in range(world)]
        bases = [h._alloc() for h in heaps]
        for r, h in enumerate(heaps):
            h.bases, h._owned = list(bases), bases[r]
        return heaps

    @property
    def base(self) -> int:
        return self.bases[self.rank]

    def view(self, offset: int, shape, dtype):
        """A torch tensor over this rank's own heap."""
        import torch
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty((), dtype=dtype).element_size()
        class _I:
            pass
        o = _I()
        o.__cuda_array_interface__ = {"shape": (n * esz,), "strides": None, "typestr": "|u1", "data": (self.base + offset, False), "version": 3}
        t = torch.as_tensor(o, device="cuda")
        self._keep = getattr(self, "_keep", []) + [o]
        return t.view(dtype).reshape(shape)

    def close(self) -> None:
        """Unmap the peers' heaps and free this rank's own (idempotent; a barrier first when peers are mapped)."""
        if getattr(self, "_owned", None) is None and not self._opened:
            return
        import torch
        torch.cuda.synchronize()
        if self._opened:
            try:
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    dist.barrier()
            except Exception:
                pass
        for p in self._opened:
            _lib.cuda().sfb_ipc_close_handle(c_void_p(p))
        self._opened = []
        self._keep = []
        if getattr(self, "_owned", None) is not None:
            _lib.cuda().sfb_symm_free(c_void_p(self._owned))
            self._owned = None
        self.bases = []
