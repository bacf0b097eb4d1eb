"""Fused collectives over symmetric memory: the producer pushes, the consumer folds.

Every rank owns one symmetric allocation laid out as

    y      [2 sublayer kinds][W slots][R rows][d]   bf16   partial sublayer outputs, slot = producer rank
    best   [W][R] f32 + [W][R] i32                         per-rank sampler winners
    flags  [3][W] u32 (attention, ffn, sampler)            arrival epochs, one word per producer rank
    epoch  u32                                             this rank's step counter (bumped once per step)

and maps every other rank's allocation (CUDA IPC inside one box; peer stores travel over NVLink through
NVSwitch).  Producer kernels (the tcgen05 GEMM epilogue of ``wo_b`` and of the MoE down projection, or the
generic ``push_rows`` kernel) store this rank's partial into slot ``rank`` of *every* rank's ``y`` and then
raise flag ``rank`` everywhere; the mHC seam on each rank waits - with a time limit - on its own flags and
folds its own W slots in rank order.  That is the all-reduce: one kernel boundary, no separate collective.
Many-row partials can go in two shots instead (``push_rs`` / ``fold_push_rs``): reduce-scatter into rows [0, rs) of the
slots, fold on the owner, all-gather into rows [rs, 2 rs); a rank then sends 2 (W - 1) / W of a partial, not W - 1.

Reference behaviour replaced: crates/sparkflash-comm/src/device_reduce.rs:693-1082 (RunReduce),
rdma/write_exchange.rs, tp4_forward.rs:13234-13249 (one-shot exchange + opt_sum_ranks_bf16).

``FusedComm.local_group(W, ...)`` builds W communicators inside one process over one GPU's memory: the
multi-rank protocol can then be exercised on a single GPU by running the ranks' stages in lockstep.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_uint32, c_uint64, c_void_p

import torch

from .. import _lib
from ..ops import native as N

ATTN, FFN, BEST = 0, 1, 2


def _L():
    return _lib.cuda()


class SymmLayout:
    def __init__(self, W: int, R: int, d: int):
        self.W, self.R, self.d = W, R, d
        self.y_bytes = R * d * 2
        self.y_off = 0
        self.best_val_off = 2 * W * self.y_bytes
        self.best_id_off = self.best_val_off + W * R * 4
        self.flags_off = self.best_id_off + W * R * 4
        self.flags_off = (self.flags_off + 255) // 256 * 256
        self.epoch_off = self.flags_off + 3 * 256
        self.done_off = self.epoch_off + 256
        self.total = self.done_off + 256

    def y(self, base: int, kind: int, slot: int) -> int:
        return base + self.y_off + (kind * self.W + slot) * self.y_bytes

    def flag(self, base: int, kind: int, slot: int) -> int:
        return base + self.flags_off + kind * 256 + slot * 4

    def best_val(self, base: int, slot: int) -> int:
        return base + self.best_val_off + slot * self.R * 4

    def best_id(self, base: int, slot: int) -> int:
        return base + self.best_id_off + slot * self.R * 4


class FusedComm:
    name = "fused"

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.bases: list[int] = []     # base address of every rank's allocation as mapped in this process
        self.layout: SymmLayout | None = None
        self.engine = None
        self._owned = None
        self._opened: list[int] = []
        self.wait_ns = 2_000_000_000

    # ---- bootstrap -----------------------------------------------------------------------------------
    def attach(self, engine) -> None:
        """Allocate this rank's symmetric memory, exchange IPC handles through torch.distributed and map
        every peer."""
        import torch.distributed as dist
        self.engine = engine
        cfg = engine.cfg
        self.layout = SymmLayout(self.world, engine.max_rows, cfg.hidden_size)
        p = c_void_p()
        N._check(_L().sfb_symm_alloc(ctypes.byref(p), c_int64(self.layout.total)), "symm_alloc")
        self._owned = p.value
        handle = ctypes.create_string_buffer(64)
        N._check(_L().sfb_ipc_get_handle(c_void_p(self._owned), handle), "ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw))
        self.bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self._owned)
            else:
                q = c_void_p()
                N._check(_L().sfb_ipc_open_handle(ctypes.create_string_buffer(h, 64), ctypes.byref(q)), "ipc_open_handle")
                self.bases.append(q.value)
                self._opened.append(q.value)
        dist.barrier()

    @classmethod
    def local_group(cls, world: int, max_rows: int, d: int) -> list["FusedComm"]:
        """W communicators whose 'ranks' all live in this process on the current GPU (lockstep emulation)."""
        lay = SymmLayout(world, max_rows, d)
        bases = []
        for _ in range(world):
            p = c_void_p()
            N._check(_L().sfb_symm_alloc(ctypes.byref(p), c_int64(lay.total)), "symm_alloc")
            bases.append(p.value)
        out = []
        for r in range(world):
            c = cls(r, world)
            c.layout, c.bases, c._owned = lay, list(bases), bases[r]
            out.append(c)
        return out

    def attach_local(self, engine) -> None:
        self.engine = engine

    # ---- addresses -----------------------------------------------------------------------------------
    @property
    def base(self) -> int:
        return self.bases[self.rank]

    @property
    def epoch_ptr(self) -> int:
        return self.base + self.layout.epoch_off

    @property
    def done_ptr(self) -> int:
        return self.base + self.layout.done_off

    def push_targets(self, kind: int):
        """(this rank's slot on every rank, this rank's flag on every rank)."""
        lay = self.layout
        return ([lay.y(b, kind, self.rank) for b in self.bases], [lay.flag(b, kind, self.rank) for b in self.bases])

    def slots(self, kind: int):
        """(the W slots of this rank's own buffer, its W flags) - what the consumer reads."""
        lay = self.layout
        return ([lay.y(self.base, kind, s) for s in range(self.world)],
                [lay.flag(self.base, kind, s) for s in range(self.world)])

    # ---- per-step ------------------------------------------------------------------------------------
    def epoch_stride(self) -> int:
        return 2 * len(self.engine.w.layers) + 4

    def begin_step(self) -> None:
        N._check(_L().sfb_epoch_bump(c_void_p(self.epoch_ptr), c_uint32(self.epoch_stride()), N._stream()), "epoch_bump")

    def arm_umma_push(self, kind: int, epoch_add: int) -> None:
        outs, flags = self.push_targets(kind)
        N._check(_L().sfb_umma_set_push(N._ptr_array(outs), N._ptr_array(flags), c_int(self.world),
                                        c_void_p(self.epoch_ptr), c_uint32(epoch_add), c_void_p(self.done_ptr)),
                 "umma_set_push")

    def push(self, y: torch.Tensor, n: int, kind: int, epoch_add: int) -> None:
        outs, flags = self.push_targets(kind)
        nbytes = n * y.stride(0) * y.element_size()
        N._check(_L().sfb_push_rows(N._p(y), N._ptr_array(outs), N._ptr_array(flags), c_int(self.world),
                                    c_int64(nbytes), c_void_p(self.epoch_ptr), c_uint32(epoch_add),
                                    c_void_p(self.done_ptr), N._stream()), "push_rows")

    # ---- two-shot all-reduce of a many-row partial (reduce-scatter, fold on the owner, all-gather) --------------------
    @staticmethod
    def rs_rows(n: int, world: int) -> int:
        """Rows a rank owns in the two-shot exchange of an n-row partial."""
        return (n + world - 1) // world

    def push_rs(self, y: torch.Tensor, n: int, kind: int, epoch_add: int) -> None:
        """Shot 1: rows [j rs, (j + 1) rs) of this rank's partial go to rows [0, rs) of this rank's slot on rank j."""
        outs, flags = self.push_targets(kind)
        row_bytes = self.layout.d * 2
        N._check(_L().sfb_push_rows_rs(N._p(y), c_int64(y.stride(0) * y.element_size()), N._ptr_array(outs), N._ptr_array(flags),
                                       c_int(self.world), c_int(n), c_int(self.rs_rows(n, self.world)), c_int64(row_bytes),
                                       c_void_p(self.epoch_ptr), c_uint32(epoch_add), c_void_p(self.done_ptr), N._stream()),
                 "push_rows_rs")

    def fold_push_rs(self, n: int, kind: int, epoch_wait: int, epoch_raise: int, status=None) -> None:
        """Shot 2: this rank adds the W slots' rows it owns (rank order, fp32, one bf16 rounding) and stores the result to rows
        [rs, 2 rs) of its slot on every rank; the flags go to the second epoch."""
        rs = self.rs_rows(n, self.world)
        rows = max(0, min(rs, n - self.rank * rs))
        slots, flags = self.slots(kind)
        outs, oflags = self.push_targets(kind)
        N._check(_L().sfb_fold_push_rs(N._ptr_array(slots), N._ptr_array(flags), N._ptr_array(outs), N._ptr_array(oflags),
                                       c_int(self.world), c_int(rows), c_int(rs), c_int64(self.layout.d * 2), c_void_p(self.epoch_ptr),
                                       c_uint32(epoch_wait), c_uint32(epoch_raise), c_uint64(self.wait_ns), c_void_p(self.done_ptr),
                                       N._p(status), N._stream()), "fold_push_rs")

    def push_best(self, best_val: torch.Tensor, best_id: torch.Tensor, n: int, epoch_add: int) -> None:
        """Publish this rank's sampler winners to every rank (values then ids; the flag follows the ids)."""
        lay = self.layout
        R = lay.R
        zero_flags = [self.base + lay.done_off + 128] * self.world   # scratch word: the first push raises no real flag
        N._check(_L().sfb_push_rows(N._p(best_val[self.rank]), N._ptr_array([lay.best_val(b, self.rank) for b in self.bases]),
                                    N._ptr_array(zero_flags), c_int(self.world), c_int64(R * 4), c_void_p(self.epoch_ptr),
                                    c_uint32(epoch_add), c_void_p(self.done_ptr), N._stream()), "push_best_val")
        N._check(_L().sfb_push_rows(N._p(best_id[self.rank]), N._ptr_array([lay.best_id(b, self.rank) for b in self.bases]),
                                    N._ptr_array([lay.flag(b, BEST, self.rank) for b in self.bases]), c_int(self.world),
                                    c_int64(R * 4), c_void_p(self.epoch_ptr), c_uint32(epoch_add),
                                    c_void_p(self.done_ptr), N._stream()), "push_best_id")

    def best_views(self):
        lay = self.layout
        return (self.base + lay.best_val_off, self.base + lay.best_id_off,
                [lay.flag(self.base, BEST, s) for s in range(self.world)])

    def close(self) -> None:
        """Unmap the peers' allocations and free this rank's own (idempotent).  Across processes every rank first
        reaches a barrier, so that nobody frees memory a peer's kernel may still be storing into; a rank that finds
        the process group gone already (fail-stop teardown) skips the barrier."""
        if self._owned is None and not self._opened:
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
            _L().sfb_ipc_close_handle(c_void_p(p))
        self._opened = []
        if self._owned is not None:
            _L().sfb_symm_free(c_void_p(self._owned))
            self._owned = None
        self.bases = []
