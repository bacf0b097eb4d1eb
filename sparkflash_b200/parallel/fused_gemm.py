"""Fused GEMM + collective operators on the tcgen05 block-scaled GEMM (csrc/k_umma.cu) and the symmetric heap.

* ``RowParallelLinear`` (GEMM -> all-reduce or reduce-scatter): every rank multiplies its K-shard; the GEMM
  epilogue stores the bf16 partial tile by tile straight into the consumer's slot over NVLink (all ranks for
  all-reduce, only the owner of the token row for reduce-scatter) and raises an arrival flag when its last tile is
  out; the consumer kernel waits on its own flags with a time limit and folds the slots in rank order in fp32,
  adds the residual, applies RMSNorm and re-quantises for the next GEMM.
* ``ColumnParallelLinear`` (all-gather -> GEMM): activations are sharded along the hidden dimension (the output
  layout of the reduce-scatter above, transposed roles); the GEMM's TMA producer reads each K-slab directly from
  the rank that owns it (plain loads from peer memory, no multicast), so the gather overlaps the MMAs slab by
  slab and no gathered copy is ever materialised.

Waits are bounded; buffers are double-buffered by step parity, which orders re-use without extra handshakes:
a rank that passed step i's wait knows every peer finished step i-1.
Reference behaviour replaced: crates/sparkflash-comm/src/device_reduce.rs:693-1082 (RunReduce all-reduce /
reduce-scatter / all-gather around cuBLAS-free GEMMs), tp4_forward.rs reduce_rows:13112, SP prefill seams.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_uint32, c_uint64, c_void_p

import torch

from .. import _lib, codecs as C
from ..ops import native as N
from .symm import SymmHeap


def _L():
    return _lib.cuda()


def _maps_device(maps: list[N.TensorMap]) -> torch.Tensor:
    """W tensor maps copied into one 64-byte aligned device buffer."""
    raw = bytearray()
    for m in maps:
        raw += ctypes.string_at(m.ptr, 128)
    buf = torch.empty((len(raw) + 64,), dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 64
    view = buf[off:off + len(raw)]
    view.copy_(torch.frombuffer(raw, dtype=torch.uint8))
    view._keep = buf
    return view


def tensor_map_at(addr: int, rows: int, K: int, box_rows: int) -> N.TensorMap:
    class _Addr:
        def __init__(self, a): self._a = a
        def data_ptr(self): return self._a
    return N.TensorMap(_Addr(addr), rows, K, K, box_rows)


class _Base:
    def __init__(self, heap: SymmHeap, M: int, wait_ns: int = 1_000_000_000):
        self.heap, self.rank, self.world, self.M = heap, heap.rank, heap.world, M
        self.wait_ns = wait_ns
        self.step = 0
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.epoch = torch.zeros(1, dtype=torch.int32, device="cuda")     # incremented on the device every step

    def _bump(self):
        N._check(_L().sfb_epoch_bump(N._p(self.epoch), c_uint32(1), N._stream()), "epoch_bump")

    def check(self):
        st = self.status.tolist()
        if st[0]:
            raise RuntimeError(f"fused collective: device status code={st[0]} where={st[1]} detail=({st[2]}, {st[3]})")


class RowParallelLinear(_Base):
    """y = sum_r x_r @ W_r^T over ranks; ``mode`` "ar" (every rank gets all M rows) or "rs" (rank r gets rows
    [r*M/W, (r+1)*M/W)).  Weight shard: FP8 codes [N, K/W] with UE8M0 scales per 32x32 block [N/32, K/W/32] (the checkpoint's form)."""

    def __init__(self, heap: SymmHeap, w_q: torch.Tensor, w_sf: torch.Tensor, M: int, mode: str = "ar", heap_offset: int = 0,
                 norm_w: torch.Tensor | None = None, eps: float = 1e-6, **kw):
        super().__init__(heap, M, **kw)
        self.N, self.Kl = w_q.shape
        W = self.world
        # all-reduce of many rows: two shots - every row goes to one owner (reduce-scatter), the owner folds it and
        # sends the folded row to everyone (all-gather): 2 (W - 1) / W of the data crosses the links instead of W - 1
        self.two_shot = mode == "ar" and W > 1 and M >= self.TWO_SHOT_ROWS and M % W == 0
        self.ar_rows = M
        if self.two_shot:
            mode = "rs"
        self.mode = mode
        if mode == "rs" and M % W:
            raise ValueError("reduce-scatter needs M divisible by the world size")
        self.rows_out = M // W if mode == "rs" else M
        self.w_q = w_q
        self.w_atoms = C.scales_to_prepared(w_sf, self.N, 32).cuda()
        self.tmap_a = N.TensorMap(w_q, self.N, self.Kl, self.Kl, 128)
        self.NP = N.umma_np(min(M, 128))
        Mp = max(self.NP, (M + 127) // 128 * 128)
        self.x_q = torch.zeros((Mp, self.Kl), dtype=torch.uint8, device="cuda")
        self.x_atom = torch.full((C.sf_bytes(Mp, self.Kl // 32),), 127, dtype=torch.uint8, device="cuda")
        self.tmap_b = N.TensorMap(self.x_q, Mp, self.Kl, self.Kl, self.NP)
        # symmetric layout: [2 parities][W slots][rows_out, N] bf16 | flags [2][W] u32 | done u32
        self.slot_bytes = self.rows_out * self.N * 2
        self.off_slots = heap_offset
        self.off_flags = heap_offset + 2 * W * self.slot_bytes
        self.off_done = self.off_flags + 2 * 256
        self.bytes = self.off_done + 256 - heap_offset
        if self.two_shot:      # | gathered rows [2][M, N] bf16 | gather flags [2][W] | done
            self.off_gather = self.off_done + 256
            self.off_gflags = self.off_gather + 2 * M * self.N * 2
            self.off_gdone = self.off_gflags + 2 * 256
            self.bytes = self.off_gdone + 256 - heap_offset
            self.gflag_ptrs = [torch.tensor([heap.base + self.off_gflags + par * 256 + r * 4 for r in range(W) if r != self.rank],
                                            dtype=torch.int64, device="cuda") for par in range(2)]
        tiles = ((self.N + 127) // 128) * ((M + self.NP - 1) // self.NP)
        ksteps = self.Kl // 128
        # few rows: split K until every SM has a CTA or two; 32..128 rows: only while the tiles alone leave most SMs idle
        # few rows: split K until every SM has a CTA or two; from 32 rows on the split's reduce costs more than it gains
        # (measured again with 148 / tiles splits at 64 rows: 42 instead of 37 us)
        self.splits = max(1, min(ksteps // 4, 296 // max(1, tiles))) if M < 32 else 1
        self.splits = int(os.environ.get("SFB_FUSED_SPLITS", self.splits))
        self.scratch = torch.zeros((tiles * self.splits * 128 * self.NP,), dtype=torch.float32, device="cuda") if self.splits > 1 else None
        self.tickets = torch.zeros((max(tiles, 1),), dtype=torch.int32, device="cuda")
        self.norm_w, self.eps = norm_w, eps
        self.out = torch.empty((self.rows_out, self.N), dtype=torch.bfloat16, device="cuda")
        self.out_sum = torch.empty_like(self.out)

    TWO_SHOT_ROWS = 512

    @classmethod
    def heap_bytes(cls, M: int, Nn: int, W: int, mode: str) -> int:
        two = mode == "ar" and W > 1 and M >= cls.TWO_SHOT_ROWS and M % W == 0
        rows = M // W if (mode == "rs" or two) else M
        return 2 * W * rows * Nn * 2 + 2 * 256 + 256 + (2 * M * Nn * 2 + 2 * 256 + 256 if two else 0)

    def _slot(self, base: int, parity: int, r: int) -> int:
        return base + self.off_slots + (parity * self.world + r) * self.slot_bytes

    def _flag(self, base: int, parity: int, r: int) -> int:
        return base + self.off_flags + parity * 256 + r * 4

    def produce(self, x: torch.Tensor) -> None:
        """x bf16 [M, K/W]: quantise, multiply, push the partial to the consumers, raise the flags."""
        self.step += 1
        par = self.step & 1
        N.quant_rows_bump(x, self.x_q, None, self.x_atom, self.M, self.Kl, self.epoch)      # quantise and count the step in one launch
        h = self.heap
        outs = [self._slot(b, par, self.rank) for b in h.bases]
        flags = [self._flag(b, par, self.rank) for b in h.bases]
        N._check(_L().sfb_umma_set_push(N._ptr_array(outs), N._ptr_array(flags), c_int(self.world), N._p(self.epoch), c_uint32(0),
                                        c_void_p(h.base + self.off_done)), "umma_set_push")
        N._check(_L().sfb_umma_bulk(c_void_p(self.tmap_a.ptr), c_void_p(self.tmap_b.ptr), N._p(self.w_atoms), c_int(self.Kl // 128),
                                    N._p(self.x_atom), c_int(self.Kl // 128), c_int(self.M), c_int(self.NP), c_int(self.N), c_int(self.Kl),
                                    c_int(self.splits), N._p(self.scratch), N._p(self.tickets), None, None, c_int64(self.N), None, c_int(0),
                                    None, c_int(0), c_int(self.rows_out if self.mode == "rs" else 0), N._p(self.status), N._stream()), "umma_bulk")

    def consume(self, residual: torch.Tensor | None = None, out_q: torch.Tensor | None = None, out_atom: torch.Tensor | None = None,
                wait: bool = True) -> torch.Tensor:
        par = self.step & 1
        b = self.heap.base
        slots = [self._slot(b, par, r) for r in range(self.world)]
        flags = [self._flag(b, par, r) for r in range(self.world)]
        out = self.out
        if self.two_shot:
            # fold this rank's rows straight into its part of the gathered buffer, send that part to every peer, wait for theirs
            h, W, rows = self.heap, self.world, self.rows_out
            g_off = self.off_gather + par * self.ar_rows * self.N * 2
            own_off = g_off + self.rank * rows * self.N * 2
            out = h.view(own_off, (rows, self.N), torch.bfloat16)
            if residual is not None and residual.shape[0] == self.ar_rows:
                residual = residual[self.rank * rows:(self.rank + 1) * rows]
        N._check(_L().sfb_fold_slots(N._ptr_array(slots), N._ptr_array(flags), c_int(self.world), c_int(self.rows_out), c_int(self.N),
                                     c_int64(self.N), N._p(self.epoch), c_uint32(0), c_uint64(self.wait_ns), N._p(residual), N._p(self.norm_w),
                                     c_float(self.eps), N._p(self.out_sum), N._p(out), N._p(out_q), N._p(out_atom), N._p(self.status),
                                     N._stream()), "fold_slots")
        if not self.two_shot:
            return self.out
        self._gather_push(out, own_off, par)
        return self.gathered() if wait else None

    def _gather_push(self, out, own_off, par):
        h, W, rows = self.heap, self.world, self.rows_out
        peers = [r for r in range(W) if r != self.rank]
        dst = [h.bases[r] + own_off for r in peers]
        gfl = [h.bases[r] + self.off_gflags + par * 256 + self.rank * 4 for r in peers]
        N._check(_L().sfb_push_rows(N._p(out), N._ptr_array(dst), N._ptr_array(gfl), c_int(len(peers)), c_int64(rows * self.N * 2),
                                    N._p(self.epoch), c_uint32(0), c_void_p(h.base + self.off_gdone), N._stream()), "push_rows")

    def gathered(self) -> torch.Tensor:
        """Second half of the two-shot all-reduce: wait (bounded) for every peer's folded rows; returns all M rows.  Separate
        from ``consume(wait=False)`` so that ranks emulated on one GPU can all push before anyone waits."""
        par = self.step & 1
        W = self.world
        N._check(_L().sfb_wait_flags(N._p(self.gflag_ptrs[par]), c_int(W - 1), N._p(self.epoch), c_uint32(0), c_uint64(self.wait_ns),
                                     N._p(self.status), N._stream()), "wait_flags")
        return self.heap.view(self.off_gather + par * self.ar_rows * self.N * 2, (self.ar_rows, self.N), torch.bfloat16)

    def forward(self, x, residual=None):
        self.produce(x)
        return self.consume(residual)


class ColumnParallelLinear(_Base):
    """y_r = x @ W_r^T with x [M, K] held as W shards along K, one per rank (FP8 + atoms).
    Weight shard: FP8 codes [N/W, K] with UE8M0 scales per 32x32 block.

    ``mode="gather"`` (default): every rank keeps W local slots; ``publish`` quantises this rank's shard into its own slot
    and pushes it (codes and atoms, one contiguous block) into slot ``rank`` of every peer, then raises its flag there.
    The GEMM reads local memory only, and its producer warp waits for a shard's flag just before the first load from it,
    so the math on the shards that are there overlaps the transfers still in flight and every byte crosses NVLink once.
    ``mode="remote"``: the shards stay where they are and the GEMM's TMA loads read them from the owners' memory (every
    weight-tile CTA fetches the remote tile again: fine for a few rows, link-bound for thousands)."""

    def __init__(self, heap: SymmHeap, w_q: torch.Tensor, w_sf: torch.Tensor, M: int, heap_offset: int = 0, mode: str = "gather", **kw):
        super().__init__(heap, M, **kw)
        if mode not in ("gather", "remote"):
            raise ValueError(f"unknown mode {mode!r}")
        self.mode = mode
        self.Nl, self.K = w_q.shape
        W = self.world
        self.Kl = self.K // W
        if self.Kl % 128:
            raise ValueError("K / world must be a multiple of 128")
        self.w_q = w_q
        self.w_atoms = C.scales_to_prepared(w_sf, self.Nl, 32).cuda()
        self.tmap_a = N.TensorMap(w_q, self.Nl, self.K, self.K, 128)
        self.NP = N.umma_np(min(M, 128))
        self.Mp = max(self.NP, (M + 127) // 128 * 128)
        self.xq_bytes = self.Mp * self.Kl
        self.atom_bytes = (C.sf_bytes(self.Mp, self.Kl // 32) + 255) // 256 * 256
        self.slot_bytes = self.xq_bytes + self.atom_bytes
        slots = W if mode == "gather" else 1
        # symmetric layout: [2 parities][slots] (x_q shard | atoms) | flags [2][W] | dummy 16 B | done
        self.off_x = heap_offset
        self.off_flags = heap_offset + 2 * slots * self.slot_bytes
        self.off_dummy = self.off_flags + 2 * 256
        self.off_done = self.off_dummy + 256
        self.bytes = self.off_done + 256 - heap_offset
        h = heap
        self.maps, self.sfb_ptrs, self.local_q, self.local_atom, self.slot_off = [], [], [], [], []
        for par in range(2):
            base_par = self.off_x + par * slots * self.slot_bytes
            if mode == "gather":      # slot r of THIS rank's memory holds rank r's shard
                addrs = [h.base + base_par + r * self.slot_bytes for r in range(W)]
                own = base_par + self.rank * self.slot_bytes
            else:                     # the one slot of rank r's memory
                addrs = [b + base_par for b in h.bases]
                own = base_par
            ms = [tensor_map_at(a, self.Mp, self.Kl, self.NP) for a in addrs]
            self._keep_maps = getattr(self, "_keep_maps", []) + ms
            self.maps.append(_maps_device(ms))
            self.sfb_ptrs.append([a + self.xq_bytes for a in addrs])
            self.slot_off.append(own)
            self.local_q.append(h.view(own, (self.Mp, self.Kl), torch.uint8))
            self.local_atom.append(h.view(own + self.xq_bytes, (self.atom_bytes,), torch.uint8))
            self.local_atom[-1].fill_(127)
        tiles = ((self.Nl + 127) // 128) * ((M + self.NP - 1) // self.NP)
        ksteps = self.K // 128
        # few tiles and a long reduction: split K (this GEMM has no push, so from 32 rows on the partials are added by the
        # separate reduce grid, which is cheap; the row-parallel operator's in-kernel reduce is not, see above)
        if M < 32:
            self.splits = max(1, min(ksteps // 4, 296 // max(1, tiles)))
        elif M <= 128:
            self.splits = max(1, min(ksteps // 4, 148 // max(1, tiles)))
        else:
            self.splits = 1
        self.scratch = torch.zeros((tiles * self.splits * 128 * self.NP,), dtype=torch.float32, device="cuda") if self.splits > 1 else None
        self.tickets = torch.zeros((max(tiles, 1),), dtype=torch.int32, device="cuda")
        self.out = torch.empty((M, self.Nl), dtype=torch.bfloat16, device="cuda")
        self.flag_addr = [[h.base + self.off_flags + par * 256 + r * 4 for r in range(W)] for par in range(2)]
        self.flag_ptrs = [torch.tensor(self.flag_addr[par], dtype=torch.int64, device="cuda") for par in range(2)]
        self._dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")

    @staticmethod
    def heap_bytes(M: int, K: int, W: int, mode: str = "gather") -> int:
        Mp = max(16, (M + 127) // 128 * 128)
        slots = W if mode == "gather" else 1
        return 2 * slots * (Mp * (K // W) + (C.sf_bytes(Mp, K // W // 32) + 255) // 256 * 256) + 2 * 256 + 512

    def publish(self, x_shard: torch.Tensor) -> None:
        """x_shard bf16 [M, K/W]: quantise into this rank's slot, (gather mode) push the slot to every peer, and tell every
        rank it is there."""
        self.step += 1
        par = self.step & 1
        N.quant_rows_bump(x_shard, self.local_q[par], None, self.local_atom[par], self.M, self.Kl, self.epoch)
        h = self.heap
        flags = [b + self.off_flags + par * 256 + self.rank * 4 for b in h.bases]
        if self.mode == "gather":
            # own rank's entry copies the slot onto itself only for W == 1; otherwise the list holds the peers
            peers = [r for r in range(self.world) if r != self.rank] or [self.rank]
            dst = [h.bases[r] + self.slot_off[par] for r in peers]
            src = h.view(self.slot_off[par], (self.slot_bytes,), torch.uint8)
            N._check(_L().sfb_push_rows(N._p(src), N._ptr_array(dst), N._ptr_array([flags[r] for r in peers]), c_int(len(peers)),
                                        c_int64(self.slot_bytes), N._p(self.epoch), c_uint32(0), c_void_p(h.base + self.off_done),
                                        N._stream()), "push_rows")
        else:
            dst = [b + self.off_dummy for b in h.bases]
            N._check(_L().sfb_push_rows(N._p(self._dummy), N._ptr_array(dst), N._ptr_array(flags), c_int(self.world), c_int64(16), N._p(self.epoch),
                                        c_uint32(0), c_void_p(h.base + self.off_done), N._stream()), "push_rows")

    def gemm(self) -> torch.Tensor:
        par = self.step & 1
        if self.mode == "gather":
            # no separate wait: the kernel's producer warp waits for shard r's flag right before it first reads slot r
            gate = [0 if r == self.rank else self.flag_addr[par][r] for r in range(self.world)]
            N._check(_L().sfb_umma_set_gather(N._ptr_array(gate), c_int(self.world), N._p(self.epoch), c_uint32(0), c_uint64(self.wait_ns)),
                     "umma_set_gather")
        else:
            N._check(_L().sfb_wait_flags(N._p(self.flag_ptrs[par]), c_int(self.world), N._p(self.epoch), c_uint32(0), c_uint64(self.wait_ns),
                                         N._p(self.status), N._stream()), "wait_flags")
        N._check(_L().sfb_umma_bulk(c_void_p(self.tmap_a.ptr), None, N._p(self.w_atoms), c_int(self.K // 128), None, c_int(self.Kl // 128),
                                    c_int(self.M), c_int(self.NP), c_int(self.Nl), c_int(self.K), c_int(self.splits), N._p(self.scratch),
                                    N._p(self.tickets), N._p(self.out), None, c_int64(self.Nl), N._p(self.maps[par]), c_int(self.Kl),
                                    N._ptr_array(self.sfb_ptrs[par]), c_int(self.world), c_int(0), N._p(self.status), N._stream()), "umma_bulk")
        return self.out

    def forward(self, x_shard):
        self.publish(x_shard)
        return self.gemm()


def _demo(argv=None) -> None:
    """Lockstep demonstration on one GPU (W virtual ranks): ``python -m sparkflash_b200.parallel.fused_gemm --m 8192``.
    Runs a few GEMM -> reduce steps and one all-gather -> GEMM step; a small fixed workload for profilers."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--mode", default="rs", choices=["ar", "rs"])
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args(argv)
    W, H, M = a.world, a.hidden, a.m
    g = torch.Generator().manual_seed(0)
    qr, sr = C.weight_quant_fp8_block32(torch.randn(H, H // W, generator=g) * 0.02)
    qc, sc = C.weight_quant_fp8_block32(torch.randn(H // W, H, generator=g) * 0.02)
    mode = a.mode if M % W == 0 else "ar"
    heaps = SymmHeap.local_group(W, RowParallelLinear.heap_bytes(M, H, W, mode))
    rows = [RowParallelLinear(heaps[r], qr.cuda(), sr, M, mode, norm_w=torch.ones(H, device="cuda")) for r in range(W)]
    heaps2 = SymmHeap.local_group(W, ColumnParallelLinear.heap_bytes(M, H, W))
    cols = [ColumnParallelLinear(heaps2[r], qc.cuda(), sc, M) for r in range(W)]
    x = torch.randn(M, H // W, generator=g).to(torch.bfloat16).cuda()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for s in range(a.steps):
        if s == a.steps - 1:
            ev[0].record()
        for o in rows:
            o.produce(x)
        for o in rows:
            o.consume(wait=False)
        for o in rows:
            if o.two_shot:
                o.gathered()
        for o in cols:
            o.publish(x)
        for o in cols:
            o.gemm()
    ev[1].record()
    torch.cuda.synchronize()
    for o in rows + cols:
        o.check()
    print(f"fused_gemm demo: M={M} hidden={H} W={W} mode={mode}: last step {ev[0].elapsed_time(ev[1]) * 1e3:.0f} us for {W} virtual ranks (eager launches)")


if __name__ == "__main__":
    _demo()
