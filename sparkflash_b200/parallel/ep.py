"""Expert-parallel MoE with fused all-to-all dispatch and combine (csrc/k_ep.cu) around the tcgen05 grouped MoE GEMMs.

Tokens are sharded over ranks, experts are sharded over ranks.  One step on every rank:

    dispatch(x, ids, wts)   route + MXFP8 quant + push rows to the experts' ranks, counts + flag
    experts()               wait for all arrivals, run gate/up (+ clamp-SwiGLU x route weight + FP8 quant) and down on
                            the received rows (W4A8 block-scaled GEMMs; empty slots are skipped inside the kernels)
    combine()               push every output row back to its token's rank, flag
    fold(addend)            wait, add the top-k rows of each token in k order (+ shared expert / residual)

Every wait is time-limited and reports through the status word.  Buffers alternate by step parity.
Reference behaviour replaced: Inkling's ``ExpertSplit::Experts`` exchange (crates/sparkflash-model-inkling2/src/
tensor.rs:49-78) and the slot exchanges of the TP4 step (docs/rdma-exchange.md:141-145).
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_uint32, c_uint64, c_void_p

import torch

from .. import _lib, codecs as C
from ..ops import native as N
from .symm import SymmHeap


def _L():
    return _lib.cuda()


class EpLayout:
    def __init__(self, W: int, t: int, d: int, top_k: int):
        self.W, self.t, self.d, self.top_k = W, t, d, top_k
        self.cap = t * top_k                       # rows one source can send to one destination
        self.KB = d // 32
        a = lambda n: (n + 255) // 256 * 256
        self.q_bytes = a(W * self.cap * d)
        self.s_bytes = a(W * self.cap * self.KB)
        self.rec_bytes = a(W * self.cap * 16)
        self.comb_bytes = a(t * top_k * d * 2)
        self.par_bytes = self.q_bytes + self.s_bytes + self.rec_bytes + self.comb_bytes + 4 * 256
        self.total = 2 * self.par_bytes + 512

    def off(self, par: int, what: str) -> int:
        base = par * self.par_bytes
        o = {"q": 0, "s": self.q_bytes, "rec": self.q_bytes + self.s_bytes, "comb": self.q_bytes + self.s_bytes + self.rec_bytes}
        tail = self.q_bytes + self.s_bytes + self.rec_bytes + self.comb_bytes
        o.update(count=tail, flag_d=tail + 256, flag_c=tail + 512)
        return base + o[what]


class EpMoE:
    def __init__(self, heap: SymmHeap, t: int, d: int, top_k: int, n_experts: int, inter: int, w13_q, w13_sf, w2_q, w2_sf,
                 limit: float = 10.0, wait_ns: int = 1_000_000_000):
        """w13_q: packed FP4 [E_local * 2 * inter, d/2] (gate rows then up rows per expert), w13_sf [rows, d/32];
        w2_q: [E_local * d, inter/2], w2_sf [rows, inter/32] - this rank's experts."""
        self.heap, self.rank, self.W = heap, heap.rank, heap.world
        self.t, self.d, self.top_k, self.E, self.inter, self.limit = t, d, top_k, n_experts, inter, limit
        self.epr = n_experts // self.W
        self.lay = EpLayout(self.W, t, d, top_k)
        L = self.lay
        self.wait_ns = wait_ns
        dev = "cuda"
        self.w13_q, self.w2_q = w13_q, w2_q
        self.t13 = N.TensorMap(w13_q, self.epr * 2 * inter, d, d // 2, 128, fp4=True)
        self.t2 = N.TensorMap(w2_q, self.epr * d, inter, inter // 2, 128, fp4=True)
        self.a13 = C.scales_to_prepared(w13_sf, self.epr * 2 * inter, 1).to(dev)
        self.a2 = C.scales_to_prepared(w2_sf, self.epr * d, 1).to(dev)
        rows = self.W * L.cap
        self.rows = rows
        self.atom_bytes = C.sf_bytes(1, L.KB)
        self.ids = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        self.wts = torch.zeros((rows,), dtype=torch.float32, device=dev)
        self.atoms = torch.full((rows, self.atom_bytes), 127, dtype=torch.uint8, device=dev)
        self.act_q = torch.zeros((rows + 16, inter), dtype=torch.uint8, device=dev)
        self.act_s = torch.zeros((rows, inter // 32), dtype=torch.uint8, device=dev)
        self.act_sf = torch.full((rows, C.sf_bytes(1, inter // 32)), 127, dtype=torch.uint8, device=dev)
        self.y = torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)
        self.scratch = torch.zeros((1024,), dtype=torch.float32, device=dev)
        self.tickets = torch.zeros((rows * (d // 128) + 16,), dtype=torch.int32, device=dev)
        self.counters = torch.zeros((8,), dtype=torch.int32, device=dev)
        self.done = torch.zeros((2,), dtype=torch.int32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.zeros((t, d), dtype=torch.bfloat16, device=dev)
        self.step = 0
        self.tmap_x, self.tmap_act, self.recv_q, self.recv_s, self.recv_rec, self.recv_cnt, self.comb = [], [], [], [], [], [], []
        for par in range(2):
            rq = heap.view(L.off(par, "q"), (rows + 0, d), torch.uint8)
            self.recv_q.append(rq)
            self.recv_s.append(heap.view(L.off(par, "s"), (rows, L.KB), torch.uint8))
            self.recv_rec.append(heap.view(L.off(par, "rec"), (rows, 4), torch.int32))
            self.recv_cnt.append(heap.view(L.off(par, "count"), (self.W,), torch.int32))
            self.comb.append(heap.view(L.off(par, "comb"), (t, top_k, d), torch.bfloat16))
            self.tmap_x.append(N.TensorMap(rq, rows, d, d, 16))
        self.tmap_act = N.TensorMap(self.act_q, rows + 16, inter, inter, 16)

    @staticmethod
    def heap_bytes(W: int, t: int, d: int, top_k: int) -> int:
        return EpLayout(W, t, d, top_k).total

    def _addr(self, r: int, par: int, what: str, extra: int = 0) -> int:
        return self.heap.bases[r] + self.lay.off(par, what) + extra

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor) -> None:
        """x bf16 [t, d]; ids int32 [t, top_k] global expert ids; wts f32 [t, top_k]."""
        L, W, me = self.lay, self.W, self.rank
        self.step += 1
        par = self.step & 1
        N._check(_L().sfb_epoch_bump(N._p(self.epoch), c_uint32(1), N._stream()), "epoch_bump")
        q = [self._addr(r, par, "q", me * L.cap * self.d) for r in range(W)]
        s = [self._addr(r, par, "s", me * L.cap * L.KB) for r in range(W)]
        rec = [self._addr(r, par, "rec", me * L.cap * 16) for r in range(W)]
        cnt = [self._addr(r, par, "count", me * 4) for r in range(W)]
        fl = [self._addr(r, par, "flag_d", me * 4) for r in range(W)]
        N._check(_L().sfb_ep_dispatch(N._p(x), N._p(ids), N._p(wts), c_int(x.shape[0]), c_int(self.d), c_int(self.top_k), c_int(self.epr),
                                      c_int(W), c_int(me), c_int(L.cap), N._ptr_array(q), N._ptr_array(s), N._ptr_array(rec), N._ptr_array(cnt),
                                      N._ptr_array(fl), N._p(self.counters), N._p(self.done[0:]), N._p(self.epoch), c_uint32(0), N._stream()),
                 "ep_dispatch")

    def experts(self) -> None:
        L, W, me = self.lay, self.W, self.rank
        par = self.step & 1
        fl = [self._addr(me, par, "flag_d", r * 4) for r in range(W)]
        N._check(_L().sfb_ep_plan(N._p(self.recv_rec[par]), N._p(self.recv_cnt[par]), N._ptr_array(fl), c_int(W), c_int(L.cap), N._p(self.ids),
                                  N._p(self.wts), N._p(self.recv_s[par]), N._p(self.atoms), c_int(L.KB), c_int(self.atom_bytes), N._p(self.epoch),
                                  c_uint32(0), c_uint64(self.wait_ns), N._p(self.status), N._stream()), "ep_plan")
        N.umma_gate_up(self.t13, None, self.tmap_x[par], self.a13, None, self.atoms, self.ids, self.wts, self.act_q, self.act_s, self.act_sf,
                       self.rows, 1, 1, self.d, self.inter, self.limit, status=self.status)
        N.umma_down(self.t2, None, self.tmap_act, self.a2, None, self.act_sf, self.ids, self.y, None, self.d, self.scratch, self.tickets,
                    self.rows, 1, 1, self.d, self.inter, status=self.status)

    def combine(self) -> None:
        L, W, me = self.lay, self.W, self.rank
        par = self.step & 1
        comb = [self._addr(r, par, "comb") for r in range(W)]
        fl = [self._addr(r, par, "flag_c", me * 4) for r in range(W)]
        N._check(_L().sfb_ep_combine(N._p(self.y), N._p(self.recv_rec[par]), N._p(self.recv_cnt[par]), c_int(W), c_int(L.cap), c_int(self.d),
                                     c_int(self.top_k), c_int(me), N._ptr_array(comb), N._ptr_array(fl), N._p(self.done[1:]), N._p(self.epoch),
                                     c_uint32(0), N._stream()), "ep_combine")

    def fold(self, n_tok: int, addend: torch.Tensor | None = None) -> torch.Tensor:
        W, me = self.W, self.rank
        par = self.step & 1
        fl = [self._addr(me, par, "flag_c", r * 4) for r in range(W)]
        N._check(_L().sfb_ep_fold(N._p(self.comb[par]), N._p(addend), N._p(self.out), N._ptr_array(fl), c_int(W), c_int(n_tok), c_int(self.d),
                                  c_int(self.top_k), N._p(self.epoch), c_uint32(0), c_uint64(self.wait_ns), N._p(self.status), N._stream()), "ep_fold")
        return self.out[:n_tok]

    def check(self) -> None:
        st = self.status.tolist()
        if st[0]:
            raise RuntimeError(f"expert-parallel exchange: device status code={st[0]} where={st[1]} detail=({st[2]}, {st[3]})")
