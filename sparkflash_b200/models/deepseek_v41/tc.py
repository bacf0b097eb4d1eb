"""Tensor-core arm attachments: TMA descriptors and scale-factor atoms for every quantised matrix of a
prepared model, plus the per-engine activation-side buffers and descriptors.

The CUDA-core arm reads row-major scales; tcgen05 block-scaled MMA wants them in 128x4 atoms
(csrc/codecs.h).  ``attach`` derives the atoms from the row-major scales once (for synthetic weights
both are a constant fill) and encodes one tensor map per weight matrix.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import codecs as C
from ...ops import native as N
from .prepare import DeviceWeights, LayerW


@dataclass
class TcMatrix:
    tmap: N.TensorMap
    atoms: torch.Tensor
    rows: int
    K: int
    fp4: bool


def _atoms(sf_rowmajor: torch.Tensor, rows: int, kb: int, const_code: int | None) -> torch.Tensor:
    if const_code is not None:
        return torch.full((C.sf_bytes(rows, kb),), const_code, dtype=torch.uint8, device=sf_rowmajor.device)
    return C.scales_to_prepared(sf_rowmajor.reshape(rows, kb), rows, 1)


def _matrix(w: torch.Tensor, sf: torch.Tensor, rows: int, K: int, fp4: bool, const_code: int | None) -> TcMatrix | None:
    row_bytes = K // 2 if fp4 else K
    if K % 128 or (fp4 and row_bytes % 32):
        return None
    flat = w.reshape(rows, row_bytes)
    return TcMatrix(N.TensorMap(flat, rows, K, row_bytes, 128, fp4=fp4), _atoms(sf, rows, K // 32, const_code), rows, K, fp4)


@dataclass
class TcLayer:
    wqkv_a: TcMatrix | None = None
    wq_b: TcMatrix | None = None
    wo_a: TcMatrix | None = None
    wo_b: TcMatrix | None = None
    s13: TcMatrix | None = None
    s2: TcMatrix | None = None
    w13: TcMatrix | None = None
    w2: TcMatrix | None = None


def attach(weights: DeviceWeights, synthetic: bool = False, layers=None, n_experts: int | None = None) -> list[TcLayer]:
    """Build the tensor-core attachments for every layer.  ``synthetic``: scales are a constant fill
    (2^-12 for FP8 blocks, 2^-7 for FP4 groups), so atoms are filled instead of re-ordered."""
    cfg = weights.cfg
    W = weights.world
    d, q, hd = cfg.hidden_size, cfg.q_lora_rank, cfg.head_dim
    gl, il = cfg.o_groups // W, weights.il or cfg.moe_inter // W
    ol, gin = cfg.o_lora_rank, cfg.group_in
    E = n_experts or weights.experts_local or cfg.n_routed_experts   # experts held by this rank (expert parallelism keeps a range)
    if n_experts:
        il = -(-(cfg.moe_inter // W) // 128) * 128                    # draft stages stay width-sliced in both modes
    c8 = 115 if synthetic else None
    c4 = 120 if synthetic else None
    out = []
    for L in (weights.layers if layers is None else layers):
        T = TcLayer()
        T.wqkv_a = _matrix(L.wqkv_a, L.wqkv_a_sf, q + hd, d, False, c8)
        T.wq_b = _matrix(L.wq_b, L.wq_b_sf, L.wq_b_rows, q, False, c8)
        if ol % 128 == 0:
            T.wo_a = _matrix(L.wo_a, L.wo_a_sf, gl * ol, gin, False, c8)
        T.wo_b = _matrix(L.wo_b, L.wo_b_sf, d, gl * ol, False, c8)
        if il % 128 == 0 and d % 128 == 0:
            T.s13 = _matrix(L.s13, L.s13_sf, 2 * il, d, False, c8)
            T.s2 = _matrix(L.s2, L.s2_sf, d, il, False, c8)
            T.w13 = _matrix(L.w13, L.w13_sf, E * 2 * il, d, True, c4)
            T.w2 = _matrix(L.w2, L.w2_sf, E * d, il, True, c4)
        out.append(T)
    return out


class TcBuffers:
    """Activation-side state of the tensor-core arm for one engine: scale atoms written by the
    producers, FP8 staging of bf16 activations, split-K scratch, and cached tensor maps."""

    def __init__(self, eng):
        cfg = eng.cfg
        dev = eng.dev
        R, d, q = eng.max_rows, cfg.hidden_size, cfg.q_lora_rank
        u8 = dict(dtype=torch.uint8, device=dev)
        k = cfg.top_k + 1
        RA = max(128, R)                                                              # atom blocks cover 128 rows each
        self.xs_atom = torch.full((C.sf_bytes(RA, d // 32),), 127, **u8)             # rows = tokens
        self.xs_atom_tok = torch.full((R, C.sf_bytes(1, d // 32)), 127, **u8)        # one set per token
        self.qr_atom = torch.full((C.sf_bytes(RA, q // 32),), 127, **u8)
        ao_k = eng.hl * cfg.head_dim
        nblk = max(1, (R + 63) // 64)        # one 128-row scale-atom block per 64 rows of a step (hi | lo fill a block)
        self.nblk = nblk
        self.ao_q = torch.zeros((128 * nblk, ao_k), **u8)                             # attention out: per 64 rows, 64 hi | 64 lo
        self.ao_atom_block = C.sf_bytes(128, ao_k // 32)
        self.ao_atom = torch.full((nblk * self.ao_atom_block,), 127, **u8)
        oa_k = eng.gl * cfg.o_lora_rank
        self.oa_q = torch.zeros((R, oa_k), **u8)
        self.oa_atom_block = C.sf_bytes(128, max(1, oa_k // 32))
        self.oa_atom = torch.full((nblk * self.oa_atom_block,), 127, **u8)
        self.act_sf = torch.full((R * k, C.sf_bytes(1, max(1, eng.il // 32))), 127, **u8)
        tiles_down = min(R, 128) * ((d + 127) // 128)
        n_floats = max(tiles_down * k * 128 * 16, 64 * 16 * 128 * 128)
        pair_tiles = 0
        if R > 128:
            # many-row steps: the grouped output projection keeps one fp32 tile per (column tile, group, 64-row block), and
            # a split dense projection one per (column tile, 128-row tile, split)
            pair_tiles = ((cfg.o_lora_rank + 127) // 128) * max(1, eng.gl) * nblk
            dense_tiles = 4 * ((max(d, eng.qfull_w) + 127) // 128) * ((R + 127) // 128)
            n_floats = max(n_floats, pair_tiles * 128 * 128, dense_tiles * 128 * 128)
        self.scratch = torch.zeros((n_floats,), dtype=torch.float32, device=dev)
        self.tickets = torch.zeros((max(tiles_down, 4096, pair_tiles),), dtype=torch.int32, device=dev)
        self._maps: dict[tuple[int, int, int], N.TensorMap] = {}

    def bmap(self, t: torch.Tensor, rows: int, K: int, box_rows: int) -> N.TensorMap:
        key = (t.data_ptr(), rows, box_rows)
        m = self._maps.get(key)
        if m is None:
            m = N.TensorMap(t, rows, K, K, box_rows)
            self._maps[key] = m
        return m


def pick_splits(tiles: int, ksteps: int, target_ctas: int = 296) -> int:
    s = max(1, min(ksteps, target_ctas // max(1, tiles)))
    return s


def pick_splits_bulk(tiles: int, ksteps: int) -> int:
    """Many-row launches (tiles of 128 token rows, two CTAs per SM): split the reduction only while the grid is short of
    one wave, and never below eight k-steps per CTA."""
    return max(1, min(4, ksteps // 8, 296 // max(1, tiles)))
