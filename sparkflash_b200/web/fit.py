"""Fit estimator: will this model, context and lane count fit on N GPUs of a given size?  Per-GPU bytes of the
prepared weights (tensor-parallel slices, padded expert width), the position-addressed KV regions per lane, and
the step workspace.  Reference: crates/sparkflash-web/src/fit.rs, crates/sparkflash-device/src/budget.rs,
docs/architecture/08-kv-footprint.md."""
from __future__ import annotations

from dataclasses import dataclass

from ..config import ModelConfig


@dataclass
class FitReport:
    world: int
    weights_gb: float
    kv_gb_per_lane: float
    kv_gb: float
    workspace_gb: float
    engram_gb: float
    total_gb: float
    capacity_gb: float
    fits: bool
    max_lanes_that_fit: int

    def as_dict(self) -> dict:
        return self.__dict__.copy()


def weights_bytes_per_gpu(c: ModelConfig, world: int) -> int:
    d, V, W = c.hidden_size, c.vocab_size, world
    hd, q = c.head_dim, c.q_lora_rank
    il = -(-(c.moe_inter // W) // 128) * 128
    attn = (q + hd) * d + (c.n_heads // W) * hd * q + (c.o_groups // W) * c.o_lora_rank * c.group_in + d * (c.o_groups // W) * c.o_lora_rank
    attn = attn * (1 + 1 / 32)                                   # FP8 + one scale byte per 32
    experts = c.n_routed_experts * 3 * il * d * (0.5 + 1 / 32)   # FP4 + scales
    shared = c.n_shared_experts * 3 * il * d * (1 + 1 / 32)
    router = c.n_routed_experts * d * 2
    per_layer = attn + experts + shared + router + 3 * d * 4
    embed_head = V * d * 2 + (V // W) * d * 2
    return int(c.n_layers * per_layer + embed_head)


def kv_bytes_per_lane(c: ModelConfig, context: int, max_rows: int = 64) -> int:
    ring = 1
    while ring < c.window + max_rows:
        ring *= 2
    total = c.n_layers * ring * (c.head_dim + c.head_dim // 32)          # FP8 window rings
    for l in range(c.n_layers):
        if c.is_kv_source(l):
            r = c.ratio(l)
            entries = context // r + 1
            total += entries * (c.head_dim // 2 + c.head_dim // 16 + c.index_head_dim // 2 + c.index_head_dim // 32)
            if r > 1:
                total += ring * 2 * c.head_dim * 4
    return int(total)


def estimate(c: ModelConfig, world: int, context: int, lanes: int, gpu_gb: float = 180.0, engram_resident: bool = False,
             reserve_gb: float = 6.0) -> FitReport:
    w = weights_bytes_per_gpu(c, world) / 1e9
    kvl = kv_bytes_per_lane(c, context) / 1e9
    ws = (64 * c.hidden_size * c.hc_mult * 4 * 6 + 64 * c.vocab_size // world * 4 + 256e6) / 1e9
    eng = sum(c.engram_rows) * 272 / world / 1e9 if engram_resident else 0.0
    total = w + kvl * lanes + ws + eng + reserve_gb
    room = gpu_gb - (w + ws + eng + reserve_gb)
    return FitReport(world, round(w, 2), round(kvl, 3), round(kvl * lanes, 2), round(ws, 2), round(eng, 2), round(total, 2), gpu_gb,
                     total <= gpu_gb, max(0, int(room / kvl)) if kvl > 0 else 0)
