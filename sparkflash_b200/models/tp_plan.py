"""Tensor-parallel plan of the DeepSeek-V4.1-Flash architecture: how every tensor of a layer is placed on W ranks, and
what that costs per rank.

    replicated    wq_a, wkv, norms, mHC predictor parameters, router gate and bias, indexer and compressor weights,
                  attention sinks of the rank's heads, the draft stages' main projection
    column split  wq_b (heads), wo_a (output groups), expert and shared w1 / w3 (intermediate width), embedding and
                  vocabulary head (vocabulary)
    row split     wo_b, expert and shared w2
    expert split  (expert-parallel mode) whole routed experts per rank; the shared expert stays replicated

The plan is the single description the converter, the loader, the fit estimator and the tests read; ``bytes_per_rank``
is what the prepared rank file weighs, ``collectives_per_step`` what the ledger expects.

Reference: crates/sparkflash-device/src/resident.rs:238-339 (shard classification), crates/sparkflash-model/src/tp_plan,
docs/design.md:24-45, docs/architecture/00-overview.md:181-200 (byte budget).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass


class Split(enum.Enum):
    REPLICATED = "replicated"
    COLUMN = "column"          # output dimension divided over the ranks
    ROW = "row"                # reduction dimension divided: the outputs are partial sums, reduced by the next seam
    EXPERT = "expert"          # whole experts per rank


@dataclass(frozen=True)
class TensorPlan:
    name: str
    split: Split
    shape: tuple[int, ...]     # full (unsharded) shape; for experts the per-expert shape
    bits: int                  # bits per element in the stored layout (scales included where blocked)
    count: int = 1             # tensors of this kind per layer (experts)

    def bytes_per_rank(self, world: int) -> float:
        n = 1
        for s in self.shape:
            n *= s
        total = n * self.bits / 8 * self.count
        return total if self.split is Split.REPLICATED else total / world


# bits per element with the block scales folded in
FP8_BLOCK = 8 + 8 / 1024          # one UE8M0 byte per 32 x 32 block
FP4_ROW32 = 4 + 8 / 32            # one UE8M0 byte per 32 elements
BF16, F32 = 16, 32


@dataclass(frozen=True)
class TpPlan:
    world: int
    moe_mode: str                 # "tp": experts sliced by width; "ep": whole experts per rank
    layer: tuple[TensorPlan, ...]
    globals_: tuple[TensorPlan, ...]
    n_layers: int
    heads_per_rank: int
    groups_per_rank: int
    inter_per_rank: int
    vocab_per_rank: int
    experts_per_rank: int

    def bytes_per_rank(self) -> float:
        return self.n_layers * sum(t.bytes_per_rank(self.world) for t in self.layer) + sum(t.bytes_per_rank(self.world) for t in self.globals_)

    def collectives_per_step(self, sampled: bool = True) -> int:
        return 0 if self.world == 1 else 2 * self.n_layers + (1 if sampled else 0)

    def table(self) -> list[dict]:
        return [{"tensor": t.name, "split": t.split.value, "shape": list(t.shape), "count": t.count,
                 "gb_per_rank_per_layer": round(t.bytes_per_rank(self.world) / 1e9, 4)} for t in self.layer]


def plan(cfg, world: int, moe_mode: str = "tp") -> TpPlan:
    """The plan for ``cfg`` (config.ModelConfig) on ``world`` ranks; raises when the architecture does not divide."""
    for what, v in (("heads", cfg.n_heads), ("output groups", cfg.o_groups), ("vocabulary", cfg.vocab_size)):
        if v % world:
            raise ValueError(f"{what} ({v}) do not divide over {world} ranks")
    if moe_mode == "ep":
        if cfg.n_routed_experts % world:
            raise ValueError(f"{cfg.n_routed_experts} experts do not divide over {world} ranks")
        il, el, esplit = cfg.moe_inter, cfg.n_routed_experts // world, Split.EXPERT
    else:
        if cfg.moe_inter % world or (cfg.moe_inter // world) % 32:
            raise ValueError(f"expert width {cfg.moe_inter} does not divide over {world} ranks in multiples of 32")
        il, el, esplit = cfg.moe_inter // world, cfg.n_routed_experts, Split.COLUMN
    d, q, hd = cfg.hidden_size, cfg.q_lora_rank, cfg.head_dim
    mix = (2 + cfg.hc_mult) * cfg.hc_mult
    E = cfg.n_routed_experts
    L = (
        TensorPlan("wq_a|wkv", Split.REPLICATED, (q + hd, d), FP8_BLOCK),
        TensorPlan("wq_b", Split.COLUMN, (cfg.n_heads * hd, q), FP8_BLOCK),
        TensorPlan("wo_a", Split.COLUMN, (cfg.o_groups * cfg.o_lora_rank, cfg.group_in), FP8_BLOCK),
        TensorPlan("wo_b", Split.ROW, (d, cfg.o_groups * cfg.o_lora_rank), FP8_BLOCK),
        TensorPlan("attn_sink", Split.COLUMN, (cfg.n_heads,), F32),
        TensorPlan("norms", Split.REPLICATED, (2 * d + q + hd,), F32),
        TensorPlan("hc_fn", Split.REPLICATED, (2 * mix, cfg.hc_mult * d), F32),
        TensorPlan("gate", Split.REPLICATED, (E, d), BF16),
        TensorPlan("gate_bias", Split.REPLICATED, (2 * E,), F32),
        TensorPlan("shared.w13", Split.COLUMN, (2 * cfg.moe_inter, d), FP8_BLOCK),
        TensorPlan("shared.w2", Split.ROW, (d, cfg.moe_inter), FP8_BLOCK),
        TensorPlan("expert.w13", esplit, (2 * cfg.moe_inter, d), FP4_ROW32, count=E),
        TensorPlan("expert.w2", esplit if moe_mode == "ep" else Split.ROW, (d, cfg.moe_inter), FP4_ROW32, count=E),
    )
    if moe_mode == "ep":       # the replicated shared expert is whole on every rank
        L = tuple(TensorPlan(t.name, Split.REPLICATED, t.shape, t.bits, t.count) if t.name.startswith("shared.") else t for t in L)
    G = (
        TensorPlan("embed", Split.REPLICATED, (cfg.vocab_size, d), BF16),        # replicated on B200: 1.3 GB buys one exchange less per step
        TensorPlan("head", Split.COLUMN, (cfg.vocab_size, d), BF16),
        TensorPlan("final_norm", Split.REPLICATED, (d,), F32),
    )
    return TpPlan(world, moe_mode, L, G, cfg.n_layers, cfg.n_heads // world, cfg.o_groups // world, il, cfg.vocab_size // world, el)
