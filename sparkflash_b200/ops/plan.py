"""Planning layer between a model description and the kernels: which part runs which kernel, and which form a
collective takes.

Three pieces:

* the **parts catalogue**: every op of the forward, the kernel entry points (exported C symbols of
  ``libsfb_cuda.so``) that implement it on each arm, and the shapes each entry point accepts;
* the **resolver**: checks that every catalogued entry point exists in the loaded library (a renamed or dropped
  symbol is found at start-up, not at the first request that needs it) and picks the entry point for a concrete
  (op, arm, rows) query;
* the **step plan**: for a rows step of n rows on a given arm and world size, the variant of every stage (few-row
  or many-row kernels, segment size of the grouped experts, form of the collective).  The engine's row thresholds
  live here, so that the engine, the tests and the benchmarks agree on where the variants change.

There is one target, sm_100a; the catalogue has no per-target dimension.

Reference: crates/sparkflash-ops/src/parts.rs:51,2079 (parts catalogue), resolver/, engine_plan/,
collective.rs:29-150 (CollectiveKind, CollectivePlan), crates/sparkflash-ops/src/tp.rs:23-51,
docs/engine/02-execution-plan.md:167-178 (Architecture -> TpPlan -> EnginePlan -> KernelResolver).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


# ---- collectives ---------------------------------------------------------------------------------------------
class CollectiveKind(enum.Enum):
    NONE = "none"                      # one rank
    ONE_SHOT = "one_shot"              # every producer pushes its partial to every rank; the consumer folds W slots in rank order
    TWO_SHOT = "two_shot"              # reduce-scatter by rows, fold on the owner, all-gather of the folded rows
    REDUCE_SCATTER = "reduce_scatter"  # sequence-parallel seam, first half
    ALL_GATHER = "all_gather"          # sequence-parallel seam, second half
    OVERLAPPED = "overlapped"          # bulk chunks: the collective of chunk i runs beside the GEMMs of chunk i + 1
    NCCL = "nccl"                      # library all-reduce (baseline arm)


@dataclass(frozen=True)
class CollectivePlan:
    """Form of the per-sublayer reduction of n rows of d bf16 columns over W ranks.

    One-shot moves (W - 1) x the data but has one hop of latency, so it wins while the message is small; above
    ``two_shot_rows`` rows the reduce-scatter / all-gather form moves 2 (W - 1) / W x the data instead."""
    kind: CollectiveKind
    world: int
    rows: int
    d: int
    chunks_in_flight: int = 1

    @property
    def bytes_sent_per_rank(self) -> int:
        msg = self.rows * self.d * 2
        W = self.world
        if self.kind in (CollectiveKind.NONE,) or W <= 1:
            return 0
        if self.kind is CollectiveKind.ONE_SHOT:
            return msg * (W - 1)
        if self.kind in (CollectiveKind.TWO_SHOT, CollectiveKind.OVERLAPPED, CollectiveKind.NCCL):
            return 2 * msg * (W - 1) // W
        return msg * (W - 1) // W          # one half of a sequence-parallel seam

    def rows_owned(self, rank: int) -> tuple[int, int]:
        """Row range a rank folds in the two-shot / reduce-scatter forms (equal blocks, the tail on the last ranks short)."""
        per = -(-self.rows // max(1, self.world))
        lo = min(self.rows, rank * per)
        return lo, min(self.rows, lo + per)

    def link_seconds(self, link_bytes_per_s: float = 770e9) -> float:
        """Time the bytes need on one GPU's NVLink at the measured peer-copy rate (the communication roofline)."""
        return self.bytes_sent_per_rank / link_bytes_per_s


# reference: SPARKFLASH_TWO_SHOT_ROWS = 16 on RoCE.  Over NVLink the two extra kernels of the two-shot form cost more than the
# links save below 8 ranks (32K prefill 0.94x at 2 ranks, 0.98x at 4), so the engine takes it from 512 rows and 8 ranks on
TWO_SHOT_ROWS = 512
TWO_SHOT_WORLD = 8


def plan_collective(rows: int, d: int, world: int, arm: str = "fused", two_shot_rows: int = TWO_SHOT_ROWS,
                    bulk_chunks: int = 1, two_shot_world: int = TWO_SHOT_WORLD) -> CollectivePlan:
    if world <= 1:
        return CollectivePlan(CollectiveKind.NONE, 1, rows, d)
    if arm == "nccl":
        return CollectivePlan(CollectiveKind.NCCL, world, rows, d)
    if bulk_chunks > 1:
        return CollectivePlan(CollectiveKind.OVERLAPPED, world, rows, d, chunks_in_flight=min(3, bulk_chunks))
    if rows < two_shot_rows or world < two_shot_world:
        return CollectivePlan(CollectiveKind.ONE_SHOT, world, rows, d)
    return CollectivePlan(CollectiveKind.TWO_SHOT, world, rows, d)


# ---- parts catalogue ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Part:
    """One op of the forward and the entry points that implement it.  ``entry``: variant name -> exported symbol."""
    name: str
    stage: str                               # seam | attention | ffn | head | kv | index | comm | draft | vision | misc
    entry: dict
    tensor_cores: bool = False
    collective_after: bool = False
    note: str = ""


def _p(name, stage, entry, **kw) -> Part:
    return Part(name, stage, dict(entry), **kw)


CATALOGUE: tuple[Part, ...] = (
    _p("embed", "misc", {"rows": "sfb_embed", "image_rows": "sfb_embed_override"}),
    _p("rope_table", "misc", {"rows": "sfb_rope_table"}),
    _p("seam_fold", "seam", {"cluster": "sfb_seam_fold"}, note="one entry point; one block per row above 128 rows"),
    _p("seam_coef", "seam", {"rows": "sfb_seam_coef", "gemm": "sfb_umma_bf16", "finish": "sfb_seam_coef_finish"}, tensor_cores=True),
    _p("dense_projection", "attention", {"skinny": "sfb_umma_dense", "pair": "sfb_umma_dense_pair", "bulk": "sfb_umma_bulk",
                                         "pair_bulk": "sfb_umma_pair_bulk", "cuda_core": "sfb_gemv", "no_alloc": "sfb_umma_dense_noalloc"},
       tensor_cores=True, collective_after=True),
    _p("bf16_projection", "ffn", {"gemv": "sfb_gemv", "gemm": "sfb_umma_bf16"}, tensor_cores=True,
       note="router gate, compressor / indexer side projections, vocabulary head, predictor dots"),
    _p("qkv_post", "kv", {"rows": "sfb_qkv_post"}),
    _p("compress_append", "kv", {"rows": "sfb_compress_append"}),
    _p("index_query", "index", {"cuda_core": "sfb_index_q", "fp4": "sfb_index_q4"}),
    _p("index_scores", "index", {"cuda_core": "sfb_index_scores", "tc": "sfb_index_scores_tc"}, tensor_cores=True),
    _p("candidate_blocks", "index", {"blockmax": "sfb_hsi_blockmax", "mark": "sfb_hsi_mark"}),
    _p("select_topk", "index", {"row": "sfb_select_topk", "long": "sfb_select_topk_long"}),
    _p("attention", "attention", {"rows": "sfb_attn_rows_range", "tc": "sfb_attn_tc"}, tensor_cores=True),
    _p("router", "ffn", {"topk": "sfb_router_topk", "remap": "sfb_expert_remap"}),
    _p("moe_plan", "ffn", {"plan": "sfb_moe_plan", "permute": "sfb_moe_permute", "combine": "sfb_moe_combine"}),
    _p("moe_gate_up", "ffn", {"token": "sfb_umma_gate_up", "grouped": "sfb_umma_gate_up_grouped", "cuda_core": "sfb_moe_gate_up"},
       tensor_cores=True),
    _p("moe_down", "ffn", {"token": "sfb_umma_down", "grouped": "sfb_umma_down_grouped", "cuda_core": "sfb_moe_down"},
       tensor_cores=True, collective_after=True),
    _p("activation_quant", "misc", {"rows": "sfb_quant_rows"}),
    _p("head_sample", "head", {"sample": "sfb_sample", "fold": "sfb_sample_fold", "markov": "sfb_markov_bias"}),
    _p("taps", "draft", {"mean": "sfb_tap_mean"}),
    _p("push", "comm", {"rows": "sfb_push_rows", "arm": "sfb_umma_set_push", "gather": "sfb_umma_set_gather", "fold": "sfb_fold_slots",
                        "epoch": "sfb_epoch_bump", "wait": "sfb_wait_flags"}),
    _p("symmetric_memory", "comm", {"alloc": "sfb_symm_alloc", "free": "sfb_symm_free", "export": "sfb_ipc_get_handle",
                                    "open": "sfb_ipc_open_handle", "close": "sfb_ipc_close_handle"}),
    _p("expert_exchange", "comm", {"dispatch": "sfb_ep_dispatch", "combine": "sfb_ep_combine"},
       note="token-sharded all-to-all around the grouped expert GEMMs"),
    _p("lanes", "kv", {"pool": "sfb_lanepool_create", "region": "sfb_laneregion_create", "ensure": "sfb_laneregion_ensure",
                       "release": "sfb_laneregion_release", "copy_prefix": "sfb_laneregion_copy_prefix"}),
    _p("engram", "misc", {"gather": "sfb_engram_gather", "gate": "sfb_engram_gate_bf16"}),
    _p("vision", "vision", {"prepare": "sfb_vision_prepare", "rope": "sfb_vision_rope", "unfold": "sfb_vision_unfold3"}),
    _p("other_families", "misc", {"delta_rule": "sfb_delta_rule", "short_conv": "sfb_short_conv", "softcap": "sfb_softcap",
                                  "softcapped_swiglu": "sfb_softcapped_swiglu"}),
    _p("trace", "misc", {"mark": "sfb_trace_mark"}),
    _p("tensor_map", "misc", {"encode": "sfb_tmap_encode"}),
)


class KernelResolver:
    """Binds the catalogue to a loaded library.  ``missing()`` lists catalogued symbols the library does not export."""

    def __init__(self, lib=None, catalogue: tuple[Part, ...] = CATALOGUE):
        self.catalogue = {p.name: p for p in catalogue}
        self._lib = lib

    def _library(self):
        if self._lib is None:
            from .. import _lib
            self._lib = _lib.cuda()
        return self._lib

    def has(self, symbol: str) -> bool:
        try:
            getattr(self._library(), symbol)
            return True
        except AttributeError:
            return False

    def missing(self) -> list[tuple[str, str, str]]:
        out = []
        for p in self.catalogue.values():
            for variant, sym in p.entry.items():
                if not self.has(sym):
                    out.append((p.name, variant, sym))
        return out

    def resolve(self, part: str, variant: str) -> str:
        p = self.catalogue.get(part)
        if p is None:
            raise KeyError(f"no part named {part!r}")
        sym = p.entry.get(variant)
        if sym is None:
            raise KeyError(f"part {part!r} has no variant {variant!r} (has {sorted(p.entry)})")
        if not self.has(sym):
            raise LookupError(f"{part}.{variant}: the library does not export {sym}")
        return sym


# ---- step plan ---------------------------------------------------------------------------------------------------
MANY_ROWS = 128            # above: token-tiled GEMMs, bf16-GEMM coefficients, one-block-per-row fold
TC_ATTENTION_ROWS = 64     # above: attention on tcgen05 (a tolerance arm)
GROUP_MIN_ROWS = 4         # from here on the experts run grouped by expert
GROUP_WIDE_ROWS = 512      # from here on segments hold up to 64 pairs
HEAD_TC_MIN_ROWS = 1
SELECT_LONG_ENTRIES = 32768   # rows longer than this (and few rows) use the chunked select


@dataclass(frozen=True)
class StepPlan:
    rows: int
    arm: str
    world: int
    dense: str                 # skinny | bulk | cuda_core
    attention: str             # rows | tc
    wo_a: str                  # pair | pair_bulk | cuda_core
    coef: str                  # rows | gemm
    fold: str                  # cluster | rows
    moe: str                   # token | seg16 | seg64 | cuda_core
    gate: str                  # gemv | gemm
    head: str                  # gemv | gemm
    index_scores: str          # cuda_core | tc
    collective: CollectivePlan = field(default=None)

    def kernels_per_layer(self, index_layer: bool = False, kv_source: bool = False) -> int:
        """Launches of one layer on the main stream (the coefficient kernels run on the side stream)."""
        n = 2                                     # two seam folds
        n += 1                                    # wqkv_a
        n += 1 if (kv_source or index_layer) else 0      # side projections of the compressor / indexer
        n += 1 + (1 if kv_source else 0)          # qkv_post, compress_append
        n += 1                                    # wq_b
        n += 3 if index_layer else 0              # index query, scores, select
        n += 3                                    # attention, wo_a, wo_b
        n += 2                                    # gate, router
        n += {"token": 2, "cuda_core": 2}.get(self.moe, 5)
        return n


def plan_step(rows: int, arm: str = "tc", world: int = 1, d: int = 5120, head_dim: int = 512, collective_arm: str = "fused",
              context_entries: int = 0) -> StepPlan:
    tc = arm == "tc"
    many = rows > MANY_ROWS
    return StepPlan(
        rows=rows, arm=arm, world=world,
        dense=("bulk" if many else "skinny") if tc else "cuda_core",
        attention="tc" if (tc and rows > TC_ATTENTION_ROWS and head_dim == 512) else "rows",
        wo_a=("pair_bulk" if rows > TC_ATTENTION_ROWS else "pair") if tc else "cuda_core",
        coef="gemm" if (tc and many) else "rows",
        fold="rows" if many else "cluster",
        moe=("cuda_core" if not tc else "token" if rows < GROUP_MIN_ROWS else "seg64" if rows >= GROUP_WIDE_ROWS else "seg16"),
        gate="gemm" if (tc and many) else "gemv",
        head="gemm" if (tc and HEAD_TC_MIN_ROWS <= rows <= 128) else "gemv",
        index_scores="tc" if tc else "cuda_core",
        collective=plan_collective(rows, d, world, collective_arm),
    )
