"""Model table: every family the framework knows, what serves it, and its state.  Reference: the
``sparkflash models`` subcommand (crates/sparkflash-cli/src/models.rs) and crates/sparkflash-model
architecture descriptors."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelEntry:
    name: str
    family: str
    status: str          # "device" = serves on the GPU engine, "oracle" = CPU reference + kernels, "planned"
    summary: str
    module: str


MODELS = {m.name: m for m in [
    ModelEntry("deepseek-v4.1-flash", "deepseek", "device", "CSA2 attention, mHC, 384-expert W4A8 MoE, DSpark drafter, Engram", "sparkflash_b200.models.deepseek_v41"),
    ModelEntry("tiny-csa2", "deepseek", "device", "6-layer test model with every layer mode of the flagship", "sparkflash_b200.models.deepseek_v41"),
    ModelEntry("tiny-mla-v3", "deepseek", "oracle", "classic MLA attention with absorbed decode, CPU oracle timing config", "sparkflash_b200.models.mla_v3"),
    ModelEntry("glm-5.3-flash", "glm", "oracle", "MLA with indexer-selected keys, noaux sigmoid router, shared expert; cached decode", "sparkflash_b200.models.glm"),
    ModelEntry("qwen3.8-flash-next", "qwen", "oracle", "gated delta-net / KDA linear attention + gated softmax attention + MoE; device rows step on the state kernels", "sparkflash_b200.models.qwen"),
    ModelEntry("inkling-2-small", "inkling", "oracle", "short conv, soft-capped windowed attention and SwiGLU, MoE with expert / intermediate / row splits; device rows step", "sparkflash_b200.models.inkling"),
    ModelEntry("dory-1.0-4b", "dory", "oracle", "latent-recurrence model, loops split over a ring pipeline of ranks", "sparkflash_b200.models.dory"),
    ModelEntry("dflash-block-drafter", "drafter", "oracle", "one-forward block drafter over a ring of captured target features", "sparkflash_b200.models.dflash"),
]}
