"""Typed configuration: model architecture, engine settings and the environment-override table.

Reference behaviour: ``reference/hf_config.json`` (architecture constants),
``crates/sparkflash-model/src/profile.rs:606`` (one table of env overrides, unknown values refused),
``sparkflash.toml.example`` (sections).  Unknown keys and unknown env values raise at start-up; a
digest of the effective settings is compared across ranks at bootstrap.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Any


@dataclass
class ModelConfig:
    name: str = "deepseek-v4.1-flash"
    vocab_size: int = 129280
    hidden_size: int = 5120
    n_layers: int = 40
    n_heads: int = 64
    head_dim: int = 512
    rope_dim: int = 64
    q_lora_rank: int = 1280
    o_groups: int = 8
    o_lora_rank: int = 1024
    moe_inter: int = 2304
    n_routed_experts: int = 384
    n_shared_experts: int = 1
    top_k: int = 6
    route_scale: float = 1.5
    swiglu_limit: float = 10.0
    norm_eps: float = 1e-20
    window: int = 128
    rope_theta: float = 10000.0
    compress_rope_theta: float = 160000.0
    yarn_factor: float = 16.0
    yarn_orig_max_pos: int = 65536
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    compress_ratios: list[int] = field(default_factory=lambda: [0, 0] + [2] * 18 + [1] * 20)
    kv_source_layers: list[int] = field(default_factory=lambda: [2, 8, 14, 20])
    index_source_layers: list[int] = field(default_factory=lambda: [2, 8, 14, 20, 24, 28, 32, 36])
    candidate_source_layer: int = 20
    candidate_topk_blocks: int = 2048
    candidate_block_size: int = 8
    index_n_heads: int = 32
    index_head_dim: int = 128
    index_topk: int = 512
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    max_positions: int = 1048576
    # Engram n-gram memory
    engram_layers: list[int] = field(default_factory=lambda: [1, 14])
    engram_rows: list[int] = field(default_factory=lambda: [384006168, 384016682])
    engram_max_ngram: int = 4
    engram_n_heads: int = 8
    engram_head_dim: int = 256
    engram_compressed_vocab: int = 99092
    engram_vocab: int = 16000000          # bucket primes are drawn above this value
    engram_enabled: bool = False
    # DSpark / MTP drafter
    n_mtp_stages: int = 3
    dspark_block: int = 5
    dspark_noise_token: int = 128799
    dspark_taps: list[int] = field(default_factory=lambda: [37, 38, 39])
    dspark_markov_rank: int = 256
    dspark_n_experts: int = 128
    dspark_top_k: int = 3
    # special ids
    bos_id: int = 0
    eos_id: int = 1
    pad_id: int = 2
    image_token_id: int = 129264
    # "csa2" = the V4.1 attention (latent KV, window + compressed sparse); "mla_v3" = classic MLA
    attention_kind: str = "csa2"
    # mla_v3 only
    kv_lora_rank: int = 64
    qk_nope_dim: int = 32
    v_head_dim: int = 32

    def __post_init__(self) -> None:
        if len(self.compress_ratios) < self.n_layers:
            raise ValueError("compress_ratios shorter than n_layers")
        if self.hidden_size % 32 or self.moe_inter % 32 or self.q_lora_rank % 32:
            raise ValueError("hidden, moe_inter and q_lora_rank must be multiples of 32")
        if (self.n_heads * self.head_dim) % self.o_groups:
            raise ValueError("heads*head_dim must divide by o_groups")

    # ---- per-layer predicates (docs/engine/01-forward-order.md section 4) -----------------------
    def ratio(self, layer: int) -> int:
        return self.compress_ratios[layer] if layer < self.n_layers else 0

    def is_kv_source(self, layer: int) -> bool:
        return layer in self.kv_source_layers and layer < self.n_layers

    def is_index_source(self, layer: int) -> bool:
        return layer in self.index_source_layers and layer < self.n_layers

    def uses_candidates(self, layer: int) -> bool:
        return 0 <= self.candidate_source_layer < layer

    def kv_owner(self, layer: int) -> int:
        """Layer whose compressed KV cache this layer reads (-1 when ratio is 0)."""
        if self.ratio(layer) == 0:
            return -1
        own = [l for l in self.kv_source_layers if l <= layer and l < self.n_layers]
        return own[-1] if own else -1

    def index_owner(self, layer: int) -> int:
        if self.ratio(layer) == 0:
            return -1
        own = [l for l in self.index_source_layers if l <= layer and l < self.n_layers]
        return own[-1] if own else -1

    @property
    def group_in(self) -> int:
        return self.n_heads * self.head_dim // self.o_groups

    def digest(self) -> str:
        return hashlib.sha256(json.dumps(dataclasses.asdict(self), sort_keys=True).encode()).hexdigest()[:16]


def full_config(**over: Any) -> ModelConfig:
    return dataclasses.replace(ModelConfig(), **over)


def reduced_config(n_routed_experts: int = 160, n_layers: int = 40, **over: Any) -> ModelConfig:
    """Full per-token shapes with a smaller resident expert pool and/or fewer layers, for GPUs that
    cannot hold the 307 GB model.  Per-token work (top-6 experts of width 2304, every projection) is
    unchanged by the expert count; fewer layers keep the per-layer mode pattern of the first ones."""
    c = ModelConfig()
    ratios = c.compress_ratios[:n_layers]
    return dataclasses.replace(
        c, name=f"deepseek-v4.1-flash-L{n_layers}-E{n_routed_experts}", n_layers=n_layers,
        n_routed_experts=n_routed_experts, compress_ratios=ratios,
        dspark_taps=[max(0, n_layers - 3), max(0, n_layers - 2), n_layers - 1], **over)


def tiny_config(**over: Any) -> ModelConfig:
    """Scaled-down CSA2 model used by the oracle-parity tests: every layer mode appears once."""
    base = dict(
        name="tiny-csa2", vocab_size=1024, hidden_size=256, n_layers=6, n_heads=4, head_dim=64,
        rope_dim=32, q_lora_rank=128, o_groups=2, o_lora_rank=64, moe_inter=128,
        n_routed_experts=8, top_k=2, window=8, compress_ratios=[0, 2, 2, 1, 1, 1],
        kv_source_layers=[1, 3], index_source_layers=[1, 3, 5], candidate_source_layer=3,
        candidate_topk_blocks=6, candidate_block_size=2, index_n_heads=4, index_head_dim=32,
        index_topk=8, max_positions=4096, yarn_orig_max_pos=256, engram_layers=[],
        engram_rows=[], dspark_taps=[3, 4, 5], dspark_markov_rank=32, dspark_n_experts=4,
        dspark_top_k=2, dspark_noise_token=1000, image_token_id=1023, dspark_block=5,
    )
    if over.pop("engram", False):
        # small n-gram memory on two layers: bucket primes just above 2000, the released row width and head count
        base.update(engram_enabled=True, engram_layers=[1, 3], engram_vocab=2000, engram_compressed_vocab=1024, engram_n_heads=8,
                    engram_head_dim=256, engram_max_ngram=4)
    base.update(over)
    return dataclasses.replace(ModelConfig(), **base)


def tiny_mla_v3_config(**over: Any) -> ModelConfig:
    """The literal small decoder used for the CPU-path check: 2 layers, hidden 256, MLA with 4 heads
    (q_lora 128, kv_lora 64, rope 32, nope 32, v 32), 8 experts top-2 + 1 shared, FFN 128, vocab 1024."""
    base = dict(
        name="tiny-mla-v3", attention_kind="mla_v3", vocab_size=1024, hidden_size=256, n_layers=2,
        n_heads=4, head_dim=64, rope_dim=32, q_lora_rank=128, kv_lora_rank=64, qk_nope_dim=32,
        v_head_dim=32, o_groups=1, o_lora_rank=64, moe_inter=128, n_routed_experts=8, top_k=2,
        window=4096, compress_ratios=[0, 0], kv_source_layers=[], index_source_layers=[],
        candidate_source_layer=-1, hc_mult=1, max_positions=4096, engram_layers=[], engram_rows=[],
        n_mtp_stages=0, dspark_taps=[], image_token_id=1023, dspark_noise_token=1000,
    )
    base.update(over)
    return dataclasses.replace(ModelConfig(), **base)


@dataclass
class ParallelConfig:
    world: int = 1
    rank: int = 0
    moe_mode: str = "tp"  # "tp": every rank holds an inter-slice of every expert; "ep": whole experts
    collective: str = "fused"  # "fused" (own NVLink kernels) | "nccl" (baseline arm)

    def validate(self, m: ModelConfig) -> None:
        w = self.world
        if m.n_heads % w or m.o_groups % w and w % m.o_groups:
            raise ValueError(f"world {w} does not divide heads/groups")
        if self.moe_mode == "tp" and (m.moe_inter // w) % 32:
            raise ValueError("inter slice must be a multiple of 32")
        if self.moe_mode == "ep" and m.n_routed_experts % w:
            raise ValueError("experts must divide by world for EP")
        if self.moe_mode not in ("tp", "ep") or self.collective not in ("fused", "nccl"):
            raise ValueError("unknown moe_mode/collective")


@dataclass
class EngineConfig:
    max_lanes: int = 32
    queue_depth: int = 64
    max_rows: int = 128           # rows per step: prompt chunks and verify rows (64-row blocks inside the step above 64)
    prefill_chunk: int = 4096
    prefill_chunk_busy: int = 2048
    prefix_reuse_min_rows: int = 256
    adopt_min: int = 64
    decoder_skip: bool = True
    speculation: bool = True
    spec_depth: int = 5
    two_shot_rows: int = 512       # many-row partials cross the links in two shots from this many rows ...
    two_shot_world: int = 8        # ... and this many ranks on
    stall_secs: float = 120.0
    max_context: int = 1048576
    cuda_graphs: bool = True
    seed: int = 0


# name -> (field path, parser).  Every override the engine honours is listed here; an unknown
# SFB_* variable or an unparsable value is refused at start-up.
def _b(s: str) -> bool:
    if s.lower() in ("1", "true", "on", "yes"):
        return True
    if s.lower() in ("0", "false", "off", "no"):
        return False
    raise ValueError(f"not a boolean: {s!r}")


def _choice(*opts: str):
    def p(s: str) -> str:
        if s not in opts:
            raise ValueError(f"{s!r} not in {opts}")
        return s
    return p


ENV_OVERRIDES: dict[str, tuple[str, Any]] = {
    "SFB_MAX_LANES": ("engine.max_lanes", int),
    "SFB_QUEUE_DEPTH": ("engine.queue_depth", int),
    "SFB_MAX_ROWS": ("engine.max_rows", int),
    "SFB_PREFILL_CHUNK": ("engine.prefill_chunk", int),
    "SFB_PREFILL_CHUNK_BUSY": ("engine.prefill_chunk_busy", int),
    "SFB_PREFIX_REUSE_MIN_ROWS": ("engine.prefix_reuse_min_rows", int),
    "SFB_DECODER_SKIP": ("engine.decoder_skip", _b),
    "SFB_SPECULATION": ("engine.speculation", _b),
    "SFB_SPEC_DEPTH": ("engine.spec_depth", int),
    "SFB_TWO_SHOT_ROWS": ("engine.two_shot_rows", int),
    "SFB_TWO_SHOT_WORLD": ("engine.two_shot_world", int),
    "SFB_STALL_SECS": ("engine.stall_secs", float),
    "SFB_MAX_CONTEXT": ("engine.max_context", int),
    "SFB_CUDA_GRAPHS": ("engine.cuda_graphs", _b),
    "SFB_SEED": ("engine.seed", int),
    "SFB_MOE_MODE": ("parallel.moe_mode", _choice("tp", "ep")),
    "SFB_COLLECTIVE": ("parallel.collective", _choice("fused", "nccl")),
}
# variables that are read elsewhere and are not settings of the engine
_ENV_PASSTHROUGH = {"SFB_REBUILD", "SFB_KERNEL_MARKS", "SFB_NVCC", "SFB_LOG", "SFB_TRACE_SCOPES", "SFB_API_KEY",
                    "SFB_MODEL_ALIASES", "SFB_DEBUG_BOUNDS", "SFB_FUSED_SPLITS", "SFB_ARM", "SFB_CONTROL_TOKEN"}
# names the host gates use (ci/host_gates.py checks that every SFB_* variable the sources read is in one of the two)
ENV_TABLE = ENV_OVERRIDES
ENV_INTERNAL = _ENV_PASSTHROUGH


@dataclass
class Settings:
    model: ModelConfig = field(default_factory=ModelConfig)
    engine: EngineConfig = field(default_factory=EngineConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)

    def apply_env(self, env: dict[str, str] | None = None) -> "Settings":
        env = dict(os.environ if env is None else env)
        for k, v in env.items():
            if not k.startswith("SFB_") or k in _ENV_PASSTHROUGH:
                continue
            if k not in ENV_OVERRIDES:
                raise ValueError(f"unknown setting {k}; known: {sorted(ENV_OVERRIDES)}")
            path, parse = ENV_OVERRIDES[k]
            sect, name = path.split(".")
            try:
                setattr(getattr(self, sect), name, parse(v))
            except ValueError as e:
                raise ValueError(f"{k}={v!r}: {e}") from None
        return self

    def apply_dict(self, d: dict[str, Any]) -> "Settings":
        for sect, body in d.items():
            if not hasattr(self, sect):
                raise ValueError(f"unknown section [{sect}]")
            obj = getattr(self, sect)
            for k, v in body.items():
                if not hasattr(obj, k):
                    raise ValueError(f"unknown key {sect}.{k}")
                setattr(obj, k, v)
        return self

    def digest(self) -> str:
        """Agreement word: every rank must start with the same effective settings."""
        d = {"model": dataclasses.asdict(self.model), "engine": dataclasses.asdict(self.engine),
             "moe_mode": self.parallel.moe_mode, "collective": self.parallel.collective,
             "world": self.parallel.world}
        return hashlib.sha256(json.dumps(d, sort_keys=True).encode()).hexdigest()[:16]


def load_toml(path: str) -> dict[str, Any]:
    import tomllib
    with open(path, "rb") as f:
        return tomllib.load(f)


# released checkpoint's config.json key -> ModelConfig field (reference: crates/sparkflash-model-deepseek-v41/
# src/config.rs:64-207; keys this engine has no use for are listed so that a NEW unknown key is refused)
_HF_KEYS = {
    "vocab_size": "vocab_size", "dim": "hidden_size", "n_layers": "n_layers", "n_heads": "n_heads", "head_dim": "head_dim",
    "rope_head_dim": "rope_dim", "q_lora_rank": "q_lora_rank", "o_groups": "o_groups", "o_lora_rank": "o_lora_rank",
    "moe_inter_dim": "moe_inter", "n_routed_experts": "n_routed_experts", "n_shared_experts": "n_shared_experts",
    "n_activated_experts": "top_k", "route_scale": "route_scale", "swiglu_limit": "swiglu_limit", "norm_eps": "norm_eps",
    "window_size": "window", "rope_theta": "rope_theta", "compress_rope_theta": "compress_rope_theta", "rope_factor": "yarn_factor",
    "original_seq_len": "yarn_orig_max_pos", "beta_fast": "yarn_beta_fast", "beta_slow": "yarn_beta_slow",
    "compress_ratios": "compress_ratios", "kv_source_layers": "kv_source_layers", "index_source_layers": "index_source_layers",
    "candidate_source_layer": "candidate_source_layer", "candidate_topk_blocks": "candidate_topk_blocks",
    "candidate_block_size": "candidate_block_size", "index_n_heads": "index_n_heads", "index_head_dim": "index_head_dim",
    "index_topk": "index_topk", "hc_mult": "hc_mult", "hc_sinkhorn_iters": "hc_sinkhorn_iters", "hc_eps": "hc_eps",
    "engram_layer_ids": "engram_layers", "engram_num_embeddings": "engram_rows", "engram_max_ngram_size": "engram_max_ngram",
    "engram_n_heads": "engram_n_heads", "engram_head_dim": "engram_head_dim", "engram_compressed_vocab_size": "engram_compressed_vocab",
    "n_mtp_layers": "n_mtp_stages", "dspark_block_size": "dspark_block", "dspark_noise_token_id": "dspark_noise_token",
    "dspark_target_layer_ids": "dspark_taps", "dspark_markov_rank": "dspark_markov_rank", "dspark_n_routed_experts": "dspark_n_experts",
    "dspark_n_activated_experts": "dspark_top_k", "image_token_id": "image_token_id",
}
_HF_IGNORED = {"score_func", "dtype", "expert_dtype", "gate_temp", "norm_topk_prob", "engram_vocab_size", "engram_pad_id",
               "model_type", "architectures", "torch_dtype", "transformers_version", "max_position_embeddings", "bos_token_id",
               "eos_token_id", "pad_token_id", "tie_word_embeddings", "quantization_config", "auto_map"}


def config_from_hf(d: dict[str, Any]) -> ModelConfig:
    """ModelConfig from a checkpoint's ``config.json``.  Unknown keys are refused (a typo or a new
    architecture knob must not be silently dropped); ``vision_*`` keys belong to the vision tower's own config."""
    kw: dict[str, Any] = {}
    for k, v in d.items():
        if k in _HF_KEYS:
            kw[_HF_KEYS[k]] = v
        elif k in _HF_IGNORED or k.startswith("vision_"):
            continue
        else:
            raise ValueError(f"config.json: unknown key {k!r}")
    if d.get("score_func", "sqrtsoftplus") != "sqrtsoftplus":
        raise ValueError(f"score_func {d['score_func']!r} is not implemented (sqrtsoftplus only)")
    if "eos_token_id" in d:
        kw["eos_id"] = d["eos_token_id"]
    if "bos_token_id" in d:
        kw["bos_id"] = d["bos_token_id"]
    if "max_position_embeddings" in d:
        kw["max_positions"] = d["max_position_embeddings"]
    return dataclasses.replace(ModelConfig(), **kw)


def config_to_hf(c: ModelConfig) -> dict[str, Any]:
    inv = {v: k for k, v in _HF_KEYS.items()}
    out = {inv[f.name]: getattr(c, f.name) for f in dataclasses.fields(c) if f.name in inv}
    out.update(score_func="sqrtsoftplus", eos_token_id=c.eos_id, bos_token_id=c.bos_id, max_position_embeddings=c.max_positions,
               model_type="deepseek_v41")
    return out
