"""Tensor inventory, synthetic checkpoints and dequantisation for DeepSeek-V4.1-Flash.

Names and shapes follow the released checkpoint (reference: docs/engine/01-forward-order.md
section 2; synthetic weights: crates/sparkflash-model-deepseek-v41/src/synthetic.rs:15-146 - bytes
derived from the tensor *name* and a seed, so any subset of tensors can be generated independently
and no checkpoint is needed for tests or benchmarks).

Storage kinds:
  ``fp8``  E4M3 codes [out, in] + UE8M0 scales [ceil(out/32), in/32]   (32x32 blocks)
  ``fp4``  packed E2M1 [out, in/2] + UE8M0 scales [out, in/32]
  ``bf16`` / ``f32`` plain
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import codecs
from ...config import ModelConfig


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    kind: str          # fp8 | fp4 | bf16 | f32
    init: str = "normal"  # normal | ones | zeros | small


def _fnv1a(s: str) -> int:
    h = 0xCBF29CE484222325
    for b in s.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _block_specs(cfg: ModelConfig, p: str, n_experts: int, with_sparse: bool, layer: int) -> list[TensorSpec]:
    d, h, hd, q = cfg.hidden_size, cfg.n_heads, cfg.head_dim, cfg.q_lora_rank
    og, ol, mi, hc = cfg.o_groups, cfg.o_lora_rank, cfg.moe_inter, cfg.hc_mult
    mix = (2 + hc) * hc
    S = TensorSpec
    out = [
        S(f"{p}.attn.attn_sink", (h,), "f32", "small"),
        S(f"{p}.attn.wq_a", (q, d), "fp8"),
        S(f"{p}.attn.q_norm.weight", (q,), "bf16", "ones"),
        S(f"{p}.attn.wq_b", (h * hd, q), "fp8"),
        S(f"{p}.attn.wkv", (hd, d), "fp8"),
        S(f"{p}.attn.kv_norm.weight", (hd,), "bf16", "ones"),
        S(f"{p}.attn.wo_a", (og * ol, h * hd // og), "fp8"),
        S(f"{p}.attn.wo_b", (d, og * ol), "fp8"),
        S(f"{p}.attn_norm.weight", (d,), "bf16", "ones"),
        S(f"{p}.ffn_norm.weight", (d,), "bf16", "ones"),
        S(f"{p}.hc_attn_fn", (mix, hc * d), "f32"),
        S(f"{p}.hc_ffn_fn", (mix, hc * d), "f32"),
        S(f"{p}.hc_attn_base", (mix,), "f32", "small"),
        S(f"{p}.hc_ffn_base", (mix,), "f32", "small"),
        S(f"{p}.hc_attn_scale", (3,), "f32", "ones"),
        S(f"{p}.hc_ffn_scale", (3,), "f32", "ones"),
        S(f"{p}.ffn.gate.weight", (n_experts, d), "bf16"),
        S(f"{p}.ffn.gate.bias", (n_experts,), "f32", "small"),
        S(f"{p}.ffn.gate.bias_vl", (n_experts,), "f32", "small"),
        S(f"{p}.ffn.shared_experts.w1", (mi, d), "fp8"),
        S(f"{p}.ffn.shared_experts.w3", (mi, d), "fp8"),
        S(f"{p}.ffn.shared_experts.w2", (d, mi), "fp8"),
    ]
    for e in range(n_experts):
        out += [S(f"{p}.ffn.experts.{e}.w1", (mi, d), "fp4"), S(f"{p}.ffn.experts.{e}.w3", (mi, d), "fp4"),
                S(f"{p}.ffn.experts.{e}.w2", (d, mi), "fp4")]
    if with_sparse:
        idh, inh = cfg.index_head_dim, cfg.index_n_heads
        if cfg.is_kv_source(layer):
            out += [S(f"{p}.attn.compressor.wkv.weight", (hd, d), "bf16"),
                    S(f"{p}.attn.compressor.norm.weight", (hd,), "bf16", "ones"),
                    S(f"{p}.attn.indexer.wk.weight", (idh, hd), "bf16"),
                    S(f"{p}.attn.indexer.k_norm.weight", (idh,), "bf16", "ones")]
            if cfg.ratio(layer) > 1:
                out.append(S(f"{p}.attn.compressor.wgate.weight", (hd, d), "bf16"))
        if cfg.is_index_source(layer):
            out += [S(f"{p}.attn.indexer.wq_b", (inh * idh, q), "fp8"),
                    S(f"{p}.attn.indexer.weights_proj.weight", (inh, d), "bf16")]
    return out


def tensor_specs(cfg: ModelConfig) -> list[TensorSpec]:
    d, V = cfg.hidden_size, cfg.vocab_size
    S = TensorSpec
    out = [S("embed.weight", (V, d), "bf16"), S("head.weight", (V, d), "bf16"),
           S("norm.weight", (d,), "bf16", "ones")]
    for l in range(cfg.n_layers):
        out += _block_specs(cfg, f"layers.{l}", cfg.n_routed_experts, True, l)
    for s in range(cfg.n_mtp_stages):
        out += _block_specs(cfg, f"mtp.{s}", cfg.dspark_n_experts, False, cfg.n_layers + s)
    if cfg.engram_enabled:
        from ...engram.layout import EngramLayout
        lay = EngramLayout.build(cfg.engram_layers, cfg.engram_max_ngram, cfg.engram_n_heads, cfg.engram_vocab, cfg.engram_compressed_vocab)
        cols = (cfg.engram_max_ngram - 1) * cfg.engram_n_heads
        for j, l in enumerate(cfg.engram_layers):
            out += [S(f"engram.{l}.embed", (lay.rows[j], cfg.engram_head_dim), "fp8row", "unit"),
                    S(f"engram.{l}.wkv", ((cfg.hc_mult + 1) * d, cols * cfg.engram_head_dim), "fp8"),
                    S(f"engram.{l}.gate_w", (cfg.hc_mult, d), "f32", "ones")]      # q_weight * k_weight, folded
    if cfg.n_mtp_stages:
        r = cfg.dspark_markov_rank
        last = cfg.n_mtp_stages - 1
        out += [S("mtp.0.main_proj", (d, d * len(cfg.dspark_taps)), "fp8"),
                S("mtp.0.main_norm.weight", (d,), "bf16", "ones"),
                S(f"mtp.{last}.norm.weight", (d,), "bf16", "ones"),
                S(f"mtp.{last}.markov_head.embed.weight", (V, r), "bf16"),
                S(f"mtp.{last}.markov_head.head.weight", (V, r), "bf16"),
                S(f"mtp.{last}.confidence_head.proj.weight", (1, d + r), "bf16")]
    return out


def _master(spec: TensorSpec, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed((_fnv1a(spec.name) ^ seed) & 0x7FFFFFFFFFFFFFFF)
    if spec.init == "ones":
        return 1.0 + 0.05 * torch.randn(spec.shape, generator=g)
    if spec.init == "zeros":
        return torch.zeros(spec.shape)
    if spec.init == "small":
        return 0.1 * torch.randn(spec.shape, generator=g)
    if spec.init == "unit":
        return torch.randn(spec.shape, generator=g)
    std = 0.02
    if spec.name.endswith(("hc_attn_fn", "hc_ffn_fn")):
        std = 0.05
    return std * torch.randn(spec.shape, generator=g)


def synthetic_checkpoint(cfg: ModelConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """HF-style dict: quantised tensors appear as ``<name>.weight`` (uint8 codes) + ``<name>.scale``."""
    ck: dict[str, torch.Tensor] = {}
    for sp in tensor_specs(cfg):
        w = _master(sp, seed)
        if sp.kind == "fp8":
            q, s = codecs.weight_quant_fp8_block32(w)
            ck[sp.name + ".weight"], ck[sp.name + ".scale"] = q, s
        elif sp.kind == "fp4":
            q, s = codecs.weight_quant_fp4_row32(w)
            ck[sp.name + ".weight"], ck[sp.name + ".scale"] = q, s
        elif sp.kind == "fp8row":          # table rows: E4M3 codes with one UE8M0 scale per 32 values of the row
            q, s = codecs.act_quant_fp8(w)
            ck[sp.name + ".weight"], ck[sp.name + ".scale"] = q, s
        elif sp.kind == "bf16":
            ck[sp.name] = w.to(torch.bfloat16)
        else:
            ck[sp.name] = w.to(torch.float32)
    return ck


def dequantize_checkpoint(ck: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    """Every tensor as fp32 values (what the oracle multiplies with); quantised ones lose '.weight'."""
    out: dict[str, torch.Tensor] = {}
    for sp in tensor_specs(cfg):
        if sp.kind == "fp8":
            out[sp.name] = codecs.weight_dequant_fp8_block32(ck[sp.name + ".weight"], ck[sp.name + ".scale"])
        elif sp.kind == "fp4":
            out[sp.name] = codecs.weight_dequant_fp4_row32(ck[sp.name + ".weight"], ck[sp.name + ".scale"])
        elif sp.kind == "fp8row":
            q, sc = ck[sp.name + ".weight"], ck[sp.name + ".scale"]
            out[sp.name] = (codecs.e4m3_decode(q).reshape(q.shape[0], -1, 32) * codecs.ue8m0_decode(sc).unsqueeze(-1)).reshape(q.shape)
        else:
            out[sp.name] = ck[sp.name].to(torch.float32)
    return out


def checkpoint_bytes(cfg: ModelConfig) -> int:
    n = 0
    for sp in tensor_specs(cfg):
        e = 1
        for s in sp.shape:
            e *= s
        if sp.kind == "fp8":
            n += e + e // 1024
        elif sp.kind == "fp4":
            n += e // 2 + e // 32
        elif sp.kind == "bf16":
            n += 2 * e
        else:
            n += 4 * e
    return n
