"""GLM-5.3-Flash-style decoder: multi-head latent attention whose keys are chosen per query by a small indexer (a few
light heads score every cached position, the best ``index_topk`` are attended), a sigmoid router with a selection-only
bias (noaux) and a shared expert.  With ``index_topk`` at or above the context the indexer selects everything and the
model is the classic MLA of ``mla_v3``; below it, attention is sparse.

* ``reference_logits`` - full recompute on the CPU (fp32), un-absorbed attention, the oracle;
* ``CachedEngine`` - incremental decode with the latent cache, absorbed queries and an index-key cache, the same
  selection rule (ties to the lower position), so both give the same logits.

Reference behaviour: crates/sparkflash-model-glm5-next (device forward, tests device_forward.rs / serve_tiny.rs);
the indexer and the noaux router follow the flagship's (crates/sparkflash-deepseek-forward).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .mla_v3 import rms, rope


@dataclass(frozen=True)
class GlmConfig:
    vocab: int = 512
    dim: int = 128
    n_layers: int = 2
    n_heads: int = 4
    q_lora: int = 64
    kv_lora: int = 32
    rope: int = 16
    nope: int = 16
    v: int = 16
    index_heads: int = 2
    index_dim: int = 16
    index_topk: int = 8
    n_experts: int = 8
    top_k: int = 2
    inter: int = 64
    route_scale: float = 1.5
    theta: float = 10000.0
    eps: float = 1e-6


def init_weights(c: GlmConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g) * s[-1] ** -0.5
    w = {"embed": torch.randn(c.vocab, c.dim, generator=g), "head": n(c.vocab, c.dim), "norm": torch.ones(c.dim)}
    for l in range(c.n_layers):
        p = f"l{l}."
        w[p + "attn_norm"], w[p + "ffn_norm"] = torch.ones(c.dim), torch.ones(c.dim)
        w[p + "wq_a"], w[p + "q_norm"] = n(c.q_lora, c.dim), torch.ones(c.q_lora)
        w[p + "wq_b"] = n(c.n_heads * (c.nope + c.rope), c.q_lora)
        w[p + "wkv_a"], w[p + "kv_norm"] = n(c.kv_lora + c.rope, c.dim), torch.ones(c.kv_lora)
        w[p + "wkv_b"] = n(c.n_heads * (c.nope + c.v), c.kv_lora)
        w[p + "wo"] = n(c.dim, c.n_heads * c.v)
        w[p + "idx_q"] = n(c.index_heads * c.index_dim, c.q_lora)      # from the normalised q latent
        w[p + "idx_k"] = n(c.index_dim, c.dim)
        w[p + "idx_w"] = n(c.index_heads, c.dim)                        # per-head weights of the score
        w[p + "gate"] = n(c.n_experts, c.dim)
        w[p + "gate_bias"] = torch.randn(c.n_experts, generator=g) * 0.1
        w[p + "w1"], w[p + "w3"], w[p + "w2"] = n(c.n_experts, c.inter, c.dim), n(c.n_experts, c.inter, c.dim), n(c.n_experts, c.dim, c.inter)
        w[p + "s1"], w[p + "s3"], w[p + "s2"] = n(c.inter, c.dim), n(c.inter, c.dim), n(c.dim, c.inter)
    return w


def noaux_moe(c: GlmConfig, w, p, x):
    """Sigmoid scores; the bias only decides who is selected, the weights are the unbiased scores renormalised."""
    s = torch.sigmoid(x @ w[p + "gate"].t())
    _, idx = (s + w[p + "gate_bias"]).topk(c.top_k, -1)
    top = s.gather(-1, idx)
    top = top / (top.sum(-1, keepdim=True) + 1e-20) * c.route_scale
    out = (F.silu(x @ w[p + "s1"].t()) * (x @ w[p + "s3"].t())) @ w[p + "s2"].t()
    for t in range(x.shape[0]):
        for k in range(c.top_k):
            e = int(idx[t, k])
            h = F.silu(w[p + "w1"][e] @ x[t]) * (w[p + "w3"][e] @ x[t])
            out[t] = out[t] + top[t, k] * (w[p + "w2"][e] @ h)
    return out


def index_select(scores: torch.Tensor, n_valid: int, topk: int) -> torch.Tensor:
    """Positions (sorted) of the ``topk`` best of scores[:n_valid]; everything when n_valid <= topk; ties to the lower position."""
    if n_valid <= topk:
        return torch.arange(n_valid)
    order = sorted(range(n_valid), key=lambda j: (-float(scores[j]), j))[:topk]
    return torch.tensor(sorted(order))


def _index_scores(c: GlmConfig, w, p, h_t, q_lat_t, idx_k):
    """Score of every cached position for one query row: sum over heads of weight * relu(q_h . k)."""
    qi = (w[p + "idx_q"] @ q_lat_t).view(c.index_heads, c.index_dim)
    hw = w[p + "idx_w"] @ h_t
    return (F.relu(qi @ idx_k.t()) * hw.unsqueeze(-1)).sum(0) * c.index_dim ** -0.5


def reference_logits(c: GlmConfig, w, tokens: list[int]) -> torch.Tensor:
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    scale = 1.0 / math.sqrt(c.nope + c.rope)
    for l in range(c.n_layers):
        p = f"l{l}."
        h = rms(x, w[p + "attn_norm"], c.eps)
        ql = rms(h @ w[p + "wq_a"].t(), w[p + "q_norm"], c.eps)
        q = (ql @ w[p + "wq_b"].t()).view(T, c.n_heads, c.nope + c.rope)
        q_n, q_r = q[..., :c.nope], rope(q[..., c.nope:].transpose(0, 1), pos, c.theta).transpose(0, 1)
        kva = h @ w[p + "wkv_a"].t()
        lat, k_r = rms(kva[:, :c.kv_lora], w[p + "kv_norm"], c.eps), rope(kva[:, c.kv_lora:], pos, c.theta)
        kv = (lat @ w[p + "wkv_b"].t()).view(T, c.n_heads, c.nope + c.v)
        k_n, v = kv[..., :c.nope], kv[..., c.nope:]
        idx_k = h @ w[p + "idx_k"].t()
        o = torch.empty(T, c.n_heads * c.v)
        for t in range(T):
            sel = index_select(_index_scores(c, w, p, h[t], ql[t], idx_k[:t + 1]), t + 1, c.index_topk)
            s = (torch.einsum("hd,shd->hs", q_n[t], k_n[sel]) + torch.einsum("hd,sd->hs", q_r[t], k_r[sel])) * scale
            o[t] = torch.einsum("hs,shd->hd", F.softmax(s, -1), v[sel]).reshape(-1)
        x = x + o @ w[p + "wo"].t()
        x = x + noaux_moe(c, w, p, rms(x, w[p + "ffn_norm"], c.eps))
    return rms(x, w["norm"], c.eps) @ w["head"].t()


class CachedEngine:
    """Incremental decode: latent + rotary-key + index-key caches, absorbed queries, sparse attention over the selection."""

    def __init__(self, c: GlmConfig, w):
        self.c, self.w = c, w
        self.lat = [torch.zeros(0, c.kv_lora) for _ in range(c.n_layers)]
        self.kr = [torch.zeros(0, c.rope) for _ in range(c.n_layers)]
        self.ik = [torch.zeros(0, c.index_dim) for _ in range(c.n_layers)]
        self.wk, self.wv = [], []
        for l in range(c.n_layers):
            b = w[f"l{l}.wkv_b"].view(c.n_heads, c.nope + c.v, c.kv_lora)
            self.wk.append(b[:, :c.nope]); self.wv.append(b[:, c.nope:])
        self.pos = 0
        self.selected: list[torch.Tensor] = []      # last step's selections per layer (for tests and tracing)

    def step(self, tokens: list[int]) -> torch.Tensor:
        """Append ``tokens``; logits [len(tokens), vocab]."""
        c, w = self.c, self.w
        T = len(tokens)
        pos = torch.arange(self.pos, self.pos + T)
        x = w["embed"][torch.tensor(tokens)]
        scale = 1.0 / math.sqrt(c.nope + c.rope)
        self.selected = []
        for l in range(c.n_layers):
            p = f"l{l}."
            h = rms(x, w[p + "attn_norm"], c.eps)
            ql = rms(h @ w[p + "wq_a"].t(), w[p + "q_norm"], c.eps)
            q = (ql @ w[p + "wq_b"].t()).view(T, c.n_heads, c.nope + c.rope)
            q_r = rope(q[..., c.nope:].transpose(0, 1), pos, c.theta).transpose(0, 1)
            q_lat = torch.einsum("thd,hdk->thk", q[..., :c.nope], self.wk[l])
            kva = h @ w[p + "wkv_a"].t()
            self.lat[l] = torch.cat([self.lat[l], rms(kva[:, :c.kv_lora], w[p + "kv_norm"], c.eps)])
            self.kr[l] = torch.cat([self.kr[l], rope(kva[:, c.kv_lora:], pos, c.theta)])
            self.ik[l] = torch.cat([self.ik[l], h @ w[p + "idx_k"].t()])
            o = torch.empty(T, c.n_heads * c.v)
            for t in range(T):
                n_valid = int(pos[t]) + 1
                sel = index_select(_index_scores(c, w, p, h[t], ql[t], self.ik[l][:n_valid]), n_valid, c.index_topk)
                s = (torch.einsum("hk,sk->hs", q_lat[t], self.lat[l][sel]) + torch.einsum("hd,sd->hs", q_r[t], self.kr[l][sel])) * scale
                o_lat = torch.einsum("hs,sk->hk", F.softmax(s, -1), self.lat[l][sel])
                o[t] = torch.einsum("hk,hdk->hd", o_lat, self.wv[l]).reshape(-1)
                if t == T - 1:
                    self.selected.append(sel)
            x = x + o @ w[p + "wo"].t()
            x = x + noaux_moe(c, w, p, rms(x, w[p + "ffn_norm"], c.eps))
        self.pos += T
        return rms(x, w["norm"], c.eps) @ w["head"].t()
