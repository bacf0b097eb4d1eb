"""Classic multi-head latent attention (DeepSeek-V3 style) MoE decoder on the CPU: a full-recompute fp32 oracle and
an incremental engine that caches only the compressed latent and the shared rotary key and uses absorbed
projections for decode.  This is the reference's "tiny MLA v3" CPU configuration (2 layers, hidden 256, 4 heads,
q_lora 128, kv_lora 64, rope 32, nope 32, v 32, 8 routed experts top-2 + 1 shared, FFN 128, vocab 1024; fp32 weights
~N(0, 0.02) from seed 0; prompt of 32 ids from seed 1; greedy decode of 16 tokens).
Reference: crates/sparkflash-engine/tests/forward.rs (host oracle forward), BASELINE configuration 1.

    python -m sparkflash_b200.models.mla_v3        # prints one JSON line: tok/s of the cached engine and its max
                                                   # logit distance to the oracle
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MlaConfig:
    vocab: int = 1024
    dim: int = 256
    n_layers: int = 2
    n_heads: int = 4
    q_lora: int = 128
    kv_lora: int = 64
    rope: int = 32
    nope: int = 32
    v: int = 32
    n_experts: int = 8
    top_k: int = 2
    n_shared: int = 1
    inter: int = 128
    theta: float = 10000.0
    eps: float = 1e-6


def init_weights(c: MlaConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g) * 0.02
    w = {"embed": n(c.vocab, c.dim), "head": n(c.vocab, c.dim), "norm": torch.ones(c.dim)}
    for l in range(c.n_layers):
        p = f"l{l}."
        w[p + "attn_norm"], w[p + "ffn_norm"] = torch.ones(c.dim), torch.ones(c.dim)
        w[p + "wq_a"], w[p + "q_norm"] = n(c.q_lora, c.dim), torch.ones(c.q_lora)
        w[p + "wq_b"] = n(c.n_heads * (c.nope + c.rope), c.q_lora)
        w[p + "wkv_a"], w[p + "kv_norm"] = n(c.kv_lora + c.rope, c.dim), torch.ones(c.kv_lora)
        w[p + "wkv_b"] = n(c.n_heads * (c.nope + c.v), c.kv_lora)
        w[p + "wo"] = n(c.dim, c.n_heads * c.v)
        w[p + "gate"] = n(c.n_experts, c.dim)
        w[p + "w1"], w[p + "w3"], w[p + "w2"] = n(c.n_experts, c.inter, c.dim), n(c.n_experts, c.inter, c.dim), n(c.n_experts, c.dim, c.inter)
        w[p + "s1"], w[p + "s3"], w[p + "s2"] = n(c.n_shared * c.inter, c.dim), n(c.n_shared * c.inter, c.dim), n(c.dim, c.n_shared * c.inter)
    return w


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, pos, theta):
    """x [..., T, rd] interleaved pairs; pos [T]."""
    rd = x.shape[-1]
    inv = theta ** (-torch.arange(0, rd, 2, dtype=torch.float32) / rd)
    ang = pos.float().unsqueeze(-1) * inv
    cos, sin = ang.cos(), ang.sin()
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)


def moe(c: MlaConfig, w, p, x):
    """x [T, dim]: softmax router, top-k renormalised, plus the shared expert."""
    scores = F.softmax(x @ w[p + "gate"].t(), -1)
    top, idx = scores.topk(c.top_k, -1)
    top = top / top.sum(-1, keepdim=True)
    out = (F.silu(x @ w[p + "s1"].t()) * (x @ w[p + "s3"].t())) @ w[p + "s2"].t()
    for t in range(x.shape[0]):
        for k in range(c.top_k):
            e = int(idx[t, k])
            h = F.silu(w[p + "w1"][e] @ x[t]) * (w[p + "w3"][e] @ x[t])
            out[t] = out[t] + top[t, k] * (w[p + "w2"][e] @ h)
    return out


def oracle_logits(c: MlaConfig, w, tokens: list[int]) -> torch.Tensor:
    """Full recompute, un-absorbed attention: logits [T, vocab] for every position."""
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    mask = torch.full((T, T), float("-inf")).triu(1)
    scale = 1.0 / math.sqrt(c.nope + c.rope)
    for l in range(c.n_layers):
        p = f"l{l}."
        h = rms(x, w[p + "attn_norm"], c.eps)
        q = (rms(h @ w[p + "wq_a"].t(), w[p + "q_norm"], c.eps) @ w[p + "wq_b"].t()).view(T, c.n_heads, c.nope + c.rope)
        q_n, q_r = q[..., :c.nope], rope(q[..., c.nope:].transpose(0, 1), pos, c.theta).transpose(0, 1)
        kva = h @ w[p + "wkv_a"].t()
        lat, k_r = rms(kva[:, :c.kv_lora], w[p + "kv_norm"], c.eps), rope(kva[:, c.kv_lora:], pos, c.theta)
        kv = (lat @ w[p + "wkv_b"].t()).view(T, c.n_heads, c.nope + c.v)
        k_n, v = kv[..., :c.nope], kv[..., c.nope:]
        s = (torch.einsum("thd,shd->hts", q_n, k_n) + torch.einsum("thd,sd->hts", q_r, k_r)) * scale + mask
        o = torch.einsum("hts,shd->thd", F.softmax(s, -1), v).reshape(T, -1)
        x = x + o @ w[p + "wo"].t()
        x = x + moe(c, w, p, rms(x, w[p + "ffn_norm"], c.eps))
    return rms(x, w["norm"], c.eps) @ w["head"].t()


class CachedEngine:
    """Incremental decode: per layer the cache holds [T, kv_lora] latents and [T, rope] rotary keys; queries are
    absorbed into the latent space (q_n W_k) and values are expanded after the weighted sum (W_v)."""

    def __init__(self, c: MlaConfig, w):
        self.c, self.w = c, w
        self.lat = [torch.zeros(0, c.kv_lora) for _ in range(c.n_layers)]
        self.kr = [torch.zeros(0, c.rope) for _ in range(c.n_layers)]
        self.wk, self.wv = [], []
        for l in range(c.n_layers):
            b = w[f"l{l}.wkv_b"].view(c.n_heads, c.nope + c.v, c.kv_lora)
            self.wk.append(b[:, :c.nope]); self.wv.append(b[:, c.nope:])
        self.pos = 0

    def step(self, tokens: list[int]) -> torch.Tensor:
        """Append ``tokens`` (a prefill chunk or one decode token); logits of the last position."""
        c, w = self.c, self.w
        T = len(tokens)
        pos = torch.arange(self.pos, self.pos + T)
        x = w["embed"][torch.tensor(tokens)]
        scale = 1.0 / math.sqrt(c.nope + c.rope)
        for l in range(c.n_layers):
            p = f"l{l}."
            h = rms(x, w[p + "attn_norm"], c.eps)
            q = (rms(h @ w[p + "wq_a"].t(), w[p + "q_norm"], c.eps) @ w[p + "wq_b"].t()).view(T, c.n_heads, c.nope + c.rope)
            q_r = rope(q[..., c.nope:].transpose(0, 1), pos, c.theta).transpose(0, 1)
            q_lat = torch.einsum("thd,hdk->thk", q[..., :c.nope], self.wk[l])          # absorbed
            kva = h @ w[p + "wkv_a"].t()
            self.lat[l] = torch.cat([self.lat[l], rms(kva[:, :c.kv_lora], w[p + "kv_norm"], c.eps)])
            self.kr[l] = torch.cat([self.kr[l], rope(kva[:, c.kv_lora:], pos, c.theta)])
            S = self.lat[l].shape[0]
            s = (torch.einsum("thk,sk->hts", q_lat, self.lat[l]) + torch.einsum("thd,sd->hts", q_r, self.kr[l])) * scale
            causal = torch.arange(S).unsqueeze(0) > pos.unsqueeze(1)
            s = s.masked_fill(causal.unsqueeze(0), float("-inf"))
            o_lat = torch.einsum("hts,sk->thk", F.softmax(s, -1), self.lat[l])
            o = torch.einsum("thk,hdk->thd", o_lat, self.wv[l]).reshape(T, -1)
            x = x + o @ w[p + "wo"].t()
            x = x + moe(c, w, p, rms(x, w[p + "ffn_norm"], c.eps))
        self.pos += T
        return rms(x[-1], w["norm"], c.eps) @ w["head"].t()


def run(n_new: int = 16, prompt_len: int = 32) -> dict:
    c = MlaConfig()
    w = init_weights(c, 0)
    prompt = torch.randint(0, c.vocab, (prompt_len,), generator=torch.Generator().manual_seed(1)).tolist()
    eng = CachedEngine(c, w)
    t0 = time.perf_counter()
    logits = eng.step(prompt)
    t_prefill = time.perf_counter() - t0
    toks, got = [], []
    t0 = time.perf_counter()
    for _ in range(n_new):
        got.append(logits)
        toks.append(int(logits.argmax()))
        logits = eng.step([toks[-1]])
    t_decode = time.perf_counter() - t0
    want = oracle_logits(c, w, prompt + toks)[prompt_len - 1:prompt_len - 1 + n_new]
    err = (torch.stack(got) - want).abs().max().item()
    agree = int((torch.stack(got).argmax(-1) == want.argmax(-1)).sum())
    return {"metric": "cpu_oracle_decode_tok_s", "value": n_new / t_decode, "unit": "tok/s", "prefill_tok_s": prompt_len / t_prefill,
            "max_abs_logit_err_vs_fp32_oracle": err, "argmax_agree": f"{agree}/{n_new}", "tokens": toks,
            "config": "tiny-mla-v3: 2 layers, hidden 256, 4 heads, 8 experts top-2 + shared, vocab 1024, fp32, 1 thread pool default"}


if __name__ == "__main__":
    print(json.dumps(run()))
