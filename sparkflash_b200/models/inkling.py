"""Inkling-2-Small-style decoder: a short causal depthwise convolution in front of a sliding-window attention whose
logits are soft-capped, a MoE whose experts use a soft-capped SwiGLU, soft-capped output logits - and the three ways its
experts can be laid over ranks:

* ``experts``       whole experts per rank (expert parallelism): a rank adds the selected experts it owns;
* ``intermediate``  every rank holds a slice of every expert's intermediate width: partial sums over the slices;
* ``rows``          every rank produces a slice of the output rows of every selected expert: the slices are concatenated.

``moe_split`` computes each rank's part exactly as that rank would and combines them the way the collective does (sum in
rank order, or concatenation), so the three modes can be checked against the unsplit layer.  ``reference_logits`` is the
fp32 CPU oracle; ``DeviceEngine`` steps rows on the GPU with the convolution-history, soft-cap and soft-capped-SwiGLU
kernels (csrc/k_families.cu) and per-lane window caches.

Reference behaviour: crates/sparkflash-model-inkling2 (tensor.rs:49-78 ExpertSplit::{Experts, Intermediate, Rows};
collective.rs all_reduce / all_gather / exchange / scatter; conv_history_copy / restore), kernels/inkling_sm121.cu.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import linear_attn as LA

SPLITS = ("experts", "intermediate", "rows")


@dataclass
class InklingConfig:
    vocab: int = 512
    d: int = 128
    layers: int = 2
    heads: int = 4
    head_dim: int = 32
    window: int = 8
    conv_width: int = 4
    attn_cap: float = 50.0
    act_cap: float = 10.0
    logit_cap: float = 30.0
    experts: int = 8
    top_k: int = 2
    inter: int = 64
    eps: float = 1e-6


def init_weights(c: InklingConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)

    def r(*shape, s=None):
        s = s if s is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).float()
    w = {"embed": r(c.vocab, c.d, s=1.0), "head": r(c.vocab, c.d), "norm": torch.ones(c.d)}
    for l in range(c.layers):
        p = f"l{l}."
        H, hd = c.heads, c.head_dim
        w[p + "n1"], w[p + "n2"] = torch.ones(c.d), torch.ones(c.d)
        w[p + "conv"] = r(c.d, c.conv_width, s=0.5)
        w[p + "wq"], w[p + "wk"], w[p + "wv"], w[p + "wo"] = r(H * hd, c.d), r(H * hd, c.d), r(H * hd, c.d), r(c.d, H * hd)
        w[p + "router"] = r(c.experts, c.d)
        w[p + "w1"], w[p + "w3"], w[p + "w2"] = r(c.experts, c.inter, c.d), r(c.experts, c.inter, c.d), r(c.experts, c.d, c.inter)
    return w


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _route(c: InklingConfig, w, p, x):
    probs = torch.softmax(x @ w[p + "router"].t(), -1)
    val, idx = torch.topk(probs, c.top_k, -1)
    return val / val.sum(-1, keepdim=True), idx


def _act(c: InklingConfig, g, u):
    g = LA.softcap_reference(g, c.act_cap)
    return g * torch.sigmoid(g) * u


def moe(c: InklingConfig, w, p, x):
    val, idx = _route(c, w, p, x)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(c.top_k):
            e = int(idx[t, j])
            y[t] += val[t, j] * (w[p + "w2"][e] @ _act(c, w[p + "w1"][e] @ x[t], w[p + "w3"][e] @ x[t]))
    return y


def moe_split(c: InklingConfig, w, p, x, world: int, mode: str):
    """The MoE as ``world`` ranks would compute it under ``mode``; returns (combined output, list of per-rank parts)."""
    if mode not in SPLITS:
        raise ValueError(f"unknown expert split {mode!r}")
    val, idx = _route(c, w, p, x)                       # the router is replicated
    parts = []
    for r in range(world):
        if mode == "rows":
            lo, hi = r * c.d // world, (r + 1) * c.d // world
            part = torch.zeros(x.shape[0], hi - lo)
        else:
            part = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(c.top_k):
                e = int(idx[t, j])
                if mode == "experts":
                    per = c.experts // world
                    if not r * per <= e < (r + 1) * per:
                        continue
                    part[t] += val[t, j] * (w[p + "w2"][e] @ _act(c, w[p + "w1"][e] @ x[t], w[p + "w3"][e] @ x[t]))
                elif mode == "intermediate":
                    a, b = r * c.inter // world, (r + 1) * c.inter // world
                    h = _act(c, w[p + "w1"][e, a:b] @ x[t], w[p + "w3"][e, a:b] @ x[t])
                    part[t] += val[t, j] * (w[p + "w2"][e][:, a:b] @ h)
                else:
                    h = _act(c, w[p + "w1"][e] @ x[t], w[p + "w3"][e] @ x[t])
                    part[t] += val[t, j] * (w[p + "w2"][e][lo:hi] @ h)
        parts.append(part)
    if mode == "rows":
        return torch.cat(parts, -1), parts              # all-gather of row slices
    total = parts[0].clone()
    for part in parts[1:]:                               # all-reduce: rank order
        total += part
    return total, parts


def reference_logits(c: InklingConfig, w, tokens: list[int], world: int = 1, split: str = "experts") -> torch.Tensor:
    T = len(tokens)
    h = w["embed"][torch.tensor(tokens)]
    far = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    banned = (far < 0) | (far >= c.window)
    for l in range(c.layers):
        p = f"l{l}."
        H, hd = c.heads, c.head_dim
        x = _rms(h, w[p + "n1"], c.eps).to(torch.bfloat16)
        u = LA.short_conv_reference(x, w[p + "conv"], torch.zeros(c.d, c.conv_width - 1)).float()
        q, k, v = ((u @ w[p + n].t()).reshape(T, H, hd) for n in ("wq", "wk", "wv"))
        s = LA.softcap_reference(torch.einsum("thd,shd->hts", q, k) * hd ** -0.5, c.attn_cap)
        s = s.masked_fill(banned, float("-inf"))
        h = h + torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(T, H * hd) @ w[p + "wo"].t()
        x2 = _rms(h, w[p + "n2"], c.eps)
        h = h + (moe(c, w, p, x2) if world == 1 else moe_split(c, w, p, x2, world, split)[0])
    return LA.softcap_reference(_rms(h, w["norm"], c.eps) @ w["head"].t(), c.logit_cap)


class DeviceEngine:
    """Rows step on the GPU: per-lane convolution history and a window ring of keys and values per layer."""

    def __init__(self, c: InklingConfig, w, lanes: int = 2, device="cuda"):
        self.c, self.dev = c, device
        self.w = {k: v.to(device) for k, v in w.items()}
        self.conv = [LA.ConvState(lanes, c.d, c.conv_width, device=device) for _ in range(c.layers)]
        self.ring = c.window
        shape = (lanes, self.ring, c.heads, c.head_dim)
        self.kc = [torch.zeros(shape, device=device) for _ in range(c.layers)]
        self.vc = [torch.zeros(shape, device=device) for _ in range(c.layers)]

    def snapshot(self, lane: int) -> None:
        for s in self.conv:
            s.snapshot(lane)

    def restore(self, lane: int) -> None:
        for s in self.conv:
            s.restore(lane)

    def step(self, tokens: list[int], lanes: list[int], positions: list[int]) -> torch.Tensor:
        """One row per call per lane position, in order (the window ring keeps exactly ``window`` positions)."""
        c, w, dev = self.c, self.w, self.dev
        n = len(tokens)
        H, hd = c.heads, c.head_dim
        h = w["embed"][torch.tensor(tokens, device=dev)]
        for l in range(c.layers):
            p = f"l{l}."
            x = _rms(h, w[p + "n1"], c.eps).to(torch.bfloat16)
            u = self.conv[l].step(x, w[p + "conv"], lanes).float()
            q, k, v = ((u @ w[p + nm].t()).reshape(n, H, hd) for nm in ("wq", "wk", "wv"))
            o = torch.empty((n, H, hd), device=dev)
            for i in range(n):
                L, P = lanes[i], positions[i]
                self.kc[l][L, P % self.ring], self.vc[l][L, P % self.ring] = k[i], v[i]
                slots = [j % self.ring for j in range(max(0, P - c.window + 1), P + 1)]
                s = torch.einsum("hd,shd->hs", q[i], self.kc[l][L, slots]) * hd ** -0.5
                s = LA.softcap_(s.contiguous(), c.attn_cap)
                o[i] = torch.einsum("hs,shd->hd", torch.softmax(s, -1), self.vc[l][L, slots])
            h = h + o.reshape(n, H * hd) @ w[p + "wo"].t()
            x2 = _rms(h, w[p + "n2"], c.eps)
            val, idx = _route(c, w, p, x2)
            y = torch.zeros_like(x2)
            for t in range(n):
                for j in range(c.top_k):
                    e = int(idx[t, j])
                    g, up = (w[p + "w1"][e] @ x2[t]).to(torch.bfloat16), (w[p + "w3"][e] @ x2[t]).to(torch.bfloat16)
                    y[t] += val[t, j] * (w[p + "w2"][e] @ LA.softcapped_swiglu(g.contiguous(), up.contiguous(), c.act_cap).float())
            h = h + y
        logits = (_rms(h, w["norm"], c.eps) @ w["head"].t()).contiguous()
        return LA.softcap_(logits, c.logit_cap)
