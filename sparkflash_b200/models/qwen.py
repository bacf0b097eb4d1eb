"""Qwen3.8-Flash-Next-style hybrid decoder: three linear-attention layers (gated delta-net, or KDA with per-channel
decay) for every full-attention layer (gated softmax attention with per-head q/k RMSNorm), a softmax-router MoE with a
shared expert in every layer, tied to a recurrent state per sequence instead of a growing KV cache in the linear layers.

Two forwards over the same weights:

* ``reference_logits`` - the whole sequence on the CPU in fp32, plain PyTorch, the oracle;
* ``HybridEngine`` - a rows step on the device: any mix of lanes per step (each lane's rows consecutive and in order), the
  recurrences through the delta-rule and short-convolution kernels (csrc/k_families.cu) with per-lane states, the full
  attention over a per-lane KV cache, projections as library GEMMs.  ``snapshot`` / ``restore`` put a lane's recurrent
  state back after rejected speculative rows.

Reference behaviour: crates/sparkflash-model-qwen4-exp (host + device forward; tests batch_exactness.rs, verify_rows.rs,
checkpoint_roundtrip.rs), kernels/qwen4_scan_sm121.cu (gdn_conv, gdn_prep / kda_prep, gdn_scan / kda_scan, gdn_gate).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import linear_attn as LA


@dataclass
class HybridConfig:
    vocab: int = 512
    d: int = 128
    layers: int = 4
    full_every: int = 4          # layer l is full attention when (l + 1) % full_every == 0
    heads: int = 4               # full-attention heads
    head_dim: int = 32
    lin_heads: int = 4           # linear-attention heads
    dk: int = 32
    dv: int = 32
    conv_width: int = 4
    kda: bool = False            # per-channel decay (KDA) instead of one decay per head (GDN)
    experts: int = 8
    top_k: int = 2
    inter: int = 64
    rope_theta: float = 10000.0
    eps: float = 1e-6

    def is_full(self, l: int) -> bool:
        return (l + 1) % self.full_every == 0


def init_weights(c: HybridConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)

    def r(*shape, s=None):
        s = s if s is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).float()     # bf16-representable values
    w = {"embed": r(c.vocab, c.d, s=1.0), "head": r(c.vocab, c.d), "norm": torch.ones(c.d)}
    for l in range(c.layers):
        p = f"l{l}."
        w[p + "n1"], w[p + "n2"] = torch.ones(c.d), torch.ones(c.d)
        if c.is_full(l):
            H, hd = c.heads, c.head_dim
            w[p + "wq"], w[p + "wk"], w[p + "wv"] = r(H * hd, c.d), r(H * hd, c.d), r(H * hd, c.d)
            w[p + "wg"] = r(H * hd, c.d)                    # output gate
            w[p + "qn"], w[p + "kn"] = torch.ones(hd), torch.ones(hd)
            w[p + "wo"] = r(c.d, H * hd)
        else:
            H, dk, dv = c.lin_heads, c.dk, c.dv
            C = H * (2 * dk + dv)
            w[p + "wqkv"] = r(C, c.d)
            w[p + "conv"] = r(C, c.conv_width, s=0.5)
            w[p + "wa"] = r(H * dk if c.kda else H, c.d)    # decay logits
            w[p + "a_bias"] = torch.full((H * dk if c.kda else H,), 2.0)
            w[p + "wb"] = r(H, c.d)                          # write strength
            w[p + "wg"] = r(H * dv, c.d)
            w[p + "on"] = torch.ones(dv)
            w[p + "wo"] = r(c.d, H * dv)
        w[p + "router"] = r(c.experts, c.d)
        w[p + "w1"], w[p + "w3"] = r(c.experts, c.inter, c.d), r(c.experts, c.inter, c.d)
        w[p + "w2"] = r(c.experts, c.d, c.inter)
        w[p + "s1"], w[p + "s3"], w[p + "s2"] = r(c.inter, c.d), r(c.inter, c.d), r(c.d, c.inter)
    return w


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):
    """x [T, H, hd], pos [T]: rotate pairs (2i, 2i+1)."""
    hd = x.shape[-1]
    inv = theta ** (-torch.arange(0, hd, 2, dtype=torch.float32, device=x.device) / hd)
    ang = pos.to(torch.float32)[:, None, None] * inv
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)


def _moe(c: HybridConfig, w, p, x):
    probs = torch.softmax(x @ w[p + "router"].t(), -1)
    val, idx = torch.topk(probs, c.top_k, -1)
    val = val / val.sum(-1, keepdim=True)
    y = (F.silu(x @ w[p + "s1"].t()) * (x @ w[p + "s3"].t())) @ w[p + "s2"].t()
    for t in range(x.shape[0]):
        for j in range(c.top_k):
            e = int(idx[t, j])
            h = F.silu(w[p + "w1"][e] @ x[t]) * (w[p + "w3"][e] @ x[t])
            y[t] = y[t] + val[t, j] * (w[p + "w2"][e] @ h)
    return y


def _lin_inputs(c: HybridConfig, w, p, x, conv_out):
    """Split the convolved qkv and compute decay / strength: q,k [T,H,dk] (unit length), v [T,H,dv], a, b."""
    H, dk, dv = c.lin_heads, c.dk, c.dv
    T = x.shape[0]
    q, k, v = conv_out.split([H * dk, H * dk, H * dv], -1)
    q = F.normalize(q.reshape(T, H, dk), dim=-1) * dk ** -0.5
    k = F.normalize(k.reshape(T, H, dk), dim=-1)
    v = v.reshape(T, H, dv)
    a = torch.exp(-F.softplus(-(x @ w[p + "wa"].t() + w[p + "a_bias"])))          # sigmoid, written as a decay in (0, 1)
    a = a.reshape(T, H, dk) if c.kda else a.reshape(T, H)
    b = torch.sigmoid(x @ w[p + "wb"].t())
    return q, k, v, a, b


def reference_logits(c: HybridConfig, w, tokens: list[int]) -> torch.Tensor:
    """fp32 CPU oracle: logits [T, vocab] of one sequence."""
    T = len(tokens)
    pos = torch.arange(T)
    h = w["embed"][torch.tensor(tokens)]
    for l in range(c.layers):
        p = f"l{l}."
        x = _rms(h, w[p + "n1"], c.eps)
        if c.is_full(l):
            H, hd = c.heads, c.head_dim
            q = _rope(_rms((x @ w[p + "wq"].t()).reshape(T, H, hd), w[p + "qn"], c.eps), pos, c.rope_theta)
            k = _rope(_rms((x @ w[p + "wk"].t()).reshape(T, H, hd), w[p + "kn"], c.eps), pos, c.rope_theta)
            v = (x @ w[p + "wv"].t()).reshape(T, H, hd)
            s = torch.einsum("thd,shd->hts", q, k) * hd ** -0.5
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(T, H * hd)
            y = (o * torch.sigmoid(x @ w[p + "wg"].t())) @ w[p + "wo"].t()
        else:
            H, dk, dv = c.lin_heads, c.dk, c.dv
            qkv = (x @ w[p + "wqkv"].t()).to(torch.bfloat16)
            hist = torch.zeros(qkv.shape[1], c.conv_width - 1)
            conv = LA.short_conv_reference(qkv, w[p + "conv"], hist).float()
            q, k, v, a, b = _lin_inputs(c, w, p, x, conv)
            S = torch.zeros(H, dk, dv)
            o = LA.delta_rule_reference(q, k, v, a, b, S)
            o = _rms(o, w[p + "on"], c.eps).reshape(T, H * dv) * F.silu(x @ w[p + "wg"].t())
            y = o @ w[p + "wo"].t()
        h = h + y
        h = h + _moe(c, w, p, _rms(h, w[p + "n2"], c.eps))
    return _rms(h, w["norm"], c.eps) @ w["head"].t()


class HybridEngine:
    """Rows step on the device.  Per-lane state: delta-rule matrices and convolution histories for the linear layers, a KV
    cache for the full-attention layers."""

    def __init__(self, c: HybridConfig, w: dict[str, torch.Tensor], lanes: int = 2, max_context: int = 256, device="cuda"):
        self.c, self.dev = c, device
        self.w = {k: v.to(device) for k, v in w.items()}
        self.delta, self.conv, self.kc, self.vc = {}, {}, {}, {}
        for l in range(c.layers):
            if c.is_full(l):
                self.kc[l] = torch.zeros((lanes, max_context, c.heads, c.head_dim), device=device)
                self.vc[l] = torch.zeros_like(self.kc[l])
            else:
                self.delta[l] = LA.DeltaState(lanes, c.lin_heads, c.dk, c.dv, per_channel=c.kda, device=device)
                self.conv[l] = LA.ConvState(lanes, c.lin_heads * (2 * c.dk + c.dv), c.conv_width, device=device)

    def snapshot(self, lane: int) -> None:
        for s in list(self.delta.values()) + list(self.conv.values()):
            s.snapshot(lane)

    def restore(self, lane: int) -> None:
        for s in list(self.delta.values()) + list(self.conv.values()):
            s.restore(lane)

    def step(self, tokens: list[int], lanes: list[int], positions: list[int]) -> torch.Tensor:
        """Logits [n, vocab] (fp32, device) for the rows; a lane's rows must be consecutive and in position order."""
        c, w, dev = self.c, self.w, self.dev
        n = len(tokens)
        pos = torch.tensor(positions, device=dev)
        lane_t = torch.tensor(lanes, device=dev)
        h = w["embed"][torch.tensor(tokens, device=dev)]
        for l in range(c.layers):
            p = f"l{l}."
            x = _rms(h, w[p + "n1"], c.eps)
            if c.is_full(l):
                H, hd = c.heads, c.head_dim
                q = _rope(_rms((x @ w[p + "wq"].t()).reshape(n, H, hd), w[p + "qn"], c.eps), pos, c.rope_theta)
                k = _rope(_rms((x @ w[p + "wk"].t()).reshape(n, H, hd), w[p + "kn"], c.eps), pos, c.rope_theta)
                v = (x @ w[p + "wv"].t()).reshape(n, H, hd)
                self.kc[l][lane_t, pos] = k
                self.vc[l][lane_t, pos] = v
                o = torch.empty((n, H, hd), device=dev)
                for i in range(n):          # position-addressed cache: a row sees its lane's entries up to its own position
                    L, P = lanes[i], positions[i] + 1
                    s = torch.einsum("hd,shd->hs", q[i], self.kc[l][L, :P]) * hd ** -0.5
                    o[i] = torch.einsum("hs,shd->hd", torch.softmax(s, -1), self.vc[l][L, :P])
                y = (o.reshape(n, H * hd) * torch.sigmoid(x @ w[p + "wg"].t())) @ w[p + "wo"].t()
            else:
                H, dv = c.lin_heads, c.dv
                qkv = (x @ w[p + "wqkv"].t()).to(torch.bfloat16)
                conv = self.conv[l].step(qkv, w[p + "conv"], lanes).float()
                q, k, v, a, b = _lin_inputs(c, w, p, x, conv)
                o = self.delta[l].step(q, k, v, a, b, lanes)
                o = _rms(o, w[p + "on"], c.eps).reshape(n, H * dv) * F.silu(x @ w[p + "wg"].t())
                y = o @ w[p + "wo"].t()
            h = h + y
            h = h + _moe(c, w, p, _rms(h, w[p + "n2"], c.eps))
        return _rms(h, w["norm"], c.eps) @ w["head"].t()
