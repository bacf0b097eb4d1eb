"""Dory-1.0-style latent-recurrence decoder: a prelude layer, ONE shared transformer block applied ``loops`` times to the
latent (each loop re-injects the prelude's output and keeps its own KV cache, since loop i at position t attends to the
loop-i latents of earlier positions), a coda layer and the head.  Depth comes from iteration, not from distinct weights.

The loops are what the ring pipeline splits: rank r of W runs loops [r*loops/W, (r+1)*loops/W) on the full width, keeps the
KV caches of exactly those loops, and hands the latent rows to rank r+1 (``parallel/ring.py``).  Rank 0 also runs the
prelude, the last rank also runs the coda and the head.  ``LoopStage`` is the per-rank piece; with W = 1 it is the whole
model, which is how the one-process reference below is built.

Reference behaviour: crates/sparkflash-model-dory (host + device forward), src/recurrence.rs:15-84 (send_bf16 / recv_bf16
ring; lanes keep all ranks busy).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class DoryConfig:
    vocab: int = 256
    d: int = 64
    heads: int = 4
    loops: int = 6
    inter: int = 128
    theta: float = 10000.0
    eps: float = 1e-6


def init_weights(c: DoryConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * s[-1] ** -0.5
    w = {"embed": torch.randn(c.vocab, c.d, generator=g), "head": r(c.vocab, c.d), "norm": torch.ones(c.d),
         "inject": r(c.d, 2 * c.d)}
    for name in ("prelude", "core", "coda"):
        p = name + "."
        w[p + "n1"], w[p + "n2"] = torch.ones(c.d), torch.ones(c.d)
        for m in ("wq", "wk", "wv", "wo"):
            w[p + m] = r(c.d, c.d)
        w[p + "w1"], w[p + "w3"], w[p + "w2"] = r(c.inter, c.d), r(c.inter, c.d), r(c.d, c.inter)
    return w


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):
    hd = x.shape[-1]
    inv = theta ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)
    ang = pos.to(torch.float32)[:, None, None] * inv
    co, si = torch.cos(ang), torch.sin(ang)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * co - b * si, a * si + b * co], -1).flatten(-2)


class _Layer:
    """One transformer layer with a growing per-lane KV cache (prefill chunks and decode rows alike)."""

    def __init__(self, c: DoryConfig, w, prefix: str):
        self.c, self.w, self.p = c, w, prefix
        self.k: dict[int, torch.Tensor] = {}
        self.v: dict[int, torch.Tensor] = {}

    def run(self, lane: int, pos: int, x: torch.Tensor) -> torch.Tensor:
        c, w, p = self.c, self.w, self.p
        T, H, hd = x.shape[0], c.heads, c.d // c.heads
        at = torch.arange(pos, pos + T)
        h = _rms(x, w[p + "n1"], c.eps)
        q = _rope((h @ w[p + "wq"].t()).reshape(T, H, hd), at, c.theta)
        k = _rope((h @ w[p + "wk"].t()).reshape(T, H, hd), at, c.theta)
        v = (h @ w[p + "wv"].t()).reshape(T, H, hd)
        kc = torch.cat([self.k.get(lane, torch.zeros(0, H, hd))[:pos], k])       # a step at ``pos`` overwrites from there on
        vc = torch.cat([self.v.get(lane, torch.zeros(0, H, hd))[:pos], v])
        self.k[lane], self.v[lane] = kc, vc
        s = torch.einsum("thd,shd->hts", q, kc) * hd ** -0.5
        s = s.masked_fill(torch.arange(kc.shape[0])[None, :] > at[:, None], float("-inf"))
        x = x + torch.einsum("hts,shd->thd", torch.softmax(s, -1), vc).reshape(T, c.d) @ w[p + "wo"].t()
        h = _rms(x, w[p + "n2"], c.eps)
        return x + (F.silu(h @ w[p + "w1"].t()) * (h @ w[p + "w3"].t())) @ w[p + "w2"].t()


class LoopStage:
    """The share of the model one ring rank runs.  The latent that travels between ranks is [rows, 2d]: the recurrent
    state and the prelude output that every loop re-injects."""

    def __init__(self, c: DoryConfig, w, rank: int = 0, world: int = 1):
        self.c, self.w, self.rank, self.world = c, w, rank, world
        self.loops = range(rank * c.loops // world, (rank + 1) * c.loops // world)
        self.prelude = _Layer(c, w, "prelude.") if rank == 0 else None
        self.core = {i: _Layer(c, w, "core.") for i in self.loops}            # same weights, one KV cache per loop
        self.coda = _Layer(c, w, "coda.") if rank == world - 1 else None

    @property
    def width(self) -> int:
        return 2 * self.c.d

    def embed(self, tokens: list[int]) -> torch.Tensor:
        """Rank 0: token rows -> the [rows, 2d] frame (state starts as zeros; the prelude runs inside ``stage``)."""
        e = self.w["embed"][torch.tensor(tokens)]
        return torch.cat([torch.zeros_like(e), e], -1)

    def stage(self, lane: int, pos: int, frame: torch.Tensor) -> torch.Tensor:
        c = self.c
        s, e = frame[:, :c.d], frame[:, c.d:]
        if self.prelude is not None:
            e = self.prelude.run(lane, pos, e)
            s = e.clone()
        for i in self.loops:
            s = self.core[i].run(lane, pos, torch.cat([s, e], -1) @ self.w["inject"].t())
        return torch.cat([s, e], -1)

    def head(self, lane: int, pos: int, frame: torch.Tensor) -> torch.Tensor:
        return self.logits(lane, pos, frame).argmax(-1)

    def logits(self, lane: int, pos: int, frame: torch.Tensor) -> torch.Tensor:
        x = self.coda.run(lane, pos, frame[:, :self.c.d])
        return _rms(x, self.w["norm"], self.c.eps) @ self.w["head"].t()


def reference_logits(c: DoryConfig, w, tokens: list[int]) -> torch.Tensor:
    """The whole sequence in one process: logits [T, vocab]."""
    st = LoopStage(c, w)
    return st.logits(0, 0, st.stage(0, 0, st.embed(tokens)))


def ring_generate(c: DoryConfig, w, prompts: dict[int, list[int]], n_new: int, device="cpu") -> dict[int, list[int]] | None:
    """Greedy generation for several lanes through the recurrence ring of the current ``torch.distributed`` group.
    Every rank calls this; rank 0 returns {lane: tokens}, the others None.  The lanes' steps are interleaved so that
    up to world-1 of them are in flight."""
    import torch.distributed as dist
    from ..parallel.ring import RingStage
    rank, world = dist.get_rank(), dist.get_world_size()
    st = LoopStage(c, w, rank, world)
    ring = RingStage(st.stage, st.head if rank == world - 1 else None, st.width, device=device)
    if rank != 0:
        ring.serve()
        return None
    out = {l: [] for l in prompts}
    answers = ring.drive([(l, 0, st.embed(p)) for l, p in prompts.items()])          # prefill: one chunk per lane
    nxt = {l: int(a[-1]) for l, a in zip(prompts, answers)}
    pos = {l: len(p) for l, p in prompts.items()}
    for _ in range(n_new):
        for l in prompts:
            out[l].append(nxt[l])
        answers = ring.drive([(l, pos[l], st.embed([nxt[l]])) for l in prompts])
        for l, a in zip(prompts, answers):
            nxt[l], pos[l] = int(a[-1]), pos[l] + 1
    ring.shutdown()
    return out


def generate(c: DoryConfig, w, prompt: list[int], n_new: int) -> list[int]:
    """One process, one lane: the reference for ``ring_generate``."""
    st = LoopStage(c, w)
    tok = int(st.head(0, 0, st.stage(0, 0, st.embed(prompt)))[-1])
    out, pos = [], len(prompt)
    for _ in range(n_new):
        out.append(tok)
        tok = int(st.head(0, pos, st.stage(0, pos, st.embed([tok])))[-1])
        pos += 1
    return out
