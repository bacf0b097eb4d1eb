"""DFlash-style block drafter: a single small transformer block that proposes a whole block of tokens in ONE forward
(no token-by-token loop).  The target model leaves one feature row per position (a capture of its hidden state) in a
ring buffer; the drafter's block is [anchor token, mask, mask, ...]: every block position attends to the ring's features
and to the whole block (no causal mask inside the block), and the shared head turns positions 1.. into proposals.
Rejected proposals cost nothing to undo: the ring is written only by the target's accepted positions.

* ``FeatureRing``   position-addressed ring of target features (slot = position % size), per lane;
* ``BlockDrafter``  the drafter forward (fp32 PyTorch; the same code runs on CPU or GPU tensors);
* ``accept``        longest prefix of the proposals that the target reproduces, plus the target's own next token;
* ``speculate``     the draft -> verify -> accept loop against any target exposing ``step(tokens, pos) -> (next tokens,
                    features)``.

Reference behaviour: kernels/dflash2_sm121.cu (q4d_capture, block_embed, conv, kv_ring, attn, attn_span_chunk / merge,
topk_partial / final, select - a KV ring buffer, not ring attention); DFlash / DFlash-2 drafters of the Qwen and GLM
families (crates/sparkflash-model-qwen4-exp, crates/sparkflash-model-glm5-next).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class DFlashConfig:
    vocab: int = 256
    d: int = 64              # drafter width
    feat: int = 64           # width of the captured target feature
    heads: int = 4
    block: int = 5           # anchor + 4 proposals
    ring: int = 16
    inter: int = 128
    eps: float = 1e-6


def init_weights(c: DFlashConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * s[-1] ** -0.5
    return {"embed": torch.randn(c.vocab, c.d, generator=g), "mask": torch.randn(c.d, generator=g),
            "slot": torch.randn(c.block, c.d, generator=g) * 0.1, "feat_k": r(c.d, c.feat), "feat_v": r(c.d, c.feat),
            "n1": torch.ones(c.d), "n2": torch.ones(c.d), "wq": r(c.d, c.d), "wk": r(c.d, c.d), "wv": r(c.d, c.d),
            "wo": r(c.d, c.d), "w1": r(c.inter, c.d), "w3": r(c.inter, c.d), "w2": r(c.d, c.inter),
            "norm": torch.ones(c.d), "head": r(c.vocab, c.d)}


class FeatureRing:
    def __init__(self, c: DFlashConfig, lanes: int = 1, device="cpu"):
        self.c = c
        self.buf = torch.zeros((lanes, c.ring, c.feat), device=device)
        self.filled = [0] * lanes          # positions [max(0, filled - ring), filled) are valid

    def write(self, lane: int, pos: int, feats: torch.Tensor) -> None:
        """Features of positions pos .. pos + rows - 1 (accepted positions only)."""
        for i in range(feats.shape[0]):
            self.buf[lane, (pos + i) % self.c.ring] = feats[i]
        self.filled[lane] = pos + feats.shape[0]

    def rewind(self, lane: int, pos: int) -> None:
        self.filled[lane] = min(self.filled[lane], pos)

    def window(self, lane: int) -> torch.Tensor:
        """Valid features, oldest first."""
        hi = self.filled[lane]
        lo = max(0, hi - self.c.ring)
        return self.buf[lane, [p % self.c.ring for p in range(lo, hi)]]


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


class BlockDrafter:
    def __init__(self, c: DFlashConfig, w: dict[str, torch.Tensor]):
        self.c, self.w = c, w

    def logits(self, anchor: int, feats: torch.Tensor) -> torch.Tensor:
        """Logits [block - 1, vocab] for the positions after the anchor; ``feats`` = the ring window [n, feat]."""
        c, w = self.c, self.w
        B, H, hd = c.block, c.heads, c.d // c.heads
        x = torch.cat([w["embed"][anchor][None], w["mask"].expand(B - 1, -1)]) + w["slot"]
        h = _rms(x, w["n1"], c.eps)
        q = (h @ w["wq"].t()).reshape(B, H, hd)
        k = torch.cat([feats @ w["feat_k"].t(), h @ w["wk"].t()]).reshape(-1, H, hd)      # ring keys, then the block's own
        v = torch.cat([feats @ w["feat_v"].t(), h @ w["wv"].t()]).reshape(-1, H, hd)
        s = torch.einsum("bhd,shd->hbs", q, k) * hd ** -0.5                                 # no mask: the block sees itself whole
        x = x + torch.einsum("hbs,shd->bhd", torch.softmax(s, -1), v).reshape(B, c.d) @ w["wo"].t()
        h = _rms(x, w["n2"], c.eps)
        x = x + (F.silu(h @ w["w1"].t()) * (h @ w["w3"].t())) @ w["w2"].t()
        return _rms(x[1:], w["norm"], c.eps) @ w["head"].t()

    def propose(self, anchor: int, feats: torch.Tensor) -> list[int]:
        return self.logits(anchor, feats).argmax(-1).tolist()


def accept(proposals: list[int], target_next: list[int]) -> tuple[int, list[int]]:
    """``target_next[i]`` = the target's token after row i of [anchor, proposals...].  Returns (number of proposals kept,
    tokens emitted = the kept proposals plus the target's own token after the last kept row)."""
    a = 0
    while a < len(proposals) and proposals[a] == target_next[a]:
        a += 1
    return a, proposals[:a] + [target_next[a]]


def speculate(target, drafter: BlockDrafter, ring: FeatureRing, lane: int, first_token: int, pos: int, n_new: int):
    """Generate ``n_new`` tokens after ``first_token`` (which sits at position ``pos`` and is not yet in the target's
    caches).  ``target.step(tokens, pos)`` runs rows at pos.., returns (next token per row, feature per row) and must
    accept being called again at an earlier position (position-addressed caches).  Returns (tokens, forwards used)."""
    out, tok, forwards = [], first_token, 0
    while len(out) < n_new:
        props = drafter.propose(tok, ring.window(lane))
        nxt, feats = target.step([tok] + props, pos)
        forwards += 1
        a, emitted = accept(props, nxt)
        ring.write(lane, pos, feats[:a + 1])            # only the rows that stay
        out.extend(emitted)
        tok, pos = emitted[-1], pos + a + 1
    return out[:n_new], forwards
