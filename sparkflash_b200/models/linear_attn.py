"""Linear-attention and convolution state layers of the Qwen-style (gated delta-net, KDA) and Inkling-style (short
convolution, soft-capping) families: fp32 references, the device kernels (csrc/k_families.cu), and snapshot / restore
of the recurrent state - a speculative step that is rejected must put the state back, because unlike a
position-addressed KV cache a recurrent state cannot be rewound by moving a pointer.
Reference: crates/sparkflash-model-qwen4-exp (tests batch_exactness.rs, verify_rows.rs, checkpoint_roundtrip.rs),
crates/sparkflash-model-inkling2 (conv_history_copy / restore)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from .. import _lib
from ..ops import native as N


def delta_rule_reference(q, k, v, a, b, S):
    """One sequence.  q,k [T,H,dk], v [T,H,dv], a [T,H] or [T,H,dk], b [T,H]; S [H,dk,dv] is updated in place."""
    T = q.shape[0]
    out = torch.empty(T, q.shape[1], v.shape[2])
    for t in range(T):
        at = a[t].unsqueeze(-1) if a.dim() == 3 else a[t].reshape(-1, 1, 1)
        S.mul_(at if a.dim() == 2 else at)
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        r = (v[t] - mem) * b[t].unsqueeze(-1)
        S.add_(torch.einsum("hk,hv->hkv", k[t], r))
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def short_conv_reference(x, w, hist, silu=True):
    """x [T,C] (bf16 values), w [C,W], hist [C,W-1] updated in place; returns bf16-rounded y [T,C]."""
    W = w.shape[1]
    full = torch.cat([hist.t(), x.float()], 0)
    y = sum(full[j:j + x.shape[0]] * w[:, j] for j in range(W))
    if silu:
        y = y * torch.sigmoid(y)
    hist.copy_(full[-(W - 1):].t())
    return y.to(torch.bfloat16)


def softcap_reference(x, cap):
    return cap * torch.tanh(x / cap)


class DeltaState:
    """Per-lane recurrent states on the device with snapshots."""

    def __init__(self, lanes: int, H: int, dk: int, dv: int, per_channel: bool = False, device="cuda"):
        self.S = torch.zeros((lanes, H, dk, dv), dtype=torch.float32, device=device)
        self.H, self.dk, self.dv, self.per_channel = H, dk, dv, per_channel
        self._snap: dict[int, torch.Tensor] = {}

    def step(self, q, k, v, a, b, row_lane: list[int]) -> torch.Tensor:
        """Rows of any mix of lanes (each lane's rows consecutive and in order): fp32 tensors on the device."""
        T = q.shape[0]
        out = torch.empty((T, self.H, self.dv), dtype=torch.float32, device=q.device)
        lanes = sorted(set(row_lane))
        rl = torch.tensor(row_lane, dtype=torch.int32, device=q.device)
        li = torch.tensor(lanes, dtype=torch.int32, device=q.device)
        N._check(_lib.cuda().sfb_delta_rule(N._p(q.contiguous()), N._p(k.contiguous()), N._p(v.contiguous()), N._p(a.contiguous()), N._p(b.contiguous()),
                                            N._p(self.S), N._p(out), N._p(rl), N._p(li), c_int(len(lanes)), c_int(T), c_int(self.H), c_int(self.dk),
                                            c_int(self.dv), c_int(int(self.per_channel)), N._stream()), "delta_rule")
        return out

    def snapshot(self, lane: int) -> None:
        self._snap[lane] = self.S[lane].clone()

    def restore(self, lane: int) -> None:
        self.S[lane].copy_(self._snap[lane])


class ConvState:
    def __init__(self, lanes: int, C: int, W: int, device="cuda"):
        self.hist = torch.zeros((lanes, C, W - 1), dtype=torch.float32, device=device)
        self.C, self.W = C, W
        self._snap: dict[int, torch.Tensor] = {}

    def step(self, x, w, row_lane: list[int], silu: bool = True) -> torch.Tensor:
        T = x.shape[0]
        y = torch.empty_like(x)
        lanes = sorted(set(row_lane))
        rl = torch.tensor(row_lane, dtype=torch.int32, device=x.device)
        li = torch.tensor(lanes, dtype=torch.int32, device=x.device)
        N._check(_lib.cuda().sfb_short_conv(N._p(x.contiguous()), N._p(w), N._p(self.hist), N._p(y), N._p(rl), N._p(li), c_int(len(lanes)), c_int(T),
                                            c_int(self.C), c_int(self.W), c_int(int(silu)), N._stream()), "short_conv")
        return y

    def snapshot(self, lane: int) -> None:
        self._snap[lane] = self.hist[lane].clone()

    def restore(self, lane: int) -> None:
        self.hist[lane].copy_(self._snap[lane])


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    N._check(_lib.cuda().sfb_softcap(N._p(x), c_longlong(x.numel()), c_float(cap), N._stream()), "softcap")
    return x


def softcapped_swiglu(g: torch.Tensor, u: torch.Tensor, cap: float) -> torch.Tensor:
    y = torch.empty_like(g)
    N._check(_lib.cuda().sfb_softcapped_swiglu(N._p(g), N._p(u), N._p(y), c_longlong(g.numel()), c_float(cap), N._stream()), "softcapped_swiglu")
    return y
