"""DeepSeek-ViT tower and the 3x3 aligner: bf16 end to end with fp32 norm weights, replicated on every rank.

On the GPU every projection whose reduction length is a multiple of 64 runs on this framework's bf16 tensor-core GEMM
(csrc/k_umma.cu, kind::f16: the tower's weights are the M operand, the image's patches the token columns); the patch
embedding (K = 588) and the CPU path use torch.  Attention over one image is a single unmasked SDPA call; the rotary and
the aligner's unfold are this framework's kernels (csrc/k_vision.cu) with torch twins used on the CPU.
Reference: docs/architecture/06-vision.md sections 1, 3, 4; kernels/opt_vision_sm121.cu:172 (the reference's own bf16 GEMM).
"""
from __future__ import annotations

from ctypes import c_float, c_int

import torch
import torch.nn.functional as F

from .plan import IMAGE, IMAGE_END, IMAGE_NEW_LINE, IMAGE_START, ImagePlan, VisionConfig


def synthetic_vision_weights(c: VisionConfig, seed: int = 0, device="cpu") -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    bf = lambda *s, sc=0.02: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16).to(device)
    w = {"patch_embed.weight": bf(c.dim, 3 * c.patch_size ** 2), "patch_embed.bias": bf(c.dim), "norm.weight": torch.ones(c.dim, device=device)}
    for l in range(c.n_layers):
        p = f"blocks.{l}."
        w[p + "attn_norm.weight"] = torch.ones(c.dim, device=device) + torch.randn(c.dim, generator=g).to(device) * 0.01
        w[p + "ffn_norm.weight"] = torch.ones(c.dim, device=device)
        w[p + "wqkv.weight"], w[p + "wqkv.bias"] = bf(3 * c.dim, c.dim), bf(3 * c.dim)
        w[p + "wo.weight"], w[p + "wo.bias"] = bf(c.dim, c.dim), bf(c.dim)
        w[p + "w1.weight"], w[p + "w2.weight"] = bf(2 * c.inter_dim, c.dim), bf(c.dim, c.inter_dim)
    k = c.downsample_ratio ** 2
    w["aligner.w1.weight"], w["aligner.w1.bias"] = bf(c.llm_dim, c.dim * k), bf(c.llm_dim)
    w["aligner.w2.weight"], w["aligner.w2.bias"] = bf(c.llm_dim, c.llm_dim), bf(c.llm_dim)
    for n in ("image_start", "image_end", "image_newline"):
        w[n] = bf(c.llm_dim)
    return w


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w).to(torch.bfloat16)


def rope_reference(x: torch.Tensor, n_w: int, theta: float) -> torch.Tensor:
    """x bf16 [N, heads, hd]; half-split rotation, frequencies alternate row / column position."""
    N, _, hd = x.shape
    half = hd // 2
    k = torch.arange(half)
    inv = theta ** (-2.0 * (k // 2).float() / half)
    n = torch.arange(N)
    pos = torch.where((k % 2 == 1).unsqueeze(0), (n % n_w).unsqueeze(1), (n // n_w).unsqueeze(1)).float()
    ang = pos * inv
    cos, sin = ang.cos().to(torch.bfloat16).float().unsqueeze(1), ang.sin().to(torch.bfloat16).float().unsqueeze(1)
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([(a * cos - b * sin).to(torch.bfloat16), (b * cos + a * sin).to(torch.bfloat16)], -1)


def unfold3_reference(x: torch.Tensor, n_h: int, n_w: int) -> torch.Tensor:
    C = x.shape[-1]
    g = x.reshape(n_h, n_w, C).permute(2, 0, 1).float()
    g = F.pad(g, (0, (-n_w) % 3, 0, (-n_h) % 3))
    return F.unfold(g.unsqueeze(0), 3, stride=3)[0].t().to(torch.bfloat16).contiguous()


def _rope(x, n_w, theta):
    if x.is_cuda:
        from .. import _lib
        from ..ops import native as N
        x = x.contiguous()
        N._check(_lib.cuda().sfb_vision_rope(N._p(x), c_int(x.shape[0]), c_int(x.shape[1]), c_int(x.shape[2]), c_int(n_w), c_float(theta), N._stream()), "vision_rope")
        return x
    return rope_reference(x, n_w, theta)


def _unfold3(x, n_h, n_w):
    if x.is_cuda:
        from .. import _lib
        from ..ops import native as N
        C = x.shape[-1]
        out = torch.empty((((n_h + 2) // 3) * ((n_w + 2) // 3), C * 9), dtype=torch.bfloat16, device=x.device)
        N._check(_lib.cuda().sfb_vision_unfold3(N._p(x.contiguous()), c_int(n_h), c_int(n_w), c_int(C), N._p(out), N._stream()), "vision_unfold3")
        return out
    return unfold3_reference(x, n_h, n_w)


class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: dict[str, torch.Tensor]):
        self.c, self.w = cfg, weights
        self._maps: dict[int, object] = {}
        self.tc_gemms = 0                 # projections that ran on the tensor-core GEMM (tests look at it)

    def _linear(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """x bf16 [N, K] times weight bf16 [out, K] (+ bias): tcgen05 on the GPU when K is a multiple of 64."""
        K = weight.shape[1]
        if not x.is_cuda or K % 64 or weight.dtype != torch.bfloat16:
            return F.linear(x, weight, bias)
        from ..ops import native as N
        x = x.to(torch.bfloat16).contiguous()
        n, out_dim = x.shape[0], weight.shape[0]
        ta = self._maps.get(weight.data_ptr())
        if ta is None:
            ta = self._maps[weight.data_ptr()] = N.bf16_map(weight.contiguous(), out_dim, K, 128)
        NP = 128 if n > 128 else N.umma_np(n)
        tb = N.bf16_map(x, n, K, NP)
        y = torch.empty((n, out_dim), dtype=torch.bfloat16, device=x.device)
        N.umma_bf16(ta, tb, n, out_dim, K, out_b=y, out_stride=out_dim, NP=NP)
        self.tc_gemms += 1
        return y if bias is None else y + bias

    @torch.no_grad()
    def encode(self, patches: torch.Tensor, plan: ImagePlan) -> torch.Tensor:
        """bf16 patches [n_vit_h*n_vit_w, 588] -> bf16 [n_llm_h*n_llm_w, llm_dim] image-token embeddings (row-major)."""
        c, w = self.c, self.w
        N, H, hd = patches.shape[0], c.n_heads, c.dim // c.n_heads
        x = F.linear(patches, w["patch_embed.weight"], w["patch_embed.bias"])
        for l in range(c.n_layers):
            p = f"blocks.{l}."
            qkv = self._linear(_rms(x, w[p + "attn_norm.weight"], c.norm_eps), w[p + "wqkv.weight"], w[p + "wqkv.bias"])
            q, k, v = qkv.reshape(N, 3, H, hd).unbind(1)
            q, k = _rope(q, plan.n_vit_w, c.rope_theta), _rope(k, plan.n_vit_w, c.rope_theta)
            o = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0))
            x = x + self._linear(o[0].transpose(0, 1).reshape(N, c.dim), w[p + "wo.weight"], w[p + "wo.bias"])
            gu = self._linear(_rms(x, w[p + "ffn_norm.weight"], c.norm_eps), w[p + "w1.weight"])
            gate, up = gu.chunk(2, -1)
            x = x + self._linear(F.silu(gate) * up, w[p + "w2.weight"])
        x = _rms(x, w["norm.weight"], c.norm_eps)
        u = _unfold3(x, plan.n_vit_h, plan.n_vit_w)
        return self._linear(F.gelu(self._linear(u, w["aligner.w1.weight"], w["aligner.w1.bias"])), w["aligner.w2.weight"], w["aligner.w2.bias"])

    def span_embeddings(self, image_tokens: torch.Tensor, plan: ImagePlan) -> torch.Tensor:
        """Rows of the whole span in prompt order: start, (n_llm_w image rows + newline) * n_llm_h, end."""
        w = self.w
        grid = image_tokens.reshape(plan.n_llm_h, plan.n_llm_w, -1)
        nl = w["image_newline"].to(grid.device).expand(plan.n_llm_h, 1, -1)
        body = torch.cat([grid, nl], 1).reshape(-1, grid.shape[-1])
        return torch.cat([w["image_start"].to(grid.device).unsqueeze(0), body, w["image_end"].to(grid.device).unsqueeze(0)], 0)
