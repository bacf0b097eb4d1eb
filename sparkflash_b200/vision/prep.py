"""Image decode and preparation: decode, aspect-preserving resize with mid-grey padding, normalisation to
[-1, 1] and patch extraction.  The resample + pad + normalise + patchify chain is one CUDA kernel
(csrc/k_vision.cu) with a torch CPU twin.  Reference: crates/sparkflash-vision/src/{decode,resample,prep}.rs,
kernels/opt_vision_sm121.cu; docs/architecture/06-vision.md section 2 steps 5-7.
"""
from __future__ import annotations

import base64
import io
from ctypes import c_int, c_void_p

import torch

from .plan import ImagePlan, VisionConfig

GREY = 127


def decode_image(source) -> torch.Tensor:
    """bytes | data: URL | file path -> uint8 [H, W, 3]."""
    from PIL import Image
    import numpy as np
    if isinstance(source, str) and source.startswith("data:"):
        source = base64.b64decode(source.split(",", 1)[1])
    img = Image.open(io.BytesIO(source) if isinstance(source, (bytes, bytearray)) else source).convert("RGB")
    return torch.from_numpy(np.asarray(img).copy())


def fit_box(src_w: int, src_h: int, dst_w: int, dst_h: int) -> tuple[int, int, int, int]:
    """Aspect-preserving placement of the source inside the destination: (x0, y0, w, h), centred."""
    s = min(dst_w / src_w, dst_h / src_h)
    w, h = max(1, min(dst_w, round(src_w * s))), max(1, min(dst_h, round(src_h * s)))
    return (dst_w - w) // 2, (dst_h - h) // 2, w, h


def prepare_reference(img: torch.Tensor, plan: ImagePlan, patch: int = 14) -> torch.Tensor:
    """CPU twin: uint8 [H, W, 3] -> bf16 patches [n_vit_h * n_vit_w, 3 * patch * patch] (row-major patch order,
    channel-major inside a patch).  Bilinear sampling with half-pixel centres, clamped at the border."""
    H, W, _ = img.shape
    x0, y0, w, h = fit_box(W, H, plan.width, plan.height)
    src = img.float()
    ys = ((torch.arange(h, dtype=torch.float32) + 0.5) * (H / h) - 0.5).clamp(0, H - 1)
    xs = ((torch.arange(w, dtype=torch.float32) + 0.5) * (W / w) - 0.5).clamp(0, W - 1)
    yi, xi = ys.floor().long(), xs.floor().long()
    yf, xf = (ys - yi).reshape(h, 1, 1), (xs - xi).reshape(1, w, 1)
    yj, xj = (yi + 1).clamp(max=H - 1), (xi + 1).clamp(max=W - 1)
    top = src[yi][:, xi] * (1 - xf) + src[yi][:, xj] * xf
    bot = src[yj][:, xi] * (1 - xf) + src[yj][:, xj] * xf
    body = top * (1 - yf) + bot * yf
    canvas = torch.full((plan.height, plan.width, 3), float(GREY))
    canvas[y0:y0 + h, x0:x0 + w] = body
    norm = ((canvas / 255.0 - 0.5) / 0.5).to(torch.bfloat16)
    p = norm.permute(2, 0, 1).reshape(3, plan.n_vit_h, patch, plan.n_vit_w, patch)
    return p.permute(1, 3, 0, 2, 4).reshape(plan.n_vit_h * plan.n_vit_w, 3 * patch * patch).contiguous()


def prepare(img: torch.Tensor, plan: ImagePlan, patch: int = 14) -> torch.Tensor:
    """Device path: ``img`` uint8 [H, W, 3] on the GPU -> bf16 patches on the GPU."""
    from .. import _lib
    from ..ops import native as N
    H, W, _ = img.shape
    x0, y0, w, h = fit_box(W, H, plan.width, plan.height)
    out = torch.empty((plan.n_vit_h * plan.n_vit_w, 3 * patch * patch), dtype=torch.bfloat16, device=img.device)
    rc = _lib.cuda().sfb_vision_prepare(N._p(img.contiguous()), c_int(W), c_int(H), c_int(x0), c_int(y0), c_int(w), c_int(h),
                                        c_int(plan.width), c_int(plan.height), c_int(patch), c_int(GREY), N._p(out), N._stream())
    N._check(rc, "vision_prepare")
    return out
