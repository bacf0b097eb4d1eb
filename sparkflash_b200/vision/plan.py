"""Image planning: the pixel size an image is resized to, its ViT patch grid, its token grid after the 3x3
aligner, and the span of token types it occupies in the prompt.

Reference: crates/sparkflash-vision/src/{plan,span}.rs; docs/architecture/06-vision.md sections 2 and 5
(upscale below min_pixels, round each axis UP to the patch size, shrink only when the token budget
n_h * (n_w + 1) + 2 is exceeded, one newline token per row, start and end tokens around the span).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

TEXT, IMAGE_START, IMAGE, IMAGE_NEW_LINE, IMAGE_END = -1, 0, 1, 2, 3


@dataclass(frozen=True)
class VisionConfig:
    n_layers: int = 32
    dim: int = 1024
    n_heads: int = 16
    inter_dim: int = 2816
    patch_size: int = 14
    downsample_ratio: int = 3
    max_n_token: int = 1024
    min_pixels: int = 295936
    max_wh_ratio: float | None = None
    rope_theta: float = 10000.0
    llm_dim: int = 5120
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class ImagePlan:
    width: int          # pixels after resize/pad
    height: int
    n_vit_w: int        # patch grid
    n_vit_h: int
    n_llm_w: int        # token grid after the aligner
    n_llm_h: int

    @property
    def n_tokens(self) -> int:
        return num_image_tokens(self.n_llm_h, self.n_llm_w)


def num_image_tokens(n_h: int, n_w: int) -> int:
    return n_h * (n_w + 1) + 2


def _grid(width: int, height: int, c: VisionConfig) -> tuple[int, int, int, int]:
    nvw, nvh = math.ceil(width / c.patch_size), math.ceil(height / c.patch_size)
    return nvw, nvh, math.ceil(nvw / c.downsample_ratio), math.ceil(nvh / c.downsample_ratio)


def _solve_resize(width: int, height: int, c: VisionConfig) -> tuple[int, int]:
    """Largest aspect-preserving size whose token grid fits the budget (closed form, then a guard loop)."""
    cell = c.patch_size * c.downsample_ratio
    r = height / width
    max_w = math.sqrt((c.max_n_token - 2) / r + 0.25) - 0.5          # n_w with n_h = r * n_w solves n_h (n_w + 1) = budget - 2
    n_w = max(1, int(math.floor(max_w)))
    n_h = max(1, int(math.floor(r * n_w)))
    if n_w == 1:
        n_h = min(n_h, (c.max_n_token - 2) // 2)
    if n_h == 1:
        n_w = min(n_w, c.max_n_token - 3)
    while num_image_tokens(n_h, n_w) > c.max_n_token:
        if n_w >= n_h and n_w > 1:
            n_w -= 1
        elif n_h > 1:
            n_h -= 1
        else:
            break
    return n_w * cell, n_h * cell


def plan_image_grid(width: int, height: int, c: VisionConfig = VisionConfig()) -> ImagePlan:
    if width <= 0 or height <= 0:
        raise ValueError("image has no pixels")
    w, h = float(width), float(height)
    if c.max_wh_ratio is not None and w > h * c.max_wh_ratio:
        w = h * c.max_wh_ratio
    if 0 < w * h < c.min_pixels:
        s = math.sqrt(c.min_pixels / (w * h))
        w, h = w * s, h * s
    pw = int(math.ceil(w / c.patch_size)) * c.patch_size
    ph = int(math.ceil(h / c.patch_size)) * c.patch_size
    nvw, nvh, nlw, nlh = _grid(pw, ph, c)
    if num_image_tokens(nlh, nlw) > c.max_n_token:
        pw, ph = _solve_resize(pw, ph, c)
        nvw, nvh, nlw, nlh = _grid(pw, ph, c)
    return ImagePlan(pw, ph, nvw, nvh, nlw, nlh)


def span_types(plan: ImagePlan) -> list[int]:
    return [IMAGE_START] + ([IMAGE] * plan.n_llm_w + [IMAGE_NEW_LINE]) * plan.n_llm_h + [IMAGE_END]


def expand_prompt(tokens: list[int], image_token_id: int, plans: list[ImagePlan]) -> tuple[list[int], list[int], list[int]]:
    """Replace each placeholder by its span.  -> (tokens, token_types, span starts).  Every position of a span
    carries the placeholder id; the layout lives in the types."""
    n = sum(1 for t in tokens if t == image_token_id)
    if n != len(plans):
        raise ValueError(f"{n} image placeholder(s) in the prompt but {len(plans)} image(s) supplied")
    out, types, starts, k = [], [], [], 0
    for t in tokens:
        if t == image_token_id:
            sp = span_types(plans[k]); k += 1
            starts.append(len(out))
            out += [image_token_id] * len(sp)
            types += sp
        else:
            out.append(t); types.append(TEXT)
    return out, types, starts
