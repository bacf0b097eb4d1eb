"""Images in requests: decode, plan, run the tower, expand the prompt's placeholders into spans and hand the
span embeddings to the engine row by row.  The tower runs on the rank that owns the HTTP surface; every rank
receives the finished embeddings with the request (reference: DECISIONS D59, crates/sparkflash-api/src/{multimodal,
vision}.rs, docs/architecture/06-vision.md section 5).  Remote URLs are refused: a server does not fetch."""
from __future__ import annotations

import base64
from dataclasses import dataclass

import torch

from ..vision import plan as VP, prep
from ..vision.tower import VisionTower
from .engine_api import ApiError


@dataclass
class VisionSpan:
    start: int                 # first position of the span in the expanded prompt
    embeddings: torch.Tensor   # [n_tokens, llm_dim] bf16 on the CPU: start, rows + newlines, end


def image_bytes(part: dict) -> bytes:
    """OpenAI ``image_url`` / Responses ``input_image`` / Anthropic ``image`` part -> encoded image bytes."""
    t = part.get("type")
    url = None
    if t == "image_url":
        u = part.get("image_url")
        url = u.get("url") if isinstance(u, dict) else u
    elif t == "input_image":
        url = part.get("image_url")
    elif t == "image":
        src = part.get("source") or {}
        if src.get("type") == "base64":
            return base64.b64decode(src.get("data", ""))
        url = src.get("url")
    if not url:
        raise ApiError(400, "image part carries no image", param="messages")
    if not url.startswith("data:"):
        raise ApiError(400, "only inline images (data: URLs or base64 sources) are accepted", "unsupported_image_source", "messages")
    try:
        return base64.b64decode(url.split(",", 1)[1])
    except Exception:
        raise ApiError(400, "image data is not valid base64", param="messages") from None


class VisionFrontEnd:
    def __init__(self, tower: VisionTower, image_token_id: int, device: str = "cpu"):
        self.tower, self.cfg, self.image_token_id, self.device = tower, tower.c, image_token_id, device

    def encode(self, parts: list[dict]) -> list[tuple[VP.ImagePlan, torch.Tensor]]:
        out = []
        for p in parts:
            try:
                img = prep.decode_image(image_bytes(p))
            except ApiError:
                raise
            except Exception as e:
                raise ApiError(400, f"image could not be decoded: {e}", "invalid_image", "messages") from None
            pl = VP.plan_image_grid(img.shape[1], img.shape[0], self.cfg)
            if self.device == "cpu":
                patches = prep.prepare_reference(img, pl, self.cfg.patch_size)
            else:
                patches = prep.prepare(img.to(self.device), pl, self.cfg.patch_size)
            emb = self.tower.encode(patches, pl)
            out.append((pl, self.tower.span_embeddings(emb, pl).to("cpu")))
        return out

    def expand(self, tokens: list[int], parts: list[dict]) -> tuple[list[int], list[VisionSpan]]:
        enc = self.encode(parts)
        try:
            new, _types, starts = VP.expand_prompt(tokens, self.image_token_id, [pl for pl, _ in enc])
        except ValueError as e:
            raise ApiError(400, str(e), param="messages") from None
        return new, [VisionSpan(s, e) for s, (_, e) in zip(starts, enc)]
