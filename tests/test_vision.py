"""Vision planning, preparation, tower pieces (reference: crates/sparkflash-vision/tests/goldens.rs;
docs/architecture/06-vision.md)."""
import io

import pytest
import torch

from sparkflash_b200.vision import plan as VP, prep, tower as VT

C = VP.VisionConfig()


def test_plan_rules():
    p = VP.plan_image_grid(100, 80, C)                # below min_pixels: upscaled, then rounded up to 14
    assert p.width % 14 == 0 and p.height % 14 == 0 and p.width * p.height >= C.min_pixels
    assert (p.n_vit_w, p.n_vit_h) == (p.width // 14, p.height // 14)
    assert p.n_llm_w == -(-p.n_vit_w // 3) and p.n_tokens == p.n_llm_h * (p.n_llm_w + 1) + 2 <= C.max_n_token
    p = VP.plan_image_grid(700, 700, C)
    assert (p.width, p.height) == (700, 700) and (p.n_llm_w, p.n_llm_h) == (17, 17) and p.n_tokens == 17 * 18 + 2
    for w, h in [(4000, 3000), (10000, 200), (200, 10000), (1920, 1080), (50, 5000)]:
        p = VP.plan_image_grid(w, h, C)
        assert p.n_tokens <= C.max_n_token and p.width % 14 == 0 and p.height % 14 == 0, (w, h, p)
    big = VP.plan_image_grid(4000, 3000, C)
    assert big.n_tokens > 0.8 * C.max_n_token and abs(big.width / big.height - 4 / 3) < 0.15
    with pytest.raises(ValueError):
        VP.plan_image_grid(0, 10, C)


def test_span_protocol():
    p = VP.ImagePlan(84, 42, 6, 3, 2, 1)
    assert VP.span_types(p) == [VP.IMAGE_START, VP.IMAGE, VP.IMAGE, VP.IMAGE_NEW_LINE, VP.IMAGE_END]
    toks, types, starts = VP.expand_prompt([5, 900, 6, 900], 900, [p, p])
    assert toks == [5] + [900] * 5 + [6] + [900] * 5 and starts == [1, 7]
    assert types[0] == VP.TEXT and types[1:6] == VP.span_types(p) and len(types) == len(toks)
    with pytest.raises(ValueError):
        VP.expand_prompt([5, 900], 900, [])


def test_prepare_reference_letterboxes_normalises_and_orders_patches():
    from PIL import Image
    img = torch.zeros(40, 80, 3, dtype=torch.uint8)
    img[..., 0] = 255                                 # pure red
    buf = io.BytesIO(); Image.fromarray(img.numpy()).save(buf, format="PNG")
    dec = prep.decode_image(buf.getvalue())
    assert torch.equal(dec, img)
    p = VP.ImagePlan(56, 56, 4, 4, 2, 2)
    out = prep.prepare_reference(dec, p)
    assert out.shape == (16, 588) and out.dtype == torch.bfloat16
    x0, y0, w, h = prep.fit_box(80, 40, 56, 56)
    assert (x0, y0, w, h) == (0, 14, 56, 28)
    patch0 = out[0].float().reshape(3, 14, 14)        # top row of patches is padding: mid grey
    assert torch.allclose(patch0, torch.full_like(patch0, (127 / 255 - 0.5) / 0.5), atol=1e-2)
    mid = out[4].float().reshape(3, 14, 14)           # second row: red
    assert torch.all(mid[0] == 1.0) and torch.all(mid[1] == -1.0)


def test_tower_pieces_and_tiny_forward():
    x = (torch.randn(12, 2, 8) * 2).to(torch.bfloat16)
    r = VT.rope_reference(x, 4, 10000.0)
    assert torch.equal(r[0], x[0])                    # position (0, 0) is not rotated
    assert torch.allclose(r.float().pow(2).sum(-1), x.float().pow(2).sum(-1), rtol=0.05)
    g = torch.arange(4 * 5 * 2, dtype=torch.float32).reshape(20, 2).to(torch.bfloat16)
    u = VT.unfold3_reference(g, 4, 5)
    assert u.shape == (2 * 2, 18)
    # element c*9 + kh*3 + kw of cell (0,0) is x[kh, kw, c]
    assert u[0, 1 * 9 + 2 * 3 + 1] == g.reshape(4, 5, 2)[2, 1, 1] and u[3, 0 * 9 + 1 * 3 + 2] == 0    # padded
    c = VP.VisionConfig(n_layers=2, dim=64, n_heads=4, inter_dim=96, llm_dim=48)
    tw = VT.VisionTower(c, VT.synthetic_vision_weights(c))
    p = VP.ImagePlan(84, 42, 6, 3, 2, 1)
    patches = (torch.randn(18, 588) * 0.5).to(torch.bfloat16)
    emb = tw.encode(patches, p)
    assert emb.shape == (2, 48) and torch.isfinite(emb.float()).all()
    span = tw.span_embeddings(emb, p)
    assert span.shape == (p.n_tokens, 48) and torch.equal(span[0], tw.w["image_start"]) and torch.equal(span[3], tw.w["image_newline"])


@pytest.mark.gpu
def test_device_kernels_match_their_twins():
    g = torch.Generator().manual_seed(0)
    img = torch.randint(0, 256, (123, 77, 3), generator=g, dtype=torch.uint8)
    p = VP.plan_image_grid(77, 123, C)
    a = prep.prepare(img.cuda(), p).float().cpu()
    b = prep.prepare_reference(img, p).float()
    assert a.shape == b.shape and (a - b).abs().max() <= 2 ** -6         # one bf16 step of bilinear rounding slack
    x = (torch.randn(35, 4, 64, generator=g)).to(torch.bfloat16)
    assert (VT._rope(x.cuda(), 7, 10000.0).float().cpu() - VT.rope_reference(x, 7, 10000.0).float()).abs().max() <= 2 ** -5
    y = torch.randn(5 * 7, 32, generator=g).to(torch.bfloat16)
    assert torch.equal(VT._unfold3(y.cuda(), 5, 7).cpu(), VT.unfold3_reference(y, 5, 7))
    c = VP.VisionConfig(n_layers=2, dim=128, n_heads=4, inter_dim=192, llm_dim=64)
    w = VT.synthetic_vision_weights(c)
    pl = VP.ImagePlan(84, 84, 6, 6, 2, 2)
    patches = (torch.randn(36, 588, generator=g) * 0.5).to(torch.bfloat16)
    cpu = VT.VisionTower(c, w).encode(patches, pl).float()
    tower = VT.VisionTower(c, {k: v.cuda() for k, v in w.items()})
    gpu = tower.encode(patches.cuda(), pl).float().cpu()
    assert (cpu - gpu).abs().max() < 0.05 * cpu.abs().max() + 1e-3
    assert tower.tc_gemms >= 4 * c.n_layers          # the blocks' projections ran on the tensor-core GEMM
