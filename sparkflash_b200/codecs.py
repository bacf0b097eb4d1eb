"""Vectorised (torch) twins of the bit rules in ``csrc/codecs.h``.

They run on CPU or GPU tensors and are what the oracle, the synthetic-weight generator and the
converter use; ``tests/test_codecs.py`` pins them against the C++ scalar codecs code by code.
Reference behaviour: crates/sparkflash-weights/src/quant*, kernels/m4_activation_quant_sm121.cuh,
docs/architecture/01-csa2-attention.md section 8.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
E2M1_MAX = 6.0
_E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


# ---- UE8M0 -----------------------------------------------------------------------------------------
def ue8m0_ceil_code(x: torch.Tensor) -> torch.Tensor:
    """Code of the smallest power of two >= x (x > 0)."""
    m, e = torch.frexp(x.to(torch.float32))  # x = m * 2^e, m in [0.5, 1)
    exp = torch.where(m > 0.5, e, e - 1)
    return (exp + 127).clamp(0, 254).to(torch.uint8)


def ue8m0_decode(code: torch.Tensor) -> torch.Tensor:
    c = code.to(torch.int32)
    bits = torch.where(c > 0, c << 23, torch.full_like(c, 0x00400000))
    return bits.view(torch.float32)


# ---- E4M3 ------------------------------------------------------------------------------------------
def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float32).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(code: torch.Tensor) -> torch.Tensor:
    return code.view(torch.float8_e4m3fn).to(torch.float32)


# ---- E2M1 ------------------------------------------------------------------------------------------
def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    x = x.to(torch.float32)
    a = x.abs()
    c = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
         + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
         + (a > 5.0).to(torch.uint8))
    sign = (torch.signbit(x)).to(torch.uint8) << 3
    return c | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    tab = torch.tensor(_E2M1_VALUES + [-v for v in _E2M1_VALUES], dtype=torch.float32, device=code.device)
    return tab[code.to(torch.int64) & 15]


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., k] codes (0..15) -> [..., k/2] bytes, even element in the low nibble."""
    lo, hi = codes[..., 0::2], codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_nibbles(b: torch.Tensor) -> torch.Tensor:
    out = torch.stack([b & 15, b >> 4], dim=-1)
    return out.flatten(-2)


# ---- activation quantisers -------------------------------------------------------------------------
def act_quant_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-32 FP8: returns (codes [..., k] uint8, scale codes [..., k/32] uint8)."""
    x = x.to(torch.float32)
    g = x.unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1).clamp_min(1.0e-4)
    sc = ue8m0_ceil_code(amax * (1.0 / 448.0))
    q = e4m3_encode(g / ue8m0_decode(sc).unsqueeze(-1))
    return q.flatten(-2), sc


def act_dequant_fp8(q: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    return (e4m3_decode(q).unflatten(-1, (-1, 32)) * ue8m0_decode(sc).unsqueeze(-1)).flatten(-2)


def act_roundtrip_fp8(x: torch.Tensor) -> torch.Tensor:
    return act_dequant_fp8(*act_quant_fp8(x))


def act_quant_fp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """MXFP4 (indexer): per-32 UE8M0 ceil scale; returns (unpacked codes, scale codes)."""
    x = x.to(torch.float32)
    g = x.unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1).clamp_min(7.052966e-38)
    sc = ue8m0_ceil_code(amax * (1.0 / 6.0))
    q = e2m1_encode(g / ue8m0_decode(sc).unsqueeze(-1))
    return q.flatten(-2), sc


def act_roundtrip_fp4(x: torch.Tensor) -> torch.Tensor:
    q, sc = act_quant_fp4(x)
    return (e2m1_decode(q).unflatten(-1, (-1, 32)) * ue8m0_decode(sc).unsqueeze(-1)).flatten(-2)


def kv_quant_fp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """NVFP4-style KV: group 16, E4M3 scale = e4m3(max(amax, 6*2^-9)/6)."""
    x = x.to(torch.float32)
    g = x.unflatten(-1, (-1, 16))
    amax = g.abs().amax(-1).clamp_min(6.0 * 2.0 ** -9)
    sc = e4m3_encode(amax / 6.0)
    q = e2m1_encode(g / e4m3_decode(sc).unsqueeze(-1))
    return q.flatten(-2), sc


def kv_dequant_fp4(q: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    return (e2m1_decode(q).unflatten(-1, (-1, 16)) * e4m3_decode(sc).unsqueeze(-1)).flatten(-2)


def kv_roundtrip_fp4(x: torch.Tensor) -> torch.Tensor:
    return kv_dequant_fp4(*kv_quant_fp4(x))


# ---- weight quantisers (checkpoint grid: scale = 2^(floor(log2 amax) - emax)) -----------------------
def _weight_scale_code(amax: torch.Tensor, emax: int) -> torch.Tensor:
    m, e = torch.frexp(amax.to(torch.float32))  # amax = m*2^e, floor(log2) = e-1
    code = (e - 1 - emax + 127).clamp(0, 254)
    return torch.where(amax > 0, code, torch.full_like(code, 107)).to(torch.uint8)


def weight_quant_fp8_block32(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [out, in] -> (codes [out, in], scales [ceil(out/32), in/32]) with 32x32 blocks."""
    out, inn = w.shape
    po = (32 - out % 32) % 32
    wp = torch.nn.functional.pad(w.to(torch.float32), (0, 0, 0, po))
    blk = wp.view((out + po) // 32, 32, inn // 32, 32)
    amax = blk.abs().amax(dim=(1, 3))
    sc = _weight_scale_code(amax, 8)
    q = e4m3_encode(blk / ue8m0_decode(sc)[:, None, :, None]).view(out + po, inn)[:out]
    return q.contiguous(), sc


def weight_dequant_fp8_block32(q: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    out, inn = q.shape
    s = ue8m0_decode(sc).repeat_interleave(32, 0)[:out].repeat_interleave(32, 1)
    return e4m3_decode(q) * s


def weight_quant_fp4_row32(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [out, in] -> (packed [out, in/2], scales [out, in/32])."""
    g = w.to(torch.float32).unflatten(-1, (-1, 32))
    sc = _weight_scale_code(g.abs().amax(-1), 2)
    q = e2m1_encode(g / ue8m0_decode(sc).unsqueeze(-1)).flatten(-2)
    return pack_nibbles(q), sc


def weight_dequant_fp4_row32(packed: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    q = unpack_nibbles(packed)
    return (e2m1_decode(q).unflatten(-1, (-1, 32)) * ue8m0_decode(sc).unsqueeze(-1)).flatten(-2)


# ---- prepared scale layout ---------------------------------------------------------------------------
def sf_bytes(rows: int, kblocks: int) -> int:
    return ((rows + 127) // 128) * ((kblocks + 3) // 4) * 512


def sf_offsets(rows: int, kblocks: int, device=None) -> torch.Tensor:
    r = torch.arange(rows, device=device).unsqueeze(1)
    kb = torch.arange(kblocks, device=device).unsqueeze(0)
    katoms = (kblocks + 3) // 4
    atom = (r // 128) * katoms + kb // 4
    rr = r % 128
    return atom * 512 + (rr % 32) * 16 + (rr // 32) * 4 + kb % 4


def scales_to_prepared(sc: torch.Tensor, rows: int, block_rows: int) -> torch.Tensor:
    """Checkpoint scales ([ceil(rows/block_rows), kb]) -> per-row swizzled bytes (see csrc/codecs.h)."""
    kb = sc.shape[1]
    per_row = sc.repeat_interleave(block_rows, 0)[:rows] if block_rows > 1 else sc
    out = torch.full((sf_bytes(rows, kb),), 127, dtype=torch.uint8, device=sc.device)
    out[sf_offsets(rows, kb, sc.device).flatten()] = per_row.flatten()
    return out


def prepared_to_scales(buf: torch.Tensor, rows: int, kblocks: int) -> torch.Tensor:
    return buf[sf_offsets(rows, kblocks, buf.device)]
