"""Codec golden tables: the torch codecs, the C++ scalar codecs and hand-written values agree
(reference: crates/sparkflash-kernels/tests/m4_codec_golden.rs)."""
import ctypes

import numpy as np
import torch

from sparkflash_b200 import _lib, codecs as C


def test_e4m3_all_codes_roundtrip():
    L = _lib.host()
    for c in range(256):
        f = L.sfb_e4m3_to_f32(c)
        if c & 0x7f == 0x7f:
            assert f != f
            continue
        assert L.sfb_f32_to_e4m3(f) == c or (f == 0.0 and c in (0, 0x80))
        t = C.e4m3_decode(torch.tensor([c], dtype=torch.uint8))
        assert float(t) == f


def test_e4m3_goldens():
    L = _lib.host()
    table = {0.0: 0x00, 1.0: 0x38, -1.0: 0xb8, 448.0: 0x7e, 1000.0: 0x7e, -1000.0: 0xfe, 2 ** -9: 0x01,
             2 ** -6: 0x08, 0.5: 0x30, 1.0625: 0x38, 1.1875: 0x3a, 1.125: 0x39, 464.0: 0x7e, 2 ** -10: 0x00,
             1.5 * 2 ** -10: 0x01, 3 * 2 ** -10: 0x02}
    for f, code in table.items():
        assert L.sfb_f32_to_e4m3(f) == code, (f, hex(L.sfb_f32_to_e4m3(f)), hex(code))


def test_e4m3_encode_matches_torch_on_random():
    L = _lib.host()
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(4000, generator=g) * s for s in (1e-3, 0.1, 1, 30, 300)])
    ref = C.e4m3_encode(x)
    got = torch.tensor([L.sfb_f32_to_e4m3(float(v)) for v in x], dtype=torch.uint8)
    assert torch.equal(ref, got)


def test_e2m1_codes_and_ties():
    L = _lib.host()
    vals = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i, v in enumerate(vals):
        assert L.sfb_e2m1_to_f32(i) == v and L.sfb_e2m1_to_f32(i | 8) == -v
        assert L.sfb_f32_to_e2m1(v) == i
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6, 100.0: 7, -0.3: 9}
    for f, code in ties.items():
        assert L.sfb_f32_to_e2m1(f) == code, f
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5000, generator=g) * 3
    ref = C.e2m1_encode(x)
    got = torch.tensor([L.sfb_f32_to_e2m1(float(v)) for v in x], dtype=torch.uint8)
    assert torch.equal(ref, got)


def test_ue8m0_ceil_rule():
    L = _lib.host()
    assert L.sfb_ue8m0_ceil(1.0) == 127 and L.sfb_ue8m0_ceil(1.0001) == 128 and L.sfb_ue8m0_ceil(0.5) == 126
    assert L.sfb_act_scale_code_fp8(448.0) == 127 and L.sfb_act_scale_code_fp8(449.0) == 128
    assert L.sfb_act_scale_code_fp8(0.0) == L.sfb_act_scale_code_fp8(1e-4)  # the amax floor
    x = torch.rand(3000, generator=torch.Generator().manual_seed(2)) * 100 + 1e-6
    ref = C.ue8m0_ceil_code(x)
    got = torch.tensor([L.sfb_ue8m0_ceil(float(v)) for v in x], dtype=torch.uint8)
    assert torch.equal(ref, got)


def _np(t):
    return t.contiguous().numpy()


def test_bulk_act_quant_matches_torch():
    L = _lib.host()
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(7, 96, generator=g) * torch.tensor([1e-5, 0.01, 1.0, 5.0, 80.0, 1000.0, 0.3]).unsqueeze(1)).contiguous()
    x[0, :32] = 0
    q = np.zeros((7, 96), np.uint8); s = np.zeros((7, 3), np.uint8)
    L.sfb_act_quant_fp8(_np(x).ctypes.data, 7, 96, q.ctypes.data, s.ctypes.data)
    rq, rs = C.act_quant_fp8(x)
    assert np.array_equal(q, _np(rq)) and np.array_equal(s, _np(rs))
    # fp4 (indexer) and kv fp4
    q4 = np.zeros((7, 48), np.uint8); s4 = np.zeros((7, 3), np.uint8)
    L.sfb_act_quant_fp4(_np(x).ctypes.data, 7, 96, q4.ctypes.data, s4.ctypes.data)
    rq4, rs4 = C.act_quant_fp4(x)
    assert np.array_equal(q4, _np(C.pack_nibbles(rq4))) and np.array_equal(s4, _np(rs4))
    qk = np.zeros((7, 48), np.uint8); sk = np.zeros((7, 6), np.uint8)
    L.sfb_kv_quant_fp4(_np(x).ctypes.data, 7, 96, qk.ctypes.data, sk.ctypes.data)
    rqk, rsk = C.kv_quant_fp4(x)
    assert np.array_equal(qk, _np(C.pack_nibbles(rqk))) and np.array_equal(sk, _np(rsk))
    back = np.zeros((7, 96), np.float32)
    L.sfb_kv_dequant_fp4(qk.ctypes.data, sk.ctypes.data, 7, 96, back.ctypes.data)
    assert np.array_equal(back, _np(C.kv_dequant_fp4(rqk, rsk)))


def test_weight_quant_and_prepared_scales():
    L = _lib.host()
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(70, 64, generator=g) * 0.02).contiguous()
    q = np.zeros((70, 64), np.uint8); s = np.zeros((3, 2), np.uint8)
    L.sfb_weight_quant_fp8_block32(_np(w).ctypes.data, 70, 64, q.ctypes.data, s.ctypes.data)
    rq, rs = C.weight_quant_fp8_block32(w)
    assert np.array_equal(q, _np(rq)) and np.array_equal(s, _np(rs))
    deq = C.weight_dequant_fp8_block32(rq, rs)
    assert (deq - w).abs().max() < w.abs().max() / 14
    q4 = np.zeros((70, 32), np.uint8); s4 = np.zeros((70, 2), np.uint8)
    L.sfb_weight_quant_fp4_row32(_np(w).ctypes.data, 70, 64, q4.ctypes.data, s4.ctypes.data)
    rq4, rs4 = C.weight_quant_fp4_row32(w)
    assert np.array_equal(q4, _np(rq4)) and np.array_equal(s4, _np(rs4))
    # prepared layout: C++ and torch agree and invert
    prep = C.scales_to_prepared(rs, 70, 32)
    buf = np.full(C.sf_bytes(70, 2), 127, np.uint8)
    L.sfb_scales_to_prepared(_np(rs).ctypes.data, 70, 2, 32, buf.ctypes.data)
    assert np.array_equal(buf, _np(prep))
    assert torch.equal(C.prepared_to_scales(prep, 70, 2), rs.repeat_interleave(32, 0)[:70])
    assert L.sfb_sf_offset(130, 5, 6) == int(C.sf_offsets(131, 6)[130, 5])


def test_sf_atom_layout_is_a_bijection():
    off = C.sf_offsets(256, 8).flatten()
    assert off.unique().numel() == off.numel() and int(off.max()) < C.sf_bytes(256, 8)


def test_mla_v3_cached_engine_matches_the_fp32_oracle():
    from sparkflash_b200.models import mla_v3
    r = mla_v3.run(n_new=6, prompt_len=12)
    assert r["max_abs_logit_err_vs_fp32_oracle"] < 1e-4 and r["argmax_agree"] == "6/6"
