"""The allocation-free GEMM entry point, called through its exported C symbol.

Some users of the library may not allocate device memory at all: a server that gave the whole GPU to
its KV-cache pool at start-up, a decode thread that cannot afford the device-wide synchronisation
cudaMalloc implies, a plugin whose host owns every allocation.  For them the split-K scratch lives
inside the library.  This test calls the exported symbol directly (ctypes, no Python wrapper), twice
in a row so that the second call sees the first call's leftovers, and compares each result with the
ordinary entry point that takes caller-provided scratch.  It is collected last on purpose.
"""
import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

from sparkflash_b200 import codecs as C

pytestmark = pytest.mark.gpu


def _operands(rows, K, n, seed, groups=1):
    """Weights [rows, K] and activations [n, groups * K], both quantised, with their scale atoms."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, K, generator=g) * 0.05
    x = torch.randn(n, groups * K, generator=g)
    q, s = C.weight_quant_fp8_block32(w)
    xq, xs = C.act_quant_fp8(x)
    return q, C.scales_to_prepared(s, rows, 32), xq, C.scales_to_prepared(xs, n, 1)


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    from sparkflash_b200 import _lib
    from sparkflash_b200.ops import native as N
    L = _lib.cuda()
    fn = L.sfb_umma_dense_noalloc
    fn.restype = c_int
    L.sfb_noalloc_last_error.restype = ctypes.c_char_p
    dev = "cuda"
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # (columns per group, K, rows, splits, groups): few rows (the last CTA of a tile adds the splits), 17+ rows (the
    # partial sums stay in the built-in array for the separate reduce grid), two groups, and a single split
    cases = [(256, 1024, 7, 4, 1), (384, 512, 3, 2, 1), (256, 1024, 20, 4, 1), (128, 512, 40, 2, 2), (256, 512, 5, 1, 1)]
    for call, (N_, K, n, splits, groups) in enumerate(cases):
        q, sfa, xq, sfb = _operands(groups * N_, K, n, seed=100 + call, groups=groups)
        NP = N.umma_np(n)
        qd = q.to(dev).contiguous()
        xpad = torch.zeros(NP, groups * K, dtype=torch.uint8, device=dev)
        xpad[:n] = xq.to(dev)
        sfa_d, sfb_d = sfa.to(dev), sfb.to(dev)
        ta = N.TensorMap(qd, groups * N_, K, K, 128)
        tb = N.TensorMap(xpad, NP, groups * K, groups * K, NP)
        tiles = groups * (N_ // 128)
        # ordinary entry point, caller-provided scratch
        ref = torch.zeros(n, groups * N_, dtype=torch.float32, device=dev)
        scratch = torch.zeros(tiles * splits * 128 * NP, dtype=torch.float32, device=dev)
        tickets = torch.zeros(tiles, dtype=torch.int32, device=dev)
        N.umma_dense(ta, tb, sfa_d, sfb_d, n, N_, K, groups=groups, splits=splits, scratch=scratch, tickets=tickets, out_f=ref)
        # allocation-free entry point through the exported symbol
        out = torch.full((n, groups * N_), float("nan"), dtype=torch.float32, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        rc = fn(c_void_p(ta.ptr), c_void_p(tb.ptr), c_void_p(sfa_d.data_ptr()), c_int(K // 128),
                c_void_p(sfb_d.data_ptr()), c_int(groups * K // 128), c_int(n), c_int(NP), c_int(N_), c_int(K), c_int(groups),
                c_int(0), c_int(splits), None, c_void_p(out.data_ptr()), c_int64(groups * N_), c_void_p(status.data_ptr()),
                stream)
        assert rc == 0, (rc, L.sfb_noalloc_last_error())
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        # same kernel, same split order: the two entry points agree bit for bit
        assert torch.equal(out, ref), (call, (out - ref).abs().max().item())
    # a problem beyond the built-in scratch is refused with a message and launches nothing
    rc = fn(c_void_p(ta.ptr), c_void_p(tb.ptr), c_void_p(sfa_d.data_ptr()), c_int(K // 128),
            c_void_p(sfb_d.data_ptr()), c_int(K // 128), c_int(n), c_int(128), c_int(128 * 4000), c_int(K), c_int(2),
            c_int(0), c_int(2), None, c_void_p(out.data_ptr()), c_int64(N_), c_void_p(status.data_ptr()), stream)
    assert rc == -2 and b"built-in scratch" in L.sfb_noalloc_last_error()
