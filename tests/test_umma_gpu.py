"""tcgen05 block-scaled GEMM against a plain fp32 reference (same quantised operands)."""
import pytest
import torch

from sparkflash_b200 import codecs as C

pytestmark = pytest.mark.gpu


def _case(N_, K, n, fp4, groups=1, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(groups * N_, K, generator=g) * 0.05
    x = torch.randn(n, groups * K, generator=g)
    if fp4:
        q, s = C.weight_quant_fp4_row32(w)
        wd = C.weight_dequant_fp4_row32(q, s)
        sfa = C.scales_to_prepared(s, groups * N_, 1)
    else:
        q, s = C.weight_quant_fp8_block32(w)
        wd = C.weight_dequant_fp8_block32(q, s)
        sfa = C.scales_to_prepared(s, groups * N_, 32)
    xq, xs = C.act_quant_fp8(x)
    xd = C.act_dequant_fp8(xq, xs)
    ref = torch.cat([xd[:, gi * K:(gi + 1) * K] @ wd[gi * N_:(gi + 1) * N_].t() for gi in range(groups)], 1)
    sfb = C.scales_to_prepared(xs, n, 1)
    return q, sfa, xq, sfb, ref


@pytest.mark.parametrize("N_,K,n,fp4,splits,groups", [
    (128, 128, 1, False, 1, 1), (256, 512, 5, False, 1, 1), (256, 512, 16, False, 2, 1), (384, 1024, 3, False, 4, 1),
    (128, 256, 2, True, 1, 1), (256, 512, 9, True, 2, 1), (128, 256, 4, False, 1, 2), (256, 1280, 33, False, 1, 1),
    # production shapes: wo_b / expert down column count with 7-way split-K, wqkv_a with 21-way split-K, wq_b without a split,
    # many rows with the separate split-K reduce grid, a grouped matrix with eight groups
    (5120, 8192, 1, False, 7, 1), (1792, 5120, 1, False, 21, 1), (4096, 1280, 3, False, 1, 1), (5120, 5120, 40, False, 7, 1),
    (1024, 4096, 6, False, 4, 8), (2304, 5120, 16, True, 2, 1)])
def test_umma_dense_matches_reference(N_, K, n, fp4, splits, groups):
    from sparkflash_b200.ops import native as N
    q, sfa, xq, sfb, ref = _case(N_, K, n, fp4, groups, seed=N_ + K + n)
    dev = "cuda"
    NP = N.umma_np(n)
    qd = q.to(dev).contiguous()
    xpad = torch.zeros(NP, groups * K, dtype=torch.uint8, device=dev)
    xpad[:n] = xq.to(dev)
    ta = N.TensorMap(qd, groups * N_, K, K // 2 if fp4 else K, 128, fp4=fp4)
    tb = N.TensorMap(xpad, NP, groups * K, groups * K, NP)
    out = torch.full((n, groups * N_), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    tiles = groups * N_ // 128
    scratch = torch.zeros(tiles * splits * 128 * NP, dtype=torch.float32, device=dev) if splits > 1 else None
    tickets = torch.zeros(tiles, dtype=torch.int32, device=dev) if splits > 1 else None
    for _ in range(2):  # twice: tickets must come back to zero
        N.umma_dense(ta, tb, sfa.to(dev), sfb.to(dev), n, N_, K, groups=groups, a_fp4=fp4, splits=splits,
                     scratch=scratch, tickets=tickets, out_f=out, status=status)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        err = (out.cpu() - ref).abs().max().item()
        assert err <= 2e-3 * ref.abs().max().item() + 1e-5, (err, ref.abs().max().item())
