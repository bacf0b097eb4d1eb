"""Expert-parallel dispatch / grouped experts / combine, W virtual ranks in lockstep on one GPU, against a plain
fp32 reference of the same arithmetic (FP8 activations, W4A8 experts, clamp-SwiGLU, FP8 re-quant, k-order sum)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_dispatch_experts_combine_matches_reference():
    from sparkflash_b200 import codecs as C
    from sparkflash_b200.parallel.ep import EpMoE
    from sparkflash_b200.parallel.symm import SymmHeap
    W, t, d, k, E, inter, limit = 2, 5, 512, 3, 8, 256, 10.0
    epr = E // W
    g = torch.Generator().manual_seed(0)
    w13 = torch.randn(E, 2 * inter, d, generator=g) * 0.08
    w2 = torch.randn(E, d, inter, generator=g) * 0.08
    q13, s13 = C.weight_quant_fp4_row32(w13.reshape(E * 2 * inter, d))
    q2, s2 = C.weight_quant_fp4_row32(w2.reshape(E * d, inter))
    d13 = C.weight_dequant_fp4_row32(q13, s13).reshape(E, 2 * inter, d)
    d2 = C.weight_dequant_fp4_row32(q2, s2).reshape(E, d, inter)
    heaps = SymmHeap.local_group(W, EpMoE.heap_bytes(W, t, d, k))
    ops = []
    for r in range(W):
        r13 = slice(r * epr * 2 * inter, (r + 1) * epr * 2 * inter)
        r2 = slice(r * epr * d, (r + 1) * epr * d)
        ops.append(EpMoE(heaps[r], t, d, k, E, inter, q13[r13].cuda().contiguous(), s13[r13], q2[r2].cuda().contiguous(), s2[r2], limit, wait_ns=200_000_000))
    bf = lambda v: v.to(torch.bfloat16).float()
    for step in range(3):
        xs = [torch.randn(t, d, generator=g).to(torch.bfloat16) for _ in range(W)]
        ids = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(t)]).int() for _ in range(W)]
        wts = [torch.rand(t, k, generator=g) + 0.2 for _ in range(W)]
        add = [torch.randn(t, d, generator=g).to(torch.bfloat16) for _ in range(W)]
        for r in range(W):
            ops[r].dispatch(xs[r].cuda(), ids[r].cuda(), wts[r].cuda())
        for r in range(W):
            ops[r].experts()
        for r in range(W):
            ops[r].combine()
        outs = [ops[r].fold(t, add[r].cuda()).float().cpu() for r in range(W)]
        torch.cuda.synchronize()
        for r in range(W):
            ops[r].check()
            xq = C.act_roundtrip_fp8(xs[r].float())
            want = torch.zeros(t, d)
            for i in range(t):
                acc = torch.zeros(d)
                for j in range(k):
                    e = int(ids[r][i, j])
                    gu = d13[e] @ xq[i]
                    gg = torch.clamp(bf(gu[:inter]), max=limit)
                    uu = torch.clamp(bf(gu[inter:]), -limit, limit)
                    act = bf(gg * torch.sigmoid(gg) * uu * wts[r][i, j])
                    acc += bf(d2[e] @ C.act_roundtrip_fp8(act.unsqueeze(0))[0])
                want[i] = bf(acc + add[r][i].float())
            err = (outs[r] - want).abs().max()
            assert err < 0.03 * want.abs().max() + 0.02, (step, r, float(err), float(want.abs().max()))
