"""Fused GEMM + collective operators, W virtual ranks in lockstep on one GPU (all producers run, then all
consumers: nobody ever waits for a kernel that has not been launched).  Numerics against a plain fp32 reference
of the same arithmetic: FP8-quantised activations times dequantised FP8 weights, summed over ranks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(rows, K, seed):
    from sparkflash_b200 import codecs as C
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, K, generator=g) * 0.05
    q, sf = C.weight_quant_fp8_block32(w)
    return q, sf, C.weight_dequant_fp8_block32(q, sf)


def _ref_act(x):
    from sparkflash_b200 import codecs as C
    return C.act_roundtrip_fp8(x.float())


@pytest.mark.parametrize("M,mode", [(1, "ar"), (8, "ar"), (64, "ar"), (256, "ar"), (256, "rs"), (512, "rs")])
def test_row_parallel_gemm_then_reduce(M, mode):
    from sparkflash_b200.parallel.fused_gemm import RowParallelLinear
    from sparkflash_b200.parallel.symm import SymmHeap
    W, N, K = 2, 512, 1024
    Kl = K // W
    heaps = SymmHeap.local_group(W, RowParallelLinear.heap_bytes(M, N, W, mode))
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    norm_w = (1 + 0.1 * torch.randn(N, generator=g)).cuda()
    ops, ref = [], torch.zeros(M, N)
    for r in range(W):
        q, sf, wd = _weights(N, Kl, 10 + r)
        ops.append(RowParallelLinear(heaps[r], q.cuda(), sf, M, mode, norm_w=norm_w, eps=1e-6, wait_ns=200_000_000))
        part = _ref_act(x[:, r * Kl:(r + 1) * Kl]) @ wd.t()
        ref += part.to(torch.bfloat16).float()           # partials travel as bf16
    for step in range(3):                                 # several steps: parity buffers and epochs
        for r in range(W):
            ops[r].produce(x[:, r * Kl:(r + 1) * Kl].cuda().contiguous())
        outs = []
        for r in range(W):
            rows = slice(r * (M // W), (r + 1) * (M // W)) if mode == "rs" else slice(0, M)
            outs.append((rows, ops[r].consume(res[rows].cuda().contiguous()).float().cpu(), ops[r].out_sum.float().cpu()))
        torch.cuda.synchronize()
        for r in range(W):
            ops[r].check()
        for rows, out, out_sum in outs:
            want_sum = (ref[rows] + res[rows].float())
            assert (out_sum - want_sum).abs().max() < 0.02 * want_sum.abs().max() + 0.02
            wn = want_sum.to(torch.bfloat16).float() * 0 + want_sum
            wn = wn * torch.rsqrt(wn.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.cpu()
            assert (out - wn).abs().max() < 0.03 * wn.abs().max() + 0.02


def test_two_shot_all_reduce_of_many_rows():
    """From 512 rows on the all-reduce runs as reduce-scatter + fold on the owner + all-gather of the folded rows; every rank
    ends with all rows.  (Emulated ranks: all produce, all fold and push, then all wait.)"""
    from sparkflash_b200.parallel.fused_gemm import RowParallelLinear
    from sparkflash_b200.parallel.symm import SymmHeap
    W, N, K, M = 2, 512, 1024, 640
    Kl = K // W
    heaps = SymmHeap.local_group(W, RowParallelLinear.heap_bytes(M, N, W, "ar"))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    norm_w = (1 + 0.1 * torch.randn(N, generator=g)).cuda()
    ops, ref = [], torch.zeros(M, N)
    for r in range(W):
        q, sf, wd = _weights(N, Kl, 20 + r)
        ops.append(RowParallelLinear(heaps[r], q.cuda(), sf, M, "ar", norm_w=norm_w, eps=1e-6, wait_ns=200_000_000))
        assert ops[-1].two_shot
        ref += (_ref_act(x[:, r * Kl:(r + 1) * Kl]) @ wd.t()).to(torch.bfloat16).float()
    want = ref + res.float()
    want = want * torch.rsqrt(want.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.cpu()
    for step in range(3):
        for r in range(W):
            ops[r].produce(x[:, r * Kl:(r + 1) * Kl].cuda().contiguous())
        for r in range(W):
            ops[r].consume(res.cuda(), wait=False)
        outs = [ops[r].gathered().float().cpu() for r in range(W)]
        torch.cuda.synchronize()
        for r in range(W):
            ops[r].check()
            assert (outs[r] - want).abs().max() < 0.03 * want.abs().max() + 0.02
        assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("mode", ["gather", "remote"])
@pytest.mark.parametrize("M", [1, 16, 128, 384])
def test_all_gather_then_column_parallel_gemm(M, mode):
    from sparkflash_b200.parallel.fused_gemm import ColumnParallelLinear
    from sparkflash_b200.parallel.symm import SymmHeap
    W, N, K = 2, 512, 1024
    Nl, Kl = N // W, K // W
    heaps = SymmHeap.local_group(W, ColumnParallelLinear.heap_bytes(M, K, W, mode))
    g = torch.Generator().manual_seed(1)
    ops, wds = [], []
    for r in range(W):
        q, sf, wd = _weights(Nl, K, 20 + r)
        ops.append(ColumnParallelLinear(heaps[r], q.cuda(), sf, M, mode=mode, wait_ns=200_000_000))
        wds.append(wd)
    for step in range(3):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        xr = _ref_act(x)
        for r in range(W):
            ops[r].publish(x[:, r * Kl:(r + 1) * Kl].cuda().contiguous())
        outs = [ops[r].gemm().float().cpu() for r in range(W)]
        torch.cuda.synchronize()
        for r in range(W):
            ops[r].check()
            want = xr @ wds[r].t()
            assert (outs[r] - want).abs().max() < 0.02 * want.abs().max() + 0.01, (M, r, step)


def test_a_gather_gemm_whose_peer_shard_never_arrives_times_out_with_a_status():
    """The all-gather -> GEMM kernel waits for a shard inside its producer warp; the wait is bounded, later CTAs do not wait
    again, nothing is written, and the context stays usable."""
    from sparkflash_b200.parallel.fused_gemm import ColumnParallelLinear
    from sparkflash_b200.parallel.symm import SymmHeap
    W, N, K, M = 2, 512, 1024, 16
    heaps = SymmHeap.local_group(W, ColumnParallelLinear.heap_bytes(M, K, W))
    q, sf, _ = _weights(N // W, K, 5)
    op = ColumnParallelLinear(heaps[0], q.cuda(), sf, M, wait_ns=50_000_000)           # 50 ms limit
    op.publish(torch.randn(M, K // W).to(torch.bfloat16).cuda())                       # rank 1 never publishes
    op.gemm()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status"):
        op.check()
    assert torch.zeros(4, device="cuda").sum().item() == 0


def test_a_consumer_whose_producer_never_arrives_times_out_with_a_status():
    from sparkflash_b200.parallel.fused_gemm import RowParallelLinear
    from sparkflash_b200.parallel.symm import SymmHeap
    W, N, K, M = 2, 256, 512, 8
    heaps = SymmHeap.local_group(W, RowParallelLinear.heap_bytes(M, N, W, "ar"))
    q, sf, _ = _weights(N, K // W, 3)
    op = RowParallelLinear(heaps[0], q.cuda(), sf, M, "ar", wait_ns=50_000_000)      # 50 ms limit
    op.produce(torch.randn(M, K // W).to(torch.bfloat16).cuda())                      # rank 1 never produces
    op.consume()
    torch.cuda.synchronize()                                                           # returns: the wait is bounded
    with pytest.raises(RuntimeError, match="device status"):
        op.check()
    assert torch.zeros(4, device="cuda").sum().item() == 0                            # the context is still usable
