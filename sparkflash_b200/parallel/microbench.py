"""Fused TP collective microbenchmark: row-parallel GEMM -> all-reduce / reduce-scatter and all-gather ->
column-parallel GEMM at K = N = hidden size, M in {1, 8, 64, 512, 8192}, against the NCCL + cuBLAS path and the
NVLink roofline.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port 29511 \
        -m sparkflash_b200.parallel.microbench [--hidden 5120] [--m 1,8,64,512,8192] [--iters 30]

Timing: CUDA events on the launching stream around replays of a CUDA graph holding two operations (both arms), after
warm-up, max over ranks.  Weights of every M are distinct buffers and larger than nothing but L2 is not flushed between
iterations: the activations change every iteration, the weights (13-26 MB per rank) stay L2-resident exactly as
they do inside a decode step.  Roofline: the slower of FLOPs / measured GEMM peak and bytes over NVLink / 770 GB/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def timed(fn, iters, warm=4):
    """Microseconds per call, max over ranks.  Two calls (both buffer parities) are captured into one CUDA graph and
    the graph is replayed, so that launch overhead of the Python layer is outside the measurement for both arms."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn(); fn()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, iters // 2)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / (2 * reps)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del g
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--m", "--rows", dest="m", default="1,8,64,512,8192", help="row counts (use --rows under torch.distributed.run, which claims --m)")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--peak-tflops", type=float, default=1376.0)     # sustained cuBLAS bf16 of this pool
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))))
    from .. import codecs as C
    from .fused_gemm import ColumnParallelLinear, RowParallelLinear
    from .symm import SymmHeap
    H = a.hidden
    Kl = H // W
    g = torch.Generator().manual_seed(100 + rank)
    w_row = torch.randn(H, Kl, generator=g) * 0.02          # row-parallel shard [N, K/W]
    w_col = torch.randn(H // W, H, generator=g) * 0.02      # column-parallel shard [N/W, K]
    qr, sr = C.weight_quant_fp8_block32(w_row)
    qc, sc = C.weight_quant_fp8_block32(w_col)
    wr_bf, wc_bf = w_row.to(torch.bfloat16).cuda(), w_col.to(torch.bfloat16).cuda()
    rows = []
    for M in [int(x) for x in a.m.split(",")]:
        x_l = torch.randn(M, Kl, generator=g).to(torch.bfloat16).cuda()
        res = torch.randn(M, H, generator=g).to(torch.bfloat16).cuda()
        flops = 2.0 * M * H * H / W
        t_compute = flops / (a.peak_tflops * 1e12) * 1e6
        # ---- GEMM -> all-reduce ------------------------------------------------------------------------------
        heap = SymmHeap(rank, W, RowParallelLinear.heap_bytes(M, H, W, "ar")).attach()
        op = RowParallelLinear(heap, qr.cuda(), sr, M, "ar", norm_w=torch.ones(H, device="cuda"))
        fused = timed(lambda: op.forward(x_l, res), a.iters)
        op.check()
        y = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")

        def base_ar():
            torch.mm(x_l, wr_bf.t(), out=y)
            dist.all_reduce(y)
            z = y + res
            torch.nn.functional.rms_norm(z, (H,), eps=1e-6)
        base = timed(base_ar, a.iters)
        # bytes every rank must send: one shot = its whole partial to each peer; two shots (reduce-scatter + all-gather of the
        # folded rows, the form used from RowParallelLinear.TWO_SHOT_ROWS rows on) = 2 (W - 1) / W of the partial
        two = op.two_shot
        link = M * H * 2 * ((2 * (W - 1) / W) if two else (W - 1)) / (a.link_gbs * 1e9) * 1e6
        rows.append({"op": "gemm_allreduce", "M": M, "fused_us": fused, "nccl_cublas_us": base, "roofline_us": max(t_compute, link),
                     "frac_of_roofline": max(t_compute, link) / fused, "form": "two_shot" if two else "one_shot"})
        del op; heap.close()
        # ---- GEMM -> reduce-scatter ----------------------------------------------------------------------------
        if M % W == 0:
            heap = SymmHeap(rank, W, RowParallelLinear.heap_bytes(M, H, W, "rs")).attach()
            op = RowParallelLinear(heap, qr.cuda(), sr, M, "rs", norm_w=torch.ones(H, device="cuda"))
            r_own = res[rank * (M // W):(rank + 1) * (M // W)].contiguous()
            fused = timed(lambda: op.forward(x_l, r_own), a.iters)
            op.check()
            ys = torch.empty(M // W, H, dtype=torch.bfloat16, device="cuda")

            def base_rs():
                torch.mm(x_l, wr_bf.t(), out=y)
                dist.reduce_scatter_tensor(ys, y)
                z = ys + r_own
                torch.nn.functional.rms_norm(z, (H,), eps=1e-6)
            base = timed(base_rs, a.iters)
            link = M * H * 2 * (W - 1) / W / (a.link_gbs * 1e9) * 1e6
            rows.append({"op": "gemm_reducescatter", "M": M, "fused_us": fused, "nccl_cublas_us": base, "roofline_us": max(t_compute, link),
                         "frac_of_roofline": max(t_compute, link) / fused})
            del op; heap.close()
        # ---- all-gather -> GEMM ----------------------------------------------------------------------------------
        fused_by_mode = {}
        for mode in ("gather", "remote"):
            heap = SymmHeap(rank, W, ColumnParallelLinear.heap_bytes(M, H, W, mode)).attach()
            op = ColumnParallelLinear(heap, qc.cuda(), sc, M, mode=mode)
            fused_by_mode[mode] = timed(lambda: op.forward(x_l), a.iters)
            op.check()
            del op; heap.close()
        fused = fused_by_mode["gather"]
        gathered = torch.empty(W * M, Kl, dtype=torch.bfloat16, device="cuda")
        yc = torch.empty(M, H // W, dtype=torch.bfloat16, device="cuda")

        def base_ag():
            dist.all_gather_into_tensor(gathered, x_l)
            xf = gathered.view(W, M, Kl).permute(1, 0, 2).reshape(M, H)
            torch.mm(xf, wc_bf.t(), out=yc)
        base = timed(base_ag, a.iters)
        link = M * H * (W - 1) / W / (a.link_gbs * 1e9) * 1e6          # FP8 activations cross once
        rows.append({"op": "allgather_gemm", "M": M, "fused_us": fused, "nccl_cublas_us": base, "roofline_us": max(t_compute, link),
                     "frac_of_roofline": max(t_compute, link) / fused, "fused_remote_reads_us": fused_by_mode["remote"],
                     "remote_reads_nvlink_reread_factor": max(1, (H // W) // 128)})
    # The compute term above uses the measured bf16 GEMM rate; the kernels run kind::mxf8f6f4, whose hardware rate is about
    # twice that, and no FP8 rate was measured on this pool: a second fraction against 2 x the bf16 figure is printed too.
    for r in rows:
        t_c8 = 2.0 * r["M"] * H * H / W / (2 * a.peak_tflops * 1e12) * 1e6
        link_us = {"gemm_allreduce": r["M"] * H * 2 * ((2 * (W - 1) / W) if r.get("form") == "two_shot" else (W - 1)), "gemm_reducescatter": r["M"] * H * 2 * (W - 1) / W,
                   "allgather_gemm": r["M"] * H * (W - 1) / W}[r["op"]] / (a.link_gbs * 1e9) * 1e6
        r["roofline_fp8peak_us"] = max(t_c8, link_us)
        r["frac_of_roofline_fp8peak"] = max(t_c8, link_us) / r["fused_us"]
        r["fused_vs_nccl_cublas"] = r["nccl_cublas_us"] / r["fused_us"]
    if rank == 0:
        for r in rows:
            print(json.dumps({"world": W, "hidden": H, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
