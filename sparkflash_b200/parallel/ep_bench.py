"""Expert-parallel MoE layer over real ranks: the fused all-to-all dispatch (route + MXFP8 quantisation + peer stores),
the W4A8 expert GEMMs on the received rows, the combine (peer stores back to each token's rank) and the k-order fold, at
the flagship's per-token shapes (d = 5120, 384 routed experts, top-6, expert width 2304), tokens sharded over the ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port 29513 \
        -m sparkflash_b200.parallel.ep_bench [--tokens 1,2,8,64] [--iters 20] [--experts 384]

For every tokens-per-rank count it prints one JSON line (rank 0): the layer's time (CUDA events around replays of a CUDA
graph holding two steps, after warm-up, max over ranks), the time of the two NCCL ``all_to_all_single`` calls that move
the same payloads (FP8 rows + scales + records out, bf16 rows back), and the NVLink time of those bytes at 770 GB/s.
With ``--check`` rank 0 also runs the same tokens through a one-rank instance that holds every expert and compares: the
per-pair arithmetic and the k-order sum do not depend on where an expert lives, so every rank's output must match bit
for bit.  Reference behaviour: crates/sparkflash-model-inkling2/src/tensor.rs:49-78 (ExpertSplit::Experts exchange),
docs/rdma-exchange.md:141-145 (slot exchanges of the TP4 step).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _expert_weights(e0: int, e1: int, d: int, inter: int, dev):
    """Random packed FP4 codes and UE8M0 scales of experts [e0, e1): the same bytes whichever rank generates them."""
    q13, s13, q2, s2 = [], [], [], []
    for e in range(e0, e1):
        g = torch.Generator(device=dev).manual_seed(1000 + e)
        q13.append(torch.randint(0, 256, (2 * inter, d // 2), dtype=torch.uint8, device=dev, generator=g))
        q2.append(torch.randint(0, 256, (d, inter // 2), dtype=torch.uint8, device=dev, generator=g))
        s13.append(torch.randint(117, 122, (2 * inter, d // 32), dtype=torch.uint8, device=dev, generator=g))
        s2.append(torch.randint(117, 122, (d, inter // 32), dtype=torch.uint8, device=dev, generator=g))
    return torch.cat(q13), torch.cat(s13).cpu(), torch.cat(q2), torch.cat(s2).cpu()


def timed(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn(); fn()
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
    ap.add_argument("--tokens", default="1,2,8,64", help="tokens per rank (streams = tokens x ranks)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--inter", type=int, default=2304)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    rank, W = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from .ep import EpMoE
    from .symm import SymmHeap
    E, d, inter, k = a.experts, a.hidden, a.inter, a.top_k
    epr = E // W
    q13, s13, q2, s2 = _expert_weights(rank * epr, (rank + 1) * epr, d, inter, dev)
    full = None
    for t in [int(x) for x in a.tokens.split(",")]:
        heap = SymmHeap(rank, W, EpMoE.heap_bytes(W, t, d, k)).attach()
        op = EpMoE(heap, t, d, k, E, inter, q13, s13, q2, s2)
        g = torch.Generator().manual_seed(7 * t + rank)
        x = (torch.randn(t, d, generator=g) * 0.5).to(torch.bfloat16).cuda()
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(t)]).int().cuda()
        wts = (torch.rand(t, k, generator=g) + 0.2).cuda()
        add = torch.randn(t, d, generator=g).to(torch.bfloat16).cuda()

        def layer():
            op.dispatch(x, ids, wts)
            op.experts()
            op.combine()
            return op.fold(t, add)
        fused = timed(layer, a.iters)
        op.check()
        out = layer().clone()
        torch.cuda.synchronize()
        # the same payloads through NCCL: every rank sends t*k/W rows on average to each peer; all_to_all_single of the full
        # capacity split evenly is the closest library call (it cannot skip empty rows)
        rows_out = t * k
        send = torch.empty((W, max(1, rows_out // W) * (d + d // 32 + 16)), dtype=torch.uint8, device=dev)
        recv = torch.empty_like(send)
        back = torch.empty((W, max(1, rows_out // W) * d), dtype=torch.bfloat16, device=dev)
        back_r = torch.empty_like(back)

        def nccl_pair():
            dist.all_to_all_single(recv, send)
            dist.all_to_all_single(back_r, back)
        base = timed(nccl_pair, a.iters)
        moved = rows_out * (W - 1) / W * (d + d // 32 + 16 + 2 * d)
        rec = {"world": W, "tokens_per_rank": t, "streams": t * W, "fused_layer_us": round(fused, 1), "nccl_two_all_to_all_us": round(base, 1),
               "bytes_per_rank": int(moved), "nvlink_roofline_us": round(moved / (a.link_gbs * 1e9) * 1e6, 2), "experts_per_rank": epr}
        if a.check:
            outs = [torch.empty_like(out) for _ in range(W)]
            xs, idss, wtss, adds = ([torch.empty_like(v) for _ in range(W)] for v in (x, ids, wts, add))
            for lst, v in ((outs, out), (xs, x), (idss, ids), (wtss, wts), (adds, add)):
                dist.all_gather(lst, v)
            if rank == 0:
                if full is None:
                    full = _expert_weights(0, E, d, inter, dev)
                one = EpMoE(SymmHeap.local_group(1, EpMoE.heap_bytes(1, t, d, k))[0], t, d, k, E, inter, *full)
                same = True
                for r in range(W):
                    one.dispatch(xs[r], idss[r], wtss[r]); one.experts(); one.combine()
                    want = one.fold(t, adds[r]).clone()
                    torch.cuda.synchronize()
                    same = same and bool(torch.equal(want, outs[r]))
                one.check()
                rec["matches_single_rank_bits"] = same
                del one
        if rank == 0:
            print(json.dumps(rec), flush=True)
        del op
        heap.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
