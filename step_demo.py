"""A few rows steps of a three-layer model at full per-token shapes, without CUDA graphs, for launch lists and
single-kernel captures:

    python step_demo.py --rows 64            # prompt chunks of one sequence
    python step_demo.py --rows 16 --decode   # one row per sequence

Only the last step sits between cudaProfilerStart/Stop, so a profiler started with its collection off sees exactly one
step (three layers: two window-only, one with the compressor, indexer and selection; plus the head when decoding).
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--decode", action="store_true", help="one row per sequence at the same position instead of a prompt chunk")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--steps", type=int, default=12, help="prompt chunks to run (the last one is the profiled / timed one)")
    ap.add_argument("--persistent-counters", action="store_true", help="read moe_gate_up / moe_down marks as the persistent kernels' cycle counters")
    ap.add_argument("--marks", default="", help="kernels whose in-kernel phase marks are printed for the last step, e.g. moe_down,moe_gate_up")
    ap.add_argument("--tune", default="", help="measurement switches of the MoE launchers, key=value[,key=value]")
    args = ap.parse_args()
    from sparkflash_b200.config import reduced_config
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P
    from sparkflash_b200.ops import native as N
    for kv in filter(None, args.tune.split(",")):
        k, v = kv.split("=")
        N.umma_tune(int(k), int(v))
    cfg = reduced_config(args.experts, args.layers)
    w = P.prepare_synthetic(cfg, 0, 1)
    rows = args.rows
    ctx = max(2048, rows * args.steps + 64)
    eng = E.Engine(w, max_lanes=max(2, rows if args.decode else 2), max_context=ctx, max_rows=max(64, rows), arm="tc",
                   synthetic_scales=True, use_graphs=False)
    prompt = torch.randint(0, cfg.vocab_size, (ctx,)).tolist()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.decode:
        for s in range(rows):
            eng.step(prompt[:64], [s] * 64, list(range(64)), head=False)
        for i in range(3):
            if i == 2:
                eng.kernel_marks = {k: ([torch.zeros(16 * 4096, dtype=torch.int64, device="cuda") for _ in range(args.layers)] if k == "attn" else
                                        torch.zeros(16 * 16384, dtype=torch.int64, device="cuda")) for k in filter(None, args.marks.split(","))}
                torch.cuda.synchronize(); torch.cuda.profiler.start()
            eng.step(prompt[:rows], list(range(rows)), [64 + i] * rows)
    else:
        pos = 0
        for i in range(args.steps):
            if i == args.steps - 1:
                eng.kernel_marks = {k: ([torch.zeros(16 * 4096, dtype=torch.int64, device="cuda") for _ in range(args.layers)] if k == "attn" else
                                        torch.zeros(16 * 16384, dtype=torch.int64, device="cuda")) for k in filter(None, args.marks.split(","))}
                torch.cuda.synchronize(); torch.cuda.profiler.start(); ev0.record()
            eng.step(prompt[pos:pos + rows], [0] * rows, list(range(pos, pos + rows)), head=False, sync=False); pos += rows
        ev1.record()
    torch.cuda.synchronize(); torch.cuda.profiler.stop()
    eng.check_status()
    for name, buf in getattr(eng, "kernel_marks", {}).items():
        from sparkflash_b200.utils import kernel_marks as KM
        if name == "attn":
            for li, b in enumerate(buf):
                print(name, "layer", li, KM.summarize_attention(b))
        elif name == "seam":
            words = N.seam_read_marks(rows)
            print(name, KM.summarize_seam(words, rows) if words is not None else "no marks in this library")
        elif name in ("moe_gate_up", "moe_down") and args.persistent_counters:
            print(name, KM.summarize_persistent(buf, "gate_up" if name == "moe_gate_up" else "down"))
        else:
            print(name, KM.summarize(buf))
    if not args.decode:
        print(f"last chunk: {rows} rows at context {pos} in {ev0.elapsed_time(ev1):.3f} ms ({args.layers} layers)")
    print("ok")


if __name__ == "__main__":
    main()
