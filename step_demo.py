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
    args = ap.parse_args()
    from sparkflash_b200.config import reduced_config
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P
    cfg = reduced_config(args.experts, args.layers)
    w = P.prepare_synthetic(cfg, 0, 1)
    rows = args.rows
    eng = E.Engine(w, max_lanes=max(2, rows if args.decode else 2), max_context=2048, max_rows=max(64, rows), arm="tc",
                   synthetic_scales=True, use_graphs=False)
    prompt = torch.randint(0, cfg.vocab_size, (2048,)).tolist()
    if args.decode:
        for s in range(rows):
            eng.step(prompt[:64], [s] * 64, list(range(64)), head=False)
        for i in range(3):
            if i == 2:
                torch.cuda.synchronize(); torch.cuda.profiler.start()
            eng.step(prompt[:rows], list(range(rows)), [64 + i] * rows)
    else:
        pos = 0
        for i in range(12):
            if i == 11:
                torch.cuda.synchronize(); torch.cuda.profiler.start()
            eng.step(prompt[pos:pos + rows], [0] * rows, list(range(pos, pos + rows)), head=False); pos += rows
    torch.cuda.synchronize(); torch.cuda.profiler.stop()
    eng.check_status()
    print("ok")


if __name__ == "__main__":
    main()
