"""Command line: ``python -m sparkflash_b200 <models|doctor|trace|convert|pack-engram|serve|bench-serving|web|device-chain|
inkling-tp4|plan|roofline|gates|served-gate>``.
Reference: crates/sparkflash-cli/src/main.rs:50-76 (subcommand table), convert.rs:76 (convert usage),
serve.rs:6418-6590 (serve orchestration)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def _models(args) -> int:
    from .models import registry
    for m in registry.MODELS.values():
        print(f"{m.name:28s} {m.family:10s} {m.status:12s} {m.summary}")
    return 0


def _doctor(args) -> int:
    from .utils import doctor
    text, ok = doctor.report(doctor.run_checks(need_gpus=args.gpus, weights_dir=args.weights, world=args.gpus))
    print(text)
    return 0 if ok else 1


def _convert(args) -> int:
    from .weights import convert as C
    if args.inspect:
        print(json.dumps(C.inspect(args.inspect, args.verify_weights), indent=1))
        return 0
    if args.synthetic:
        from . import config as CF
        cfg = {"tiny": CF.tiny_config, "full": CF.full_config}[args.synthetic]()
        C.export_synthetic_checkpoint(args.checkpoint, cfg, seed=0)
    ranks = [int(r) for r in args.ranks.split(",")] if args.ranks else None

    def progress(done, total, detail):
        print("@progress " + json.dumps({"done": done, "total": total, "detail": detail}), flush=True)
    man = C.convert(args.checkpoint, args.output_dir, args.tp_world_size, ranks, not args.no_verify, progress, args.expert_split)
    print(f"convert: wrote {len(man['ranks'])} rank file(s) into {args.output_dir}")
    return 0


def _trace(args) -> int:
    import urllib.request
    base = args.url.rstrip("/")
    hdr = {"Authorization": f"Bearer {args.api_key}"} if args.api_key else {}
    if args.action == "arm":
        req = urllib.request.Request(base + "/v1/admin/trace", data=json.dumps({"scopes": args.scopes, "steps": args.steps}).encode(),
                                     headers={**hdr, "Content-Type": "application/json"}, method="POST")
    elif args.action == "status":
        req = urllib.request.Request(base + "/v1/admin/trace", headers=hdr)
    else:
        req = urllib.request.Request(base + "/v1/admin/trace/dump", headers=hdr)
    body = urllib.request.urlopen(req, timeout=30).read()
    if args.action == "dump" and args.output:
        with open(args.output, "wb") as f:
            f.write(body)
        print(f"trace: wrote {len(body)} bytes to {args.output}")
    else:
        print(body.decode())
    return 0


def _pack_engram(args) -> int:
    from .engram import store as packer
    rep = packer.pack(args.source, args.output_dir, world=args.world, dry_run=args.dry_run)
    print(f"pack-engram: wrote {len(rep['files'])} file(s), {rep['bytes']} bytes, into {args.output_dir}")
    return 0


def _serve(args) -> int:
    from .serve import launch
    return launch.run(args)


def _bench_serving(args) -> int:
    from .serve import bench_client
    return bench_client.run(args)


def _web(args) -> int:
    from .web import app
    return app.main(["--host", args.host, "--port", str(args.port), "--server", args.server_url])


def _device_chain(args) -> int:
    """The engine loop without HTTP: prefill a synthetic prompt in chunks, decode, print one JSON line with the rates
    (reference: crates/sparkflash-cli/src/device_chain.rs:351-383, tp4_chain.rs run_loop)."""
    import time

    import torch
    from . import config as CF
    from .models.deepseek_v41 import engine as E, prepare as P
    from .utils.evidence import run_header
    cfg = {"tiny": CF.tiny_config, "reduced": lambda: CF.reduced_config(args.experts, args.layers), "full": CF.full_config}[args.synthetic]()
    if args.synthetic == "tiny":
        from .models.deepseek_v41 import weights as W
        w = P.prepare_from_checkpoint(W.synthetic_checkpoint(cfg, 0), cfg)
    else:
        w = P.prepare_synthetic(cfg, 0, 1)
    eng = E.Engine(w, max_lanes=2, max_context=args.prompt + args.tokens + 64, max_rows=args.chunk, arm=args.arm,
                   synthetic_scales=args.synthetic != "tiny")
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=torch.Generator().manual_seed(0)).tolist()
    eng.generate(prompt[:min(len(prompt), args.chunk)], 2, lane=1, chunk=args.chunk)         # graphs and lazy set-up
    torch.cuda.synchronize(); t0 = time.perf_counter()
    pos, nxt = 0, 0
    while pos < len(prompt):
        c = prompt[pos:pos + args.chunk]
        r = eng.step(c, [0] * len(c), list(range(pos, pos + len(c))), head="last" if pos + len(c) >= len(prompt) else False)
        nxt, pos = int(r[len(c) - 1]), pos + len(c)
    t1 = time.perf_counter()
    out = []
    for _ in range(args.tokens):
        out.append(nxt)
        nxt = int(eng.step([nxt], [0], [pos])[0]); pos += 1
    t2 = time.perf_counter()
    eng.check_status()
    print(json.dumps({"header": run_header(eng), "prefill_tok_s": len(prompt) / (t1 - t0), "decode_tok_s": args.tokens / (t2 - t1),
                      "launches_per_step": eng.launches_per_step, "tokens": out[:16]}))
    return 0


def _inkling_tp4(args) -> int:
    """Inkling-2 under its three expert splits on ``world`` simulated ranks: the logits of every split against the unsplit
    model (reference: crates/sparkflash-cli inkling-tp4, crates/sparkflash-model-inkling2/src/tensor.rs:49-78)."""
    import torch
    from .models import inkling as IK
    c = IK.InklingConfig()
    w = IK.init_weights(c, 0)
    toks = torch.randint(0, c.vocab, (args.tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    base = IK.reference_logits(c, w, toks)
    rep = {}
    for split in ("experts", "intermediate", "rows"):
        got = IK.reference_logits(c, w, toks, world=args.world, split=split)
        rep[split] = float((got - base).abs().max())
    print(json.dumps({"world": args.world, "max_abs_vs_unsplit": rep}))
    return 0 if max(rep.values()) < 1e-3 else 1


def _plan(args) -> int:
    from . import config as CF
    from .models import tp_plan as TP
    from .ops import plan as OP
    cfg = CF.full_config()
    tp = TP.plan(cfg, args.world, args.moe_mode)
    steps = {str(n): OP.plan_step(n, "tc", args.world).__dict__ | {"collective": OP.plan_step(n, "tc", args.world).collective.kind.value}
             for n in (1, 5, 16, 64, 128, 1024)}
    print(json.dumps({"world": args.world, "moe_mode": args.moe_mode, "gb_per_rank": round(tp.bytes_per_rank() / 1e9, 2),
                      "heads_per_rank": tp.heads_per_rank, "inter_per_rank": tp.inter_per_rank, "vocab_per_rank": tp.vocab_per_rank,
                      "experts_per_rank": tp.experts_per_rank, "collectives_per_step": tp.collectives_per_step(), "tensors": tp.table(),
                      "step_plans": steps}, indent=1, default=str))
    return 0


def _roofline(args) -> int:
    """Per-kernel-class roofline table of one rows step at the flagship's per-token shapes (utils/roofline.py)."""
    import torch
    from . import config as CF
    from .models.deepseek_v41 import engine as E, prepare as P
    from .utils import roofline as R
    cfg = CF.reduced_config(args.experts, args.layers)
    eng = E.Engine(P.prepare_synthetic(cfg, 0, 1), max_lanes=max(2, args.rows if args.decode else 2), max_context=args.context + 2 * args.rows + 64,
                   max_rows=max(64, args.rows), arm="tc", synthetic_scales=True, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (args.context + 2 * args.rows,), generator=g).tolist()
    n = args.rows
    if args.decode:
        for s_ in range(n):
            eng.step(ids[:64], [s_] * 64, list(range(64)), head=False)
        call = (ids[:n], list(range(n)), [64] * n)
        eng.step(*call)
        ctx = 64
    else:
        pos = 0
        while pos < args.context:
            c = min(n, args.context - pos)
            eng.step(ids[pos:pos + c], [0] * c, list(range(pos, pos + c)), head=False)
            pos += c
        call = (ids[pos:pos + n], [0] * n, list(range(pos, pos + n)))
        eng.step(*call, head=False)                  # warm every lazily built buffer of this shape
        call = (ids[pos + n:pos + 2 * n], [0] * n, list(range(pos + n, pos + 2 * n)))
        ctx = pos + n
    timings = R.timed_step(eng, *call, **({} if args.decode else {"head": False}))
    eng.check_status()
    rows = R.account(timings, R.work_model(eng, n, ctx, head_rows=n if args.decode else 0))
    print(R.format_table(rows))
    print(json.dumps({"rows": n, "context": ctx, "layers": args.layers, "experts": args.experts, "launches": len(timings),
                      "step_us": round(sum(t for _, t in timings), 1), "peaks": R.peaks()}))
    return 0


def _gates(args) -> int:
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "ci", "host_gates.py")
    if not os.path.exists(script):
        print("gates: ci/host_gates.py is not part of this installation")
        return 2
    return subprocess.call([sys.executable, script] + (["--skip-tests"] if args.skip_tests else []))


def _served_gate(args) -> int:
    from .gates import served
    return served.main(["--url", args.url, "--tokens", str(args.tokens), "--concurrency", str(args.concurrency)] +
                       (["--api-key", args.api_key] if args.api_key else []))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sparkflash_b200")
    sub = ap.add_subparsers(dest="cmd")
    sub.add_parser("models").set_defaults(fn=_models)
    d = sub.add_parser("doctor"); d.add_argument("--gpus", type=int, default=1); d.add_argument("--weights"); d.set_defaults(fn=_doctor)
    c = sub.add_parser("convert")
    c.add_argument("--checkpoint"); c.add_argument("--output-dir"); c.add_argument("--tp-world-size", type=int, default=1)
    c.add_argument("--ranks"); c.add_argument("--no-verify", action="store_true"); c.add_argument("--inspect")
    c.add_argument("--verify-weights", action="store_true"); c.add_argument("--expert-split", default="tp", choices=["tp", "ep"], help="tp: experts sliced by width; ep: whole experts per rank"); c.add_argument("--synthetic", choices=["tiny", "full"])
    c.set_defaults(fn=_convert)
    t = sub.add_parser("trace")
    t.add_argument("action", choices=["arm", "status", "dump"]); t.add_argument("--url", default="http://127.0.0.1:8000")
    t.add_argument("--scopes", default="all"); t.add_argument("--steps", type=int, default=64); t.add_argument("--output"); t.add_argument("--api-key")
    t.set_defaults(fn=_trace)
    e = sub.add_parser("pack-engram")
    e.add_argument("--source", required=True); e.add_argument("--output-dir", required=True); e.add_argument("--world", type=int, default=1)
    e.add_argument("--dry-run", action="store_true"); e.set_defaults(fn=_pack_engram)
    s = sub.add_parser("serve")
    s.add_argument("--weights", help="directory of converted rank files"); s.add_argument("--synthetic", choices=["tiny", "reduced", "full"])
    s.add_argument("--tokenizer"); s.add_argument("--host", default="127.0.0.1"); s.add_argument("--port", type=int, default=8000)
    s.add_argument("--api-key", default=os.environ.get("SFB_API_KEY")); s.add_argument("--config", help="TOML settings file")
    s.add_argument("--model-id", default="deepseek-v4.1-flash"); s.add_argument("--control-port", type=int, default=29600)
    s.add_argument("--mock", action="store_true", help="serve the scripted mock engine (no GPU)")
    s.add_argument("--lane-budget-gb", type=int, default=0, help="back the per-position KV regions lazily from a pool of this size")
    s.set_defaults(fn=_serve)
    b = sub.add_parser("bench-serving")
    b.add_argument("--url", default="http://127.0.0.1:8000"); b.add_argument("--concurrency", type=int, default=16)
    b.add_argument("--requests", type=int, default=32); b.add_argument("--prompt-tokens", type=int, default=512)
    b.add_argument("--max-tokens", type=int, default=128); b.add_argument("--api-key"); b.set_defaults(fn=_bench_serving)
    wb = sub.add_parser("web"); wb.add_argument("--host", default="127.0.0.1"); wb.add_argument("--port", type=int, default=8080)
    wb.add_argument("--server-url", default="http://127.0.0.1:8000"); wb.set_defaults(fn=_web)
    dc = sub.add_parser("device-chain")
    dc.add_argument("--synthetic", default="reduced", choices=["tiny", "reduced", "full"]); dc.add_argument("--experts", type=int, default=32)
    dc.add_argument("--layers", type=int, default=8); dc.add_argument("--prompt", type=int, default=2048); dc.add_argument("--tokens", type=int, default=64)
    dc.add_argument("--chunk", type=int, default=1024); dc.add_argument("--arm", default="tc", choices=["tc", "cuda"]); dc.set_defaults(fn=_device_chain)
    ik = sub.add_parser("inkling-tp4"); ik.add_argument("--world", type=int, default=4); ik.add_argument("--tokens", type=int, default=12)
    ik.set_defaults(fn=_inkling_tp4)
    pl = sub.add_parser("plan"); pl.add_argument("--world", type=int, default=8); pl.add_argument("--moe-mode", default="tp", choices=["tp", "ep"])
    pl.set_defaults(fn=_plan)
    rf = sub.add_parser("roofline"); rf.add_argument("--rows", type=int, default=1024); rf.add_argument("--context", type=int, default=4096)
    rf.add_argument("--layers", type=int, default=3); rf.add_argument("--experts", type=int, default=128)
    rf.add_argument("--decode", action="store_true", help="one row per sequence instead of a prompt chunk"); rf.set_defaults(fn=_roofline)
    gt = sub.add_parser("gates"); gt.add_argument("--skip-tests", action="store_true"); gt.set_defaults(fn=_gates)
    sg = sub.add_parser("served-gate"); sg.add_argument("--url", default="http://127.0.0.1:8000"); sg.add_argument("--tokens", type=int, default=48)
    sg.add_argument("--concurrency", type=int, default=4); sg.add_argument("--api-key"); sg.set_defaults(fn=_served_gate)
    args = ap.parse_args(argv)
    if not getattr(args, "fn", None):
        ap.print_help()
        return 0
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
