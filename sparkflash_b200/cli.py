"""Command line: ``python -m sparkflash_b200 <models|doctor|trace|convert|pack-engram|serve|bench-serving>``.
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
    from .engram import packer
    rep = packer.pack(args.source, args.output_dir, world=args.world, dry_run=args.dry_run)
    print(f"pack-engram: wrote {len(rep['files'])} file(s), {rep['bytes']} bytes, into {args.output_dir}")
    return 0


def _serve(args) -> int:
    from .serve import launch
    return launch.run(args)


def _bench_serving(args) -> int:
    from .serve import bench_client
    return bench_client.run(args)


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
    args = ap.parse_args(argv)
    if not getattr(args, "fn", None):
        ap.print_help()
        return 0
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
