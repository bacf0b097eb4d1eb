"""``serve``: build the engine of this rank, start the driver, and (on rank 0) the HTTP server.

One process per GPU; with more than one rank the processes are started by ``torch.distributed.run`` and
find each other through its environment.  Rank 0 owns the HTTP surface and plans; the other ranks follow the
control channel.  SIGTERM drains: no new requests, running ones finish, then the group leaves.
Reference: crates/sparkflash-cli/src/serve.rs:6418-6590 (run), serve/device.rs (device driver boot).
"""
from __future__ import annotations

import json
import os
import signal
import sys
import time


def _boot(msg: str, **kw) -> None:
    print(json.dumps({"ts": round(time.time(), 3), "pid": os.getpid(), "boot": msg, **kw}), file=sys.stderr, flush=True)


def build_engine(args, settings, rank: int, world: int):
    import torch
    from .. import config as CF
    from ..models.deepseek_v41 import engine as E, prepare as P
    from ..parallel import comm as PC
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if args.weights:
        from ..weights.convert import rank_path
        from ..weights.files import load_rank_file
        w = load_rank_file(rank_path(args.weights, rank, world), "cuda", expect_rank=rank, expect_world=world)
        if w.moe_mode != settings.parallel.moe_mode:
            raise SystemExit(f"rank files were converted for moe_mode={w.moe_mode!r}, the settings ask for {settings.parallel.moe_mode!r}")
        synthetic = False
    else:
        cfg = {"tiny": CF.tiny_config, "reduced": lambda: CF.reduced_config(128, 40), "full": CF.full_config}[args.synthetic or "tiny"]()
        if (args.synthetic or "tiny") == "tiny":
            from ..models.deepseek_v41 import weights as W
            w = P.prepare_from_checkpoint(W.synthetic_checkpoint(cfg, 0), cfg, rank, world, moe_mode=settings.parallel.moe_mode)
            synthetic = False
        else:
            w = P.prepare_synthetic(cfg, rank, world, moe_mode=settings.parallel.moe_mode, mtp=settings.engine.speculation)
            synthetic = True
    comm = PC.make_comm(settings.parallel.collective, rank, world) if world > 1 else None
    ec = settings.engine
    make = E.Engine.with_guards if os.environ.get("SFB_DEBUG_BOUNDS") == "1" else E.Engine
    eng = make(w, max_lanes=ec.max_lanes, max_context=min(ec.max_context, 1 << 16) if args.synthetic else ec.max_context,
                   max_rows=ec.max_rows, comm=comm, use_graphs=ec.cuda_graphs, arm="tc", synthetic_scales=synthetic, constrained=True,
                   drafter=ec.speculation and bool(w.mtp_layers) and settings.parallel.moe_mode == "tp",
                   lane_budget_bytes=getattr(args, "lane_budget_gb", 0) * (1 << 30) or None)
    if comm is not None:
        comm.attach(eng)
    return eng


def run(args) -> int:
    from .. import config as CF
    from ..utils.trace import TraceController
    from .server import Server
    from .tokenizer import load_tokenizer
    settings = CF.Settings()
    if args.config:
        settings.apply_dict(CF.load_toml(args.config))
    settings.apply_env()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    settings.parallel.world = world
    _boot("settings", digest=settings.digest(), rank=rank, world=world)
    trace = TraceController()
    if args.mock:
        from .engine_api import MockEngine
        tok = load_tokenizer(args.tokenizer)
        engine = MockEngine(tok, model_id=args.model_id)
        driver = None
    else:
        import torch.distributed as dist
        if world > 1:
            import torch
            local = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local)          # before the first collective: every rank on its own GPU
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            # every rank must start from the same effective settings
            words = [None] * world
            dist.all_gather_object(words, settings.digest())
            if len(set(words)) != 1:
                raise SystemExit(f"settings differ across ranks: {words}")
        from ..parallel.control import ControlChannel
        from .driver import DeviceDriver, NgramDrafter
        eng = build_engine(args, settings, rank, world)
        tok = load_tokenizer(args.tokenizer, eng.cfg.vocab_size)
        chan = ControlChannel(rank, world, addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), port=args.control_port) if world > 1 else None
        from .driver import DSparkDrafter
        drafter = None
        if settings.engine.speculation:      # the model's own draft stages when the weights carry them, prompt look-up otherwise
            drafter = DSparkDrafter(settings.engine.spec_depth) if eng.drafter else NgramDrafter(settings.engine.spec_depth)
        driver = DeviceDriver(eng, tok, model_id=args.model_id, channel=chan, drafter=drafter, queue_depth=settings.engine.queue_depth,
                              prefix_reuse_min=settings.engine.prefix_reuse_min_rows, stall_seconds=settings.engine.stall_secs,
                              decoder_skip=settings.engine.decoder_skip).start()
        engine = driver
        _boot("engine ready", rank=rank, weights_gb=round(eng.w.nbytes() / 1e9, 2), kv_gb=round(eng.kv.nbytes() / 1e9, 2))
        if rank != 0:
            # followers have no HTTP surface: they serve ticks until the channel closes
            while driver.failed is None and chan.alive()[0]:
                time.sleep(0.2)
            orderly = 0 in chan.departed           # the leader drained and said goodbye: not a failure
            _boot("follower leaving", rank=rank, reason=driver.failed or chan.alive()[1], orderly=orderly)
            driver.shutdown(1.0)
            eng.close()
            if world > 1:
                dist.destroy_process_group()
            return 0 if (driver.failed is None or orderly) else 1
    aliases = dict(kv.split("=", 1) for kv in os.environ.get("SFB_MODEL_ALIASES", "").split(",") if "=" in kv)
    srv = Server(engine, api_key=args.api_key, aliases=aliases, trace=trace)
    import uvicorn
    config = uvicorn.Config(srv.app, host=args.host, port=args.port, log_level="warning")
    server = uvicorn.Server(config)

    def drain(signum, frame):
        srv.draining = True
        server.should_exit = True
    signal.signal(signal.SIGTERM, drain)
    _boot("listening", host=args.host, port=args.port, model=engine.model_id)
    server.run()
    if driver is not None:
        driver.shutdown(30.0)
        if world > 1:
            import torch.distributed as dist
            driver.engine.close()
            dist.destroy_process_group()
    return 0
