#!/usr/bin/env python
"""Headline benchmark: single-stream decode tok/s of the DeepSeek-V4.1-Flash architecture (random-init
weights in the stored layout: MXFP4 routed experts, MXFP8 dense/attention, bf16 norms/embeddings), with the
other configurations of the metric reported under ``extra``:

* prefill of a 32,768-token prompt in chunks of rows (all layers on every row, and with the decoder-layer skip),
* decode at 4 / 8 / 16 streams (device-timed and end to end), decode at temperature 1.0,
* the DSpark draft path: per-forward latency with speculation off and on,
* decode against 131,072 and 1,048,576 cached tokens,
* on 2+ GPUs: whole experts per rank (expert parallelism) at 4 / 8 / 16 streams.

    python bench.py --gpus 1 --steps 64 --warmup 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 64 --warmup 4
    python bench.py --impl reference ...        # the reference arm (see below)

One "step" is one decode step of one stream (one generated token through every layer, the LM head
and the sampler).  The device-timed value replays the captured step K times between CUDA events;
the end-to-end value goes through ``Engine.step`` (the public call), which copies the step's token
ids / positions from pinned host memory and reads the sampled token back, every step.  Every timed
loop of K steps is repeated (``--reps``) and the median repetition is reported, with min and max.

The published comparison point is the reference's 131.8 tok/s (4x GB10, TP4, speculation on).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

BASELINE_DECODE_TOK_S = 131.8       # README.md:59 of the reference
BASELINE_16STREAM_TOK_S = 304.0     # docs/performance.md:76-90
BASELINE_PREFILL_TOK_S = 6400.0     # docs/performance.md:573-577
BASELINE_STREAMS = {2: 175.0, 4: 224.0, 8: 270.0, 16: 304.0}      # aggregate tok/s, docs/performance.md:76-90
BASELINE_T1_TOK_S = 80.0            # README.md:60 (temperature 1.0, thinking on)
BASELINE_208K_TOK_S = 56.0          # docs/performance.md:580-581


def reference_arm() -> None:
    # The reference is 23 Rust crates plus sm_121a-only CUDA; there is no Python package to install,
    # no cargo/rustc in the image, and its tensor-core kernels do not assemble for sm_100a.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a Rust workspace (no setup.py/pyproject; pip install fails), "
                                     "no cargo/rustc offline, kernels are sm_121a-only mma.sync forms"}))


class ClockSampler:
    def __init__(self, gpu_index: int):
        self.proc = None
        self.path = f"/tmp/sfb_clocks_{os.getpid()}.csv"
        self.idx = gpu_index

    def start(self):
        q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark(self) -> None:
        """Samples written from here on belong to the timed window."""
        try:
            self.f.flush()
            self.skip = sum(1 for _ in open(self.path))
        except Exception:
            self.skip = 0

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = open(self.path).read().splitlines()
        skip = getattr(self, "skip", 0)
        window = "timed regions"
        if len(lines) - skip < 2:      # a run shorter than two sampling periods: fall back to every sample taken under load
            skip, window = 0, "warm-up and timed regions"
        sm, mx, reasons = [], [], set()
        for line in lines[skip:]:
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for nm, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def pick_config(n_gpus: int, args):
    from sparkflash_b200.config import full_config, reduced_config
    if args.experts or args.layers:
        return reduced_config(args.experts or 384, args.layers or 40), True
    if n_gpus >= 4:
        return full_config(), False
    # 307 GB of weights do not fit one or two 180 GB GPUs: keep all 40 layers and every per-token
    # shape (top-6 of width 2304, all projections) and shrink only the resident expert pool.
    return reduced_config(128 if n_gpus == 1 else 256, 40), True


class Bench:
    """Shared plumbing of the timed sections: barriers, device-timed repetitions (max over ranks), decode replays."""

    def __init__(self, args, world: int, rank: int, local: int):
        import torch
        self.torch = torch
        self.args, self.world, self.rank, self.local = args, world, rank, local
        self.dev = torch.device("cuda", local)

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, xs: list[float]) -> list[float]:
        if self.world == 1:
            return xs
        import torch.distributed as dist
        t = self.torch.tensor(xs, dtype=self.torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed(self, fn, reps: int) -> list[float]:
        """``fn()`` runs one timed loop; returns the device time in ms of every repetition (max over ranks)."""
        torch = self.torch
        out = []
        for _ in range(reps):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            ev0.record()
            fn()
            ev1.record()
            self.barrier()
            out.append(ev0.elapsed_time(ev1))
        return self.max_over_ranks(out)

    @staticmethod
    def stats(ms: list[float], tokens_per_rep: float) -> dict:
        med = statistics.median(ms)
        return {"tok_s": tokens_per_rep / (med / 1e3), "ms_per_step_median": None, "rep_ms_median": med, "rep_ms_min": min(ms),
                "rep_ms_max": max(ms), "reps": len(ms)}

    def replay(self, eng, rows: int, steps: int, bucket: int) -> None:
        """``steps`` replays of the captured rows step; tokens and positions advance on the device."""
        one = self._one(eng)
        for _ in range(steps):
            eng.tokens[:rows].copy_(eng.tokens_out[:rows])
            eng.run_rows(rows, bucket)
            eng.row_pos[:rows].add_(one)

    def _one(self, eng):
        if not hasattr(self, "_one_t"):
            self._one_t = self.torch.ones((), dtype=self.torch.int32, device=eng.dev)
        return self._one_t


def make_engine(B: Bench, weights, lanes: int, max_ctx: int, max_rows: int, drafter: bool = False, pin_bucket: bool = True):
    from sparkflash_b200.models.deepseek_v41 import engine as E
    comm = None
    if B.world > 1:
        from sparkflash_b200.parallel import comm as PC
        comm = PC.make_comm(B.args.collective, B.rank, B.world)
    eng = E.Engine(weights, max_lanes=lanes, max_context=max_ctx, max_rows=max_rows, comm=comm, arm=B.args.arm,
                   synthetic_scales=True, drafter=drafter)
    if comm is not None:
        comm.attach(eng)
    if pin_bucket:
        pin_context_bucket(eng, max_ctx)
    return eng


def pin_context_bucket(eng, max_ctx: int) -> None:
    """One context bucket for a whole decode section: no graph is captured inside a timed loop."""
    b = 1024
    while b < max_ctx:
        b *= 2
    eng.min_bucket = b


def prefill(eng, prompt: list[int], lane: int, chunk: int, skip_decoder: bool = False) -> int:
    """The prompt through ``Engine.step`` in chunks of rows (token ids from pinned host memory every chunk; only the
    last chunk is sampled, on its last row, and read back).  ``skip_decoder``: chunks that end more than the decoder
    tail before the prompt's end run the layers up to the last cache owner only."""
    pos, nxt = 0, 0
    total = len(prompt)
    while pos < total:
        c = prompt[pos:pos + chunk]
        end = pos + len(c)
        last = end >= total
        rows = list(range(pos, end))
        if skip_decoder and not last and total - end >= eng.decoder_tail:
            eng.step(c, [lane] * len(c), rows, skip_decoder=True, sync=False)
        else:
            r = eng.step(c, [lane] * len(c), rows, head="last" if last else False, sync=last)
            if last:
                nxt = int(r[len(c) - 1])
        pos = end
    return nxt


def phase_main(B: Bench, weights, cfg, extras: dict):
    """Prefill of the long prompt, the headline single-stream decode, temperature 1.0, and 4 / 8 / 16 streams."""
    torch, args = B.torch, B.args
    S = max(16, args.streams)
    chunk = args.prefill_chunk
    max_ctx = max(args.prefill_prompt, args.prompt) + chunk + 4096 + args.steps * args.reps * 4
    eng = make_engine(B, weights, S, max_ctx, max(64, chunk), pin_bucket=False)
    gen = torch.Generator().manual_seed(1234)
    out = {"eng": eng}

    # ---- prefill of the long prompt -----------------------------------------------------------------------
    if not args.skip_extras and args.prefill_prompt > 0:
        long_prompt = torch.randint(0, cfg.vocab_size, (args.prefill_prompt,), generator=gen).tolist()
        for skip in (False, True):
            key = "prefill_decoder_skip" if skip else "prefill"
            try:
                prefill(eng, long_prompt, S - 1 - int(skip), chunk, skip)           # captures every graph of the pass
                ms = B.timed(lambda: prefill(eng, long_prompt, 0, chunk, skip), max(1, args.prefill_reps))
                med = statistics.median(ms)
                extras[f"{key}_tok_s"] = len(long_prompt) / (med / 1e3)
                extras[f"{key}_ms"] = {"median": med, "min": min(ms), "max": max(ms), "reps": len(ms)}
                extras[f"vs_baseline_{key}"] = extras[f"{key}_tok_s"] / BASELINE_PREFILL_TOK_S
            except Exception as e:      # an extra never takes the headline down with it
                extras[f"{key}_error"] = f"{type(e).__name__}: {e}"[:300]
        extras["prefill_prompt_tokens"] = len(long_prompt)
        extras["prefill_chunk_rows"] = chunk
        extras["prefill_note"] = ("through Engine.step, chunk by chunk: token ids copied from pinned host memory every chunk, the last row "
                                  "sampled and read back; tcgen05 projections, attention, indexer scores and grouped experts; "
                                  "'prefill' runs every layer on every row, 'prefill_decoder_skip' runs the layers past the last cache "
                                  "owner only on the prompt's tail (the reference's policy)")
        extras["prefill_decoder_tail_rows"] = eng.decoder_tail
        eng.check_status()

    # ---- headline: single-stream decode after a 2,048-token prompt ------------------------------------------
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=gen).tolist()
    pin_context_bucket(eng, max_ctx)
    nxt = prefill(eng, prompt, 1, chunk)
    pos = len(prompt)
    for _ in range(args.warmup):
        r = eng.step([nxt], [1], [pos]); nxt = int(r[0]); pos += 1
    out["launches"] = eng.launches_per_step
    bucket = eng._bucket(max_ctx - 1)
    B.sampler.mark()
    dev_ms = B.timed(lambda: B.replay(eng, 1, args.steps, bucket), args.reps)
    pos += args.steps * args.reps
    nxt = int(eng.tokens_out[0])
    # end to end: the public call; per step H2D of (token, lane, position, temperature, seed) from pinned memory and D2H of
    # the sampled token
    state = {"nxt": nxt, "pos": pos}

    def e2e_loop():
        for _ in range(args.steps):
            r = eng.step([state["nxt"]], [1], [state["pos"]]); state["nxt"] = int(r[0]); state["pos"] += 1
    t0 = time.perf_counter()
    e2e_ms = B.timed(e2e_loop, args.reps)
    out["wall_ms_per_step"] = (time.perf_counter() - t0) * 1e3 / (args.steps * args.reps)
    out["dev_ms"], out["e2e_ms"] = dev_ms, e2e_ms
    out["h2d"], out["d2h"] = eng.h2d_bytes(1), eng.d2h_bytes(1)
    out["clocks"] = B.sampler.stop()
    eng.check_status()
    if args.skip_extras:
        return out

    # ---- temperature 1.0 (Gumbel-max sampling in the head's sampler kernel) ---------------------------------------
    try:
        nxt, pos = state["nxt"], state["pos"]
        for _ in range(args.warmup):
            r = eng.step([nxt], [1], [pos], temperature=[1.0], seeds=[7]); nxt = int(r[0]); pos += 1
        ms = B.timed(lambda: B.replay(eng, 1, args.steps, bucket), args.reps)
        pos += args.steps * args.reps
        med = statistics.median(ms)
        extras["decode_temperature_1_tok_s"] = args.steps / (med / 1e3)
        extras["decode_temperature_1_ms_per_step"] = med / args.steps
        extras["vs_baseline_temperature_1"] = extras["decode_temperature_1_tok_s"] / BASELINE_T1_TOK_S
    except Exception as e:
        extras["decode_temperature_1_error"] = f"{type(e).__name__}: {e}"[:300]

    # ---- 4 / 8 / 16 streams (one row per stream per step) --------------------------------------------------------
    try:
        streams_section(B, eng, cfg, extras, gen, "decode", max_ctx, prompt_lens=None)
    except Exception as e:
        extras["decode_streams_error"] = f"{type(e).__name__}: {e}"[:300]
    eng.check_status()
    return out


def streams_section(B: Bench, eng, cfg, extras: dict, gen, prefix: str, max_ctx: int, prompt_lens) -> None:
    """Decode at 4, 8 and 16 concurrent streams: device-timed replays and end-to-end steps.  ``prompt_lens``: per-stream
    prompt lengths to prefill first (None = 64 tokens each)."""
    torch, args = B.torch, B.args
    S = 16
    chunk = args.prefill_chunk
    lens = prompt_lens or [64] * S
    for s in range(S):
        p = torch.randint(0, cfg.vocab_size, (lens[s],), generator=gen).tolist()
        prefill(eng, p, s, chunk)
    pin_context_bucket(eng, max_ctx)
    bucket = eng._bucket(max_ctx - 1)
    for n_s in (4, 8, 16):
        toks = torch.randint(0, cfg.vocab_size, (n_s,), generator=gen).tolist()
        pos = [lens[s] for s in range(n_s)]
        for _ in range(args.warmup):
            r = eng.step(toks, list(range(n_s)), pos); toks = [int(x) for x in r]; pos = [p + 1 for p in pos]
        ms = B.timed(lambda: B.replay(eng, n_s, args.steps, bucket), args.reps)
        pos = [p + args.steps * args.reps for p in pos]
        toks = [int(x) for x in eng.tokens_out[:n_s].tolist()]
        st = {"toks": toks, "pos": pos}

        def e2e_loop():
            for _ in range(args.steps):
                r = eng.step(st["toks"], list(range(n_s)), st["pos"]); st["toks"] = [int(x) for x in r]; st["pos"] = [p + 1 for p in st["pos"]]
        ems = B.timed(e2e_loop, max(1, args.reps // 2))
        for i in range(n_s):
            lens[i] = st["pos"][i]
        med, emed = statistics.median(ms), statistics.median(ems)
        extras[f"{prefix}_{n_s}streams_aggregate_tok_s"] = n_s * args.steps / (med / 1e3)
        extras[f"{prefix}_{n_s}streams_per_stream_tok_s"] = args.steps / (med / 1e3)
        extras[f"{prefix}_{n_s}streams_ms_per_step"] = med / args.steps
        extras[f"{prefix}_{n_s}streams_e2e_aggregate_tok_s"] = n_s * args.steps / (emed / 1e3)
        extras[f"vs_baseline_{prefix}_{n_s}streams"] = n_s * args.steps / (med / 1e3) / BASELINE_STREAMS[n_s]
    extras[f"{prefix}_streams_e2e_h2d_bytes_per_step_16"] = eng.h2d_bytes(16)
    extras[f"{prefix}_streams_e2e_d2h_bytes_per_step_16"] = eng.d2h_bytes(16)


def phase_mtp(B: Bench, cfg, extras: dict) -> None:
    """DSpark draft stages on: per-forward latency with speculation off (one row per forward, draft rings seeded) and on
    (draft block + verify rows).  Acceptance is meaningless with random weights, so latencies are the result."""
    torch, args = B.torch, B.args
    from sparkflash_b200.models.deepseek_v41 import prepare as P
    weights = P.prepare_synthetic(cfg, B.rank, B.world, device=f"cuda:{B.local}", seed=0, moe_mode="tp", mtp=True)
    max_ctx = args.prompt + 4096 + args.steps * args.reps * 8
    eng = make_engine(B, weights, 2, max_ctx, 64, drafter=True)
    try:
        gen = torch.Generator().manual_seed(99)
        prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=gen).tolist()
        nxt = prefill(eng, prompt, 0, 64)
        pos = len(prompt)
        st = {"nxt": nxt, "pos": pos}
        for temp, label in ((0.0, "greedy"), (1.0, "temperature_1")):
            def off_loop():
                for _ in range(args.steps):
                    r = eng.step([st["nxt"]], [0], [st["pos"]], temperature=[temp], seeds=[5]); st["nxt"] = int(r[0]); st["pos"] += 1
            off_loop()
            ms = B.timed(off_loop, max(3, args.reps // 2))
            extras[f"mtp_off_{label}_ms_per_forward"] = statistics.median(ms) / args.steps
            extras[f"mtp_off_{label}_tok_s"] = args.steps / (statistics.median(ms) / 1e3)
            depth = min(4, cfg.dspark_block - 1)
            acc = {"emitted": 0, "accepted": 0, "forwards": 0}

            def on_loop():
                for _ in range(args.steps):
                    drafts, _conf = eng.draft(0, st["pos"] - 1, st["nxt"], temperature=temp, seed=5)
                    rows = [st["nxt"]] + drafts[:depth]
                    o = eng.step(rows, [0] * len(rows), list(range(st["pos"], st["pos"] + len(rows))), temperature=[temp] * len(rows),
                                 seeds=[5] * len(rows))
                    a = 0
                    while a < depth and int(o[a]) == rows[a + 1]:
                        a += 1
                    st["nxt"], st["pos"] = int(o[a]), st["pos"] + a + 1
                    acc["emitted"] += a + 1; acc["accepted"] += a; acc["forwards"] += 1
            on_loop()
            acc.update(emitted=0, accepted=0, forwards=0)
            ms = B.timed(on_loop, max(3, args.reps // 2))
            med = statistics.median(ms)
            extras[f"mtp_on_{label}_ms_per_forward"] = med / args.steps
            extras[f"mtp_on_{label}_tok_s"] = (acc["emitted"] / max(1, acc["forwards"])) * args.steps / (med / 1e3)
            extras[f"mtp_on_{label}_accepted_per_forward"] = acc["accepted"] / max(1, acc["forwards"])
        extras["mtp_draft_depth"] = depth
        extras["mtp_note"] = ("random weights: the draft stages predict nothing, so accepted_per_forward is the floor and mtp_on tok/s is the "
                              "cost of speculation when it never pays; tokens per second at acceptance a scale as (1 + a) / forward time")
        eng.check_status()
    finally:
        eng.close()
        del eng, weights
        release(torch)


def phase_long(B: Bench, weights, cfg, extras: dict) -> None:
    """Decode against a long cached context: the caches of lane 0 are filled with random codes (a real prefill of a million
    tokens is out of a benchmark's time); every kernel of the step then runs at that context length."""
    torch, args = B.torch, B.args
    ctxs = [int(x) for x in args.long_context.split(",") if x]
    if not ctxs:
        return
    top = max(ctxs) + args.steps * (args.reps + 2) + args.warmup + 64
    eng = make_engine(B, weights, 1, top, 16, pin_bucket=False)
    try:
        g2 = torch.Generator(device=eng.dev).manual_seed(7)
        for dct in (eng.kv.win_q, eng.kv.ckv_q, eng.kv.ik_q):
            for t in dct.values():
                t[0].copy_(torch.randint(0, 120, t[0].shape, dtype=torch.uint8, device=eng.dev, generator=g2))
        for dct, code in ((eng.kv.win_s, 122), (eng.kv.ckv_s, 0x38), (eng.kv.ik_s, 122)):
            for t in dct.values():
                t[0].fill_(code)
        for ctx in ctxs:
            p_l, tok_l = ctx, 1
            pin_context_bucket(eng, ctx + args.steps * (args.reps + 2) + args.warmup + 8)
            for _ in range(args.warmup):
                r = eng.step([tok_l], [0], [p_l]); tok_l = int(r[0]); p_l += 1
            bucket = eng.min_bucket
            reps = max(3, args.reps // 2)
            ms = B.timed(lambda: B.replay(eng, 1, args.steps, bucket), reps)
            p_l += args.steps * reps
            st = {"t": int(eng.tokens_out[0]), "p": p_l}

            def e2e_loop():
                for _ in range(args.steps):
                    r = eng.step([st["t"]], [0], [st["p"]]); st["t"] = int(r[0]); st["p"] += 1
            ems = B.timed(e2e_loop, 2)
            med = statistics.median(ms)
            extras[f"decode_tok_s_at_context_{ctx}"] = args.steps / (med / 1e3)
            extras[f"decode_ms_per_step_at_context_{ctx}"] = med / args.steps
            extras[f"decode_e2e_tok_s_at_context_{ctx}"] = args.steps / (statistics.median(ems) / 1e3)
        extras["long_context_kv_gb_per_gpu"] = eng.kv.nbytes() / 1e9
        extras["long_context_note"] = "KV caches filled with random codes up to the context length; reference: 56.0 tok/s at 208K"
        eng.check_status()
    finally:
        eng.close()
        del eng
        release(torch)


def phase_ep(B: Bench, cfg, extras: dict) -> None:
    """Whole experts per rank (expert parallelism) with tensor-parallel attention: 4 / 8 / 16 streams whose prompts are
    512..4096 tokens long."""
    torch, args = B.torch, B.args
    from sparkflash_b200.models.deepseek_v41 import prepare as P
    weights = P.prepare_synthetic(cfg, B.rank, B.world, device=f"cuda:{B.local}", seed=0, moe_mode="ep")
    chunk = args.prefill_chunk
    max_ctx = 4096 + chunk + args.steps * args.reps * 6 + 1024
    eng = make_engine(B, weights, 16, max_ctx, max(64, chunk), pin_bucket=False)
    try:
        gen = torch.Generator().manual_seed(4321)
        lens = torch.randint(512, 4097, (16,), generator=gen).tolist()
        streams_section(B, eng, cfg, extras, gen, "ep_decode", max_ctx, prompt_lens=lens)
        extras["ep_prompt_lengths"] = lens
        extras["ep_parallelism"] = f"tp{B.world} attention + ep{B.world} experts ({cfg.n_routed_experts // B.world} whole experts per rank)"
        eng.check_status()
    finally:
        eng.close()
        del eng, weights
        release(torch)


def release(torch) -> None:
    """Give a finished section's device memory back: engines and communicators reference each other, so the cycle
    collector runs before the caching allocator is emptied."""
    import gc
    gc.collect()
    torch.cuda.empty_cache()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--reps", type=int, default=10, help="repetitions of every timed loop of --steps steps (the median is reported)")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--prefill-prompt", type=int, default=32768, help="tokens of the long prompt of the prefill figure")
    ap.add_argument("--prefill-reps", type=int, default=2)
    ap.add_argument("--streams", type=int, default=16)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--collective", default=os.environ.get("SFB_COLLECTIVE", "fused"))
    ap.add_argument("--skip-extras", action="store_true")
    ap.add_argument("--arm", default=os.environ.get("SFB_ARM", "tc"), choices=["tc", "cuda"])
    ap.add_argument("--long-context", default="131072,1048576", help="comma-separated cached context lengths: decode tok/s with the KV "
                    "caches of lane 0 filled with random entries up to that position ('' = skip)")
    ap.add_argument("--prefill-chunk", type=int, default=4096, help="rows per prompt chunk (the reference prefills 4,096-row chunks)")
    ap.add_argument("--no-mtp", action="store_true", help="skip the DSpark draft-path section")
    ap.add_argument("--no-ep", action="store_true", help="skip the expert-parallel section (2+ GPUs)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    args.warmup = max(args.warmup, 3)
    args.reps = max(args.reps, 1)

    import torch
    import torch.distributed as dist
    from sparkflash_b200.models.deepseek_v41 import prepare as P

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    B = Bench(args, world, rank, local)
    B.sampler = ClockSampler(local)
    B.sampler.start()                 # started early: nvidia-smi needs a second to come up on a multi-GPU box

    cfg, reduced = pick_config(world, args)
    t0 = time.time()
    weights = P.prepare_synthetic(cfg, rank, world, device=f"cuda:{local}", seed=0, moe_mode="tp")
    torch.cuda.synchronize()
    t_init = time.time() - t0
    extras: dict = {}
    main_out = phase_main(B, weights, cfg, extras)
    eng = main_out.pop("eng")
    weights_gb, kv_gb = weights.nbytes() / 1e9, eng.kv.nbytes() / 1e9
    eng.close()
    del eng
    release(torch)
    if not args.skip_extras:
        try:
            phase_long(B, weights, cfg, extras)
        except Exception as e:
            extras["long_context_error"] = f"{type(e).__name__}: {e}"[:300]
    del weights
    release(torch)
    if not args.skip_extras:
        if not args.no_mtp and cfg.n_mtp_stages:
            try:
                phase_mtp(B, cfg, extras)
            except Exception as e:
                extras["mtp_error"] = f"{type(e).__name__}: {e}"[:300]
        if world > 1 and not args.no_ep:
            try:
                phase_ep(B, cfg, extras)
            except Exception as e:
                extras["ep_error"] = f"{type(e).__name__}: {e}"[:300]

    dev_ms, e2e_ms = main_out["dev_ms"], main_out["e2e_ms"]
    dev_med, e2e_med = statistics.median(dev_ms), statistics.median(e2e_ms)
    value = args.steps / (dev_med / 1e3)
    e2e_value = args.steps / (e2e_med / 1e3)
    launches = main_out["launches"]
    if rank == 0:
        out = {
            "metric": "decode tok/s, 1 stream (DeepSeek-V4.1-Flash architecture)", "value": value, "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_med / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": value / BASELINE_DECODE_TOK_S,
            "dtype": "mxfp4 experts (W4A8) + mxfp8 dense (W8A8), bf16 residual/norms, fp32 accumulate",
            "data": "synthetic token ids, random-init weights generated on device",
            "impl": "ours",
            "repetitions": {"reps": args.reps, "value_is": "median repetition of --steps steps",
                            "ms_per_step_min": min(dev_ms) / args.steps, "ms_per_step_max": max(dev_ms) / args.steps,
                            "e2e_ms_per_step_min": min(e2e_ms) / args.steps, "e2e_ms_per_step_max": max(e2e_ms) / args.steps},
            "config": {"model": cfg.name, "layers": cfg.n_layers, "resident_experts": cfg.n_routed_experts,
                       "reduced_expert_pool": reduced, "global_batch": 1, "seq_len": args.prompt,
                       "parallelism": f"tp{world}", "collective": args.collective if world > 1 else "none",
                       "speculation": "off (one token per step)", "sampling": "greedy",
                       "arm": "tcgen05 block-scaled MMA for projections and experts" if args.arm == "tc" else "CUDA-core",
                       "l2": "inputs larger than L2 (every step streams the step's weights, >1 GB per GPU, from HBM)",
                       "weights_gb_per_gpu": weights_gb, "kv_gb_per_gpu": kv_gb, "init_s": t_init},
            "clocks": main_out["clocks"],
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": main_out["h2d"], "d2h_bytes_per_step": main_out["d2h"],
                    "ms_per_step": e2e_med / args.steps, "wall_ms_per_step": main_out["wall_ms_per_step"]},
            "gpu_launches": launches * args.steps,
            "launches_per_step": launches,
            "extra": extras,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
