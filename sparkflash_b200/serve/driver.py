"""The serving loop: scheduler ticks -> rows steps of the device engine -> token events.

One thread owns the engine.  Every tick it (1) applies the inputs of the tick (submissions, cancels) - on
rank 0 taken from the HTTP side and broadcast through the control channel, on the other ranks received
from it - (2) asks the scheduler replica for the plan, (3) runs one rows step, (4) commits the sampled
tokens.  Every rank runs the same deterministic scheduler on the same inputs and samples the same tokens,
so only the inputs travel.  Reference behaviour: crates/sparkflash-cli/src/serve/device.rs (DeviceLink, tick
broadcast), crates/sparkflash-deepseek-forward/src/tp4_forward/batch.rs:15-54 (tick model), :2260-2485
(speculative step: anchors + draft rows verified by one rows step, accepted prefix + bonus token),
docs/serving.md:159-167 (fail-stop on a device error, stall -> 503).

Speculation: a drafter proposes tokens per decoding sequence; the rows step samples at every row with the
stateless (seed, position)-keyed sampler, so a draft is accepted exactly when it equals the token the
previous row sampled - the output is identical with and without speculation.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass, field

from ..sched.core import PHASE_DECODE, PHASE_IDLE, PHASE_PREFILL, Scheduler
from .constrained import Schema, TokenConstraint, TokenVocab
from .engine_api import ApiError, Capabilities, EngineRequest, InferenceEngine


@dataclass
class _Live:
    req: EngineRequest
    seq: int
    loop: asyncio.AbstractEventLoop | None
    out: asyncio.Queue | None
    constraint: TokenConstraint | None = None
    started: bool = False
    t_submit: float = field(default_factory=time.monotonic)
    t_first: float | None = None
    proposed: int = 0
    accepted: int = 0
    verify_steps: int = 0
    generated: int = 0
    history: list[int] = field(default_factory=list)
    choices: list[int] = field(default_factory=list)      # the model's own picks under teacher forcing


class LocalChannel:
    """World of one: the tick inputs stay in this process."""
    rank, world = 0, 1

    def broadcast(self, msg):
        return msg

    def alive(self):
        return True, "ok"

    def close(self):
        pass


class NgramDrafter:
    """Prompt-lookup drafting on the host: propose the continuation of the longest recent n-gram match in the
    sequence's own history.  Serves as the drafter for models without trained draft stages."""

    def __init__(self, depth: int = 4, max_ngram: int = 4):
        self.depth, self.max_ngram = depth, max_ngram

    def propose(self, history: list[int]) -> tuple[list[int], list[float]]:
        n = len(history)
        for k in range(min(self.max_ngram, n - 1), 0, -1):
            tail = history[n - k:]
            for i in range(n - k - 1, -1, -1):
                if history[i:i + k] == tail:
                    cont = history[i + k:i + k + self.depth]
                    if cont:
                        return cont, [float(k)] * len(cont)
        return [], []


class DSparkDrafter:
    """The model's own draft stages on the device (Engine.draft): one block of proposals per decoding sequence and step,
    sampled with the verifier's (seed, position) noise so that a good draft is accepted at any temperature."""
    device = True

    def __init__(self, depth: int = 5, min_confidence: float | None = None, policy=None, passes_of: int = 16):
        """``policy``: a sched.spec.SpecPolicy choosing every sequence's depth from the step-cost model (None keeps every
        proposal up to ``depth``, or up to the first one below ``min_confidence``)."""
        self.depth, self.min_confidence, self.policy, self.passes_of = depth, min_confidence, policy, passes_of

    def _trim(self, toks, conf):
        toks, conf = toks[:self.depth], conf[:self.depth]
        if self.min_confidence is not None:          # stop at the first position the head does not trust
            for i, c in enumerate(conf):
                if c < self.min_confidence:
                    return toks[:i], conf[:i]
        return toks, conf

    def propose_many(self, eng, items):
        """Draft blocks of several sequences in one device pass (Engine.draft_many)."""
        return [self._trim(t, c) for t, c in eng.draft_many(items)]

    def propose_device(self, eng, lane: int, pos: int, anchor: int, temperature: float, seed: int):
        toks, conf = eng.draft(lane, pos, anchor, temperature, seed)
        toks, conf = toks[:self.depth], conf[:self.depth]
        if self.min_confidence is not None:          # adaptive depth: stop at the first position the head does not trust
            for i, c in enumerate(conf):
                if c < self.min_confidence:
                    return toks[:i], conf[:i]
        return toks, conf


class DeviceDriver(InferenceEngine):
    def __init__(self, engine, tokenizer, model_id: str = "deepseek-v4.1-flash", channel=None, drafter=None,
                 max_lanes: int | None = None, queue_depth: int = 64, prefill_chunk: int | None = None,
                 prefix_reuse_min: int = 256, stall_seconds: float = 30.0, eos_id: int | None = None, decoder_skip: bool = True):
        self.engine = engine
        self.tokenizer = tokenizer
        self.model_id = model_id
        self.channel = channel or LocalChannel()
        self.drafter = drafter
        self.max_context = engine.max_context
        self.eos_id = tokenizer.eos_id if eos_id is None else eos_id
        lanes = max_lanes or engine.max_lanes
        chunk = prefill_chunk or engine.max_rows
        self.sched = Scheduler(max_lanes=lanes, queue_depth=queue_depth, max_rows=engine.max_rows, prefill_chunk=chunk,
                               prefill_chunk_busy=chunk, prefix_reuse_min=prefix_reuse_min, max_context=engine.max_context,
                               spec_depth=getattr(drafter, "depth", 0) or 0)
        tail = getattr(engine, "decoder_tail", 0)
        if decoder_skip and tail:
            self.sched.set_decoder_tail(tail)
        ring_slack = getattr(engine, "ring_slack", None)
        if ring_slack is not None:
            self.sched.set_ring_slack(ring_slack)
        self.capabilities = Capabilities(constrained=getattr(engine, "supports_mask", False), speculative=drafter is not None,
                                         vision=getattr(engine, "supports_vision", False))
        self._inbox: queue.Queue = queue.Queue()
        self._live: dict[int, _Live] = {}
        self._by_request: dict[str, int] = {}
        self._next_seq = 1
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = False
        self.failed: str | None = None
        self.stall_seconds = stall_seconds
        self._tick_started: float | None = None
        self.ticks = 0
        self._vocab: TokenVocab | None = None
        self._thread: threading.Thread | None = None

    # ---- InferenceEngine ------------------------------------------------------------------------------
    def start(self) -> "DeviceDriver":
        self._thread = threading.Thread(target=self._loop, name="engine-driver", daemon=True)
        self._thread.start()
        return self

    def shutdown(self, drain_seconds: float = 30.0) -> None:
        t0 = time.monotonic()
        while self._live and time.monotonic() - t0 < drain_seconds and self.failed is None:
            time.sleep(0.01)
        self._stop = True
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        self.channel.close()

    def healthy(self):
        if self.failed:
            return False, self.failed
        t = self._tick_started
        if t is not None and time.monotonic() - t > self.stall_seconds:
            return False, f"tick running for more than {self.stall_seconds:.0f}s"
        ok, why = self.channel.alive()
        if not ok:
            return False, why
        return True, "ok"

    def stats(self):
        st = self.sched.stats()
        return {"running": st["running"], "waiting": st["waiting"], "free_lanes": st["free_lanes"], "ticks": self.ticks,
                "prefix_hits": st["prefix_hits"], "prefix_rows": st["prefix_rows"], "preemptions": st["preemptions"]}

    def vocab(self) -> TokenVocab:
        if self._vocab is None:
            self._vocab = TokenVocab(self.tokenizer.token_bytes())
        return self._vocab

    def validate(self, req: EngineRequest) -> None:
        super().validate(req)
        if (req.top_p < 1.0 or req.top_k > 0) and not getattr(self.engine, "supports_filter", False):
            raise ApiError(400, "top_p / top_k need the candidate filter, which this engine build does not have",
                           "unsupported_parameter", "top_p")

    async def generate(self, req: EngineRequest):
        if self.failed:
            yield ("error", self.failed, "engine_failed"); return
        loop = asyncio.get_running_loop()
        out: asyncio.Queue = asyncio.Queue()
        with self._lock:
            seq = self._next_seq
            self._next_seq += 1
        live = _Live(req, seq, loop, out)
        self._inbox.put(("submit", live))
        self._wake.set()
        try:
            while True:
                ev = await out.get()
                yield ev
                if ev[0] in ("finished", "error"):
                    return
        finally:
            if seq in self._live:
                self._inbox.put(("cancel", seq))
                self._wake.set()

    def cancel(self, request_id: str) -> None:
        seq = self._by_request.get(request_id)
        if seq is not None:
            self._inbox.put(("cancel", seq))
            self._wake.set()

    # ---- the engine thread --------------------------------------------------------------------------------
    def _emit(self, live: _Live, ev: tuple) -> None:
        if live.loop is not None:
            live.loop.call_soon_threadsafe(live.out.put_nowait, ev)

    def _fail(self, why: str) -> None:
        self.failed = why
        for live in list(self._live.values()):
            self._emit(live, ("error", why, "engine_failed"))
        self._live.clear()

    def _take_inputs(self) -> dict:
        subs, cancels = [], []
        while True:
            try:
                kind, x = self._inbox.get_nowait()
            except queue.Empty:
                break
            if kind == "submit":
                subs.append(x)
            else:
                cancels.append(x)
        return {"subs": subs, "cancels": cancels}

    def _apply_inputs(self, msg: dict) -> None:
        for live in msg["subs"]:
            r = live.req
            rc = self.sched.submit(live.seq, r.prompt_tokens, r.max_tokens)
            if rc == 1:
                self._emit(live, ("error", "all lanes busy and the queue is full", "overloaded")); continue
            if rc == 2:
                self._emit(live, ("error", "prompt does not fit the context", "context_length_exceeded")); continue
            if r.constraint is not None:
                live.constraint = TokenConstraint(Schema(r.constraint), self.vocab(), self.eos_id)
            live.history = list(r.prompt_tokens)
            self._live[live.seq] = live
            self._by_request[r.request_id] = live.seq
        for seq in msg["cancels"]:
            live = self._live.pop(seq, None)
            if live is not None:
                self._by_request.pop(live.req.request_id, None)
            self.sched.cancel(seq)

    def _loop(self) -> None:
        try:
            # CUDA's current device is per thread and starts at device 0: this thread must select the engine's GPU before
            # its first launch, or rank r > 0 would launch on GPU 0 with pointers into GPU r's memory
            dev = getattr(self.engine, "dev", None)
            if dev is not None and getattr(dev, "type", None) == "cuda":
                import torch
                torch.cuda.set_device(dev)
            while not self._stop:
                inputs = self._take_inputs() if self.channel.rank == 0 else None
                # followers block here for rank 0's message; rank 0 sends one per tick
                if self.channel.world > 1:
                    inputs = self.channel.broadcast(self._wire(inputs) if inputs is not None else None)
                    inputs = self._unwire(inputs)
                self._apply_inputs(inputs)
                if not self._tick():
                    self._wake.wait(0.02)
                    self._wake.clear()
        except Exception as e:      # fail-stop: a device error ends serving, it is never retried
            self._fail(f"{type(e).__name__}: {e}")

    def _wire(self, inputs: dict) -> dict:
        """What travels to the followers: sequence numbers and requests, nothing tied to this process's event loop."""
        self._local_subs = inputs["subs"]
        return {"subs": [(l.seq, l.req) for l in inputs["subs"]], "cancels": list(inputs["cancels"])}

    def _unwire(self, msg: dict) -> dict:
        if self.channel.rank == 0:
            return {"subs": self._local_subs, "cancels": msg["cancels"]}
        return {"subs": [_Live(req, seq, None, None) for seq, req in msg["subs"]], "cancels": msg["cancels"]}

    def _collect_drafts(self) -> None:
        """Drafts of every decoding sequence for the coming step.  The device drafter runs the sequences' blocks in passes of
        several sequences each; the depth policy then keeps, per sequence, the prefix of drafts that raises the shared verify
        step's expected tokens per millisecond (anchors come first, then the likeliest drafts)."""
        eng = self.engine
        cand = []
        for live in self._live.values():
            info = self.sched.info(live.seq)
            if info and info["state"] == "decode" and live.constraint is None:
                cand.append((live, info))
        if not cand:
            return
        proposals: list[tuple] = []
        if getattr(self.drafter, "device", False):
            items = []
            for live, info in cand:
                q = live.req
                seed = (q.seed if q.seed is not None else live.seq * 0x9E3779B1) & 0x7FFFFFFFFFFFFFFF
                items.append((info["lane"], info["computed"] - 1, live.history[-1], 0.0 if q.temperature < 1e-5 else q.temperature, seed))
            per_pass = max(1, min(getattr(self.drafter, "passes_of", 16), eng.max_rows // max(1, eng.cfg.dspark_block)))
            out = []
            for p0 in range(0, len(items), per_pass):
                out += self.drafter.propose_many(eng, items[p0:p0 + per_pass])
            proposals = [(live, toks, conf) for (live, _), (toks, conf) in zip(cand, out)]
        else:
            proposals = [(live, *self.drafter.propose(live.history)) for live, _ in cand]
        policy = getattr(self.drafter, "policy", None)
        if policy is not None and proposals:
            from ..sched.spec import calibrate
            # more decoding sequences than half a step's rows take plain rows (the scheduler's rule): nothing to allocate then
            if len(proposals) <= policy.max_rows:
                alloc = policy.allocate([[calibrate(c) for c in conf] for _, _, conf in proposals])
                proposals = [(live, toks[:k], conf[:k]) for (live, toks, conf), k in zip(proposals, alloc.keep)]
                self.last_allocation = alloc
        for live, toks, conf in proposals:
            if toks:
                self.sched.set_drafts(live.seq, toks, conf)

    def _tick(self) -> bool:
        eng = self.engine
        # drafts for the coming decode step
        if self.drafter is not None:
            self._collect_drafts()
        phase, rows = self.sched.tick(eng.max_rows)
        if phase == PHASE_IDLE or not rows:
            return False
        self._tick_started = time.monotonic()
        temps, seeds = [], []
        for r in rows:
            q = self._live[r.seq].req
            temps.append(0.0 if q.temperature < 1e-5 else q.temperature)
            seeds.append((q.seed if q.seed is not None else r.seq * 0x9E3779B1) & 0x7FFFFFFFFFFFFFFF)
        # logit masks of constrained sequences: one row each (constrained sequences are never drafted)
        masks = {}
        for i, r in enumerate(rows):
            live = self._live[r.seq]
            last_of_seq = i + 1 == len(rows) or rows[i + 1].seq != r.seq
            if live.constraint is not None and last_of_seq and (phase == PHASE_DECODE or self._prefill_completes(live, rows)):
                lo, hi = eng.vocab_slice()
                n_ok, words = live.constraint.mask(lo, hi)
                total = n_ok if self.channel.world == 1 else None
                masks[i] = words
                if total == 0:
                    self._finish(live, None, error=("the constraint admits no token", "constraint_dead_end"))
                    return True
        image_rows = {}
        for i, r in enumerate(rows):
            for sp in self._live[r.seq].req.vision:
                k = r.pos - sp.start
                if 0 <= k < sp.embeddings.shape[0]:
                    image_rows[i] = sp.embeddings[k]
        kw = {"masks": masks} if masks or getattr(eng, "supports_mask", False) else {}
        if image_rows or getattr(eng, "supports_vision", False):
            kw["image_rows"] = image_rows
        filters = {}
        for i, r in enumerate(rows):
            q = self._live[r.seq].req
            if (q.top_p < 1.0 or q.top_k > 0) and q.temperature >= 1e-5:
                filters[i] = (q.top_k, q.top_p)
        if filters:
            kw["filters"] = filters
        if rows[0].kind == 3:
            kw["skip_decoder"] = True
        elif phase == PHASE_PREFILL and getattr(eng, "supports_headless", False) and not any(
                self._prefill_completes(self._live[r.seq], rows) for r in rows):
            kw["head"] = False           # no row of this chunk is sampled: skip the vocabulary projection
        out = eng.step([r.token for r in rows], [r.lane for r in rows], [r.pos for r in rows], temps, seeds, **kw)
        out = [int(x) for x in out]
        eng.check_status()
        self.ticks += 1
        # commit per sequence
        i = 0
        while i < len(rows):
            j = i
            while j + 1 < len(rows) and rows[j + 1].seq == rows[i].seq:
                j += 1
            live = self._live.get(rows[i].seq)
            if live is not None:
                if phase == PHASE_PREFILL:
                    self._commit_prefill(live, rows[i:j + 1], out[i:j + 1])
                else:
                    self._commit_decode(live, rows[i:j + 1], out[i:j + 1])
            i = j + 1
        self._tick_started = None
        return True

    def _prefill_completes(self, live: _Live, rows) -> bool:
        last = max(r.pos for r in rows if r.seq == live.seq)
        return last + 1 >= len(live.req.prompt_tokens)

    def _start(self, live: _Live) -> None:
        if not live.started:
            live.started = True
            info = self.sched.info(live.seq)
            cached = 0
            if info is not None:
                cached = getattr(live, "_cached", 0)
            self._emit(live, ("started", len(live.req.prompt_tokens), cached))

    def _force(self, live: _Live, index: int, sampled: int) -> int:
        """Teacher forcing: remember the model's own choice for generation index ``index`` and emit the forced token."""
        f = live.req.forced_tokens
        if not f:
            return sampled
        live.choices.append(int(sampled))
        return f[index] if index < len(f) else sampled

    def _commit_prefill(self, live: _Live, rows, out) -> None:
        if not live.started:
            live._cached = rows[0].pos if rows[0].pos > 0 else 0
            self._start(live)
        done = rows[-1].pos + 1 >= len(live.req.prompt_tokens)
        new = [self._force(live, 0, out[-1])] if done else []
        fin = self.sched.commit(live.seq, len(rows), new, self.eos_id)
        if done:
            self._deliver(live, new, fin)

    def _commit_decode(self, live: _Live, rows, out) -> None:
        self._start(live)
        # row 0 is the anchor; rows 1.. are drafts: draft k is accepted when it equals the token sampled at row k-1
        # (under teacher forcing the token that is fed next is the forced one, so that is what a draft has to match)
        accepted = 0
        drafts = rows[1:]
        new = []
        base = live.generated
        while True:
            t = self._force(live, base + accepted, out[accepted])
            new.append(t)
            if accepted < len(drafts) and drafts[accepted].token == t:
                accepted += 1
            else:
                break
        if drafts:
            live.proposed += len(drafts); live.accepted += accepted; live.verify_steps += 1
        # end-of-sequence inside the accepted run cuts it there
        for k, t in enumerate(new):
            if t == self.eos_id:
                new = new[:k + 1]
                break
        fin = self.sched.commit(live.seq, min(1 + accepted, len(new)), new, self.eos_id)
        self._deliver(live, new, fin)

    def _deliver(self, live: _Live, new: list[int], fin: int) -> None:
        reason = None
        for t in new:
            if live.constraint is not None and not live.constraint.advance(t):
                self._finish(live, None, error=("the sampled token left the constraint", "constraint_violation"))
                return
            if t == self.eos_id:
                reason = "stop"
                break
            live.history.append(t)
            live.generated += 1
            if live.t_first is None:
                live.t_first = time.monotonic()
            self._emit(live, ("token", t))
        if fin == 1 or reason is not None:
            self._finish(live, reason or "length")

    def _finish(self, live: _Live, reason, error=None) -> None:
        self._live.pop(live.seq, None)
        self._by_request.pop(live.req.request_id, None)
        if error is not None:
            self.sched.cancel(live.seq)
            self._emit(live, ("error", error[0], error[1]))
            return
        self.sched.release(live.seq)
        dt = max(1e-9, time.monotonic() - (live.t_first or live.t_submit))
        stats = {"decode_tokens": live.generated, "proposed": live.proposed, "accepted": live.accepted,
                 "verify_steps": live.verify_steps, "decode_tok_s": live.generated / dt}
        if live.req.forced_tokens:
            stats["model_choices"] = list(live.choices[:live.generated])
        self._emit(live, ("finished", reason, stats))


class FakeRowsEngine:
    """A stand-in with the rows-step contract of the device engine and a real notion of cached state: the
    'model' hashes the lane's token history up to each row, so a wrong position, a stale lane or a broken
    prefix reuse changes the output.  Used by the CPU tests of the driver."""

    supports_mask = True

    def __init__(self, vocab_size: int = 300, max_lanes: int = 4, max_context: int = 512, max_rows: int = 16, eos_id: int = 257,
                 eos_after: int | None = None, cycle: list[int] | None = None):
        self.vocab_size, self.max_lanes, self.max_context, self.max_rows = vocab_size, max_lanes, max_context, max_rows
        self.lane_tokens = [[0] * max_context for _ in range(max_lanes)]
        self.eos_id, self.eos_after, self.cycle = eos_id, eos_after, cycle
        self.steps: list[int] = []
        self.status_error: str | None = None
        self.ring_slack = 64
        self.supports_vision = True
        self.image_log: list[tuple] = []
        self.filter_log: list[tuple] = []
        self.skipped_rows = 0
        self.decoder_tail = 0
        self.supports_filter = True

    def vocab_slice(self):
        return 0, self.vocab_size

    def check_status(self):
        if self.status_error:
            raise RuntimeError(self.status_error)

    def _next(self, lane: int, pos: int) -> int:
        h = 1469598103934665603
        for t in self.lane_tokens[lane][:pos + 1]:
            h = ((h ^ t) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        if self.cycle:
            return self.cycle[pos % len(self.cycle)]
        if self.eos_after is not None and pos >= self.eos_after:
            return self.eos_id
        return 32 + h % 90      # printable bytes

    def step(self, tokens, lanes, positions, temperature=None, seeds=None, masks=None, image_rows=None, filters=None, skip_decoder=False):
        self.steps.append(len(tokens))
        self.skipped_rows += len(tokens) if skip_decoder else 0
        self.filter_log += [(positions[i], f) for i, f in (filters or {}).items()]
        for i, vec in (image_rows or {}).items():
            self.image_log.append((lanes[i], positions[i], float(vec.float().sum())))
        out = []
        for i, (t, l, p) in enumerate(zip(tokens, lanes, positions)):
            self.lane_tokens[l][p] = t
            nxt = self._next(l, p)
            if masks and i in masks:
                words = masks[i]
                ok = lambda x: bool((int(words[x >> 6]) >> (x & 63)) & 1)
                if not ok(nxt):
                    prefer = [self.eos_id] + [ord(c) for c in '"}]:,'] + list(range(self.vocab_size))
                    nxt = next(x for x in prefer if x < self.vocab_size and ok(x))
            out.append(nxt)
        return out
