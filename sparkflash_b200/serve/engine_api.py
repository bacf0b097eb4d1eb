"""The seam between the HTTP surface and an engine.

An engine consumes ``EngineRequest`` objects and yields raw events (started / token / finished / error);
``Generation`` turns token ids into API-level deltas (detokenise -> stop strings -> reasoning split -> tool
calls -> loop detector).  ``MockEngine`` is the scripted engine of the API tests; the real engine driver is
serve/driver.py.  Reference: crates/sparkflash-api/src/engine.rs:287-403 (request and event types), :686-755
(capabilities and validation), mock engine of crates/sparkflash-api/tests/router.rs.
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Callable

from .constrained import Schema, SchemaError, TokenConstraint, TokenVocab
from .reasoning import LoopAbortDetector, ReasoningSplitter, StopStrings
from .tokenizer import StreamDecoder
from .tool_parser import DsmlToolParser, XmlToolParser


class ApiError(Exception):
    def __init__(self, status: int, message: str, code: str = "invalid_request_error", param: str | None = None):
        super().__init__(message)
        self.status, self.message, self.code, self.param = status, message, code, param


@dataclass
class EngineRequest:
    request_id: str
    model: str
    prompt_tokens: list[int]
    max_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logprobs: int = 0
    skip_special_tokens: bool = True
    thinking: bool = False
    reasoning_effort: int | None = None
    stop: list[str] = field(default_factory=list)
    seed: int | None = None
    trace_scopes: int = 0
    trace_steps: int = 0
    constraint: dict | None = None
    images: list[Any] = field(default_factory=list)
    vision: list[Any] = field(default_factory=list)     # prepared spans (serve/vision_glue.py), in prompt order
    tools: bool = False
    tool_block_open: bool = False      # the prompt ended inside an opened calls block (tool_choice required)
    tool_dialect: str = "dsml"
    # teacher forcing (numerics / identity gates): generation index i emits forced_tokens[i] whatever the model chose; the
    # model's own choices come back with the result, so two runs of one forced sequence compare position by position
    forced_tokens: list[int] = field(default_factory=list)


@dataclass
class Capabilities:
    constrained: bool = True
    vision: bool = False
    logprobs: bool = False
    penalties: bool = False
    speculative: bool = False


class InferenceEngine:
    """Interface.  ``generate`` yields tuples: ("started", prompt_tokens, cached_tokens), ("token", id),
    ("finished", reason, stats dict), ("error", message, code)."""

    model_id = "model"
    max_context = 4096
    capabilities = Capabilities()
    tokenizer = None

    def validate(self, req: EngineRequest) -> None:
        cap = self.capabilities
        if req.logprobs and not cap.logprobs:
            raise ApiError(400, "logprobs are not served by this engine", "unsupported_parameter", "logprobs")
        if (req.repetition_penalty != 1.0 or req.presence_penalty or req.frequency_penalty) and not cap.penalties:
            raise ApiError(400, "repetition, presence and frequency penalties are not served by this engine",
                           "unsupported_parameter", "presence_penalty")
        if req.images and not cap.vision:
            raise ApiError(400, "this engine has no vision path", "missing_capability", "messages")
        if req.constraint is not None and not cap.constrained:
            raise ApiError(400, "response_format cannot be enforced by this engine", "unsupported_parameter", "response_format")
        if len(req.prompt_tokens) + req.max_tokens > self.max_context:
            raise ApiError(400, f"prompt ({len(req.prompt_tokens)}) plus max_tokens ({req.max_tokens}) exceeds the context "
                                f"length {self.max_context}", "context_length_exceeded", "messages")
        if not req.prompt_tokens:
            raise ApiError(400, "empty prompt", "invalid_request_error", "messages")

    async def generate(self, req: EngineRequest) -> AsyncIterator[tuple]:
        raise NotImplementedError
        yield

    def healthy(self) -> tuple[bool, str]:
        return True, "ok"

    def stats(self) -> dict:
        return {}

    def cancel(self, request_id: str) -> None:
        pass


class MockEngine(InferenceEngine):
    """Scripted: ``script(prompt_tokens) -> list[int]`` gives the tokens the 'model' wants to say; a
    constraint, when present, overrides a token it does not admit by the lowest admitted id."""

    def __init__(self, tokenizer, script: Callable[[list[int]], list[int]] | None = None, max_context: int = 4096,
                 lanes: int = 2, queue: int = 2, delay: float = 0.0, model_id: str = "mock-model", capabilities=None):
        self.tokenizer = tokenizer
        self.script = script or (lambda p: tokenizer.encode("Hello from the mock engine."))
        self.max_context = max_context
        self.model_id = model_id
        self.capabilities = capabilities or Capabilities()
        self.lanes, self.queue_depth, self.delay = lanes, queue, delay
        self.running = 0
        self.waiting = 0
        self._sem = asyncio.Semaphore(lanes)
        self._vocab = None
        self.seen: list[EngineRequest] = []
        self.fail: str | None = None

    def vocab(self) -> TokenVocab:
        if self._vocab is None:
            self._vocab = TokenVocab(self.tokenizer.token_bytes())
        return self._vocab

    def healthy(self):
        return (False, self.fail) if self.fail else (True, "ok")

    def stats(self):
        return {"running": self.running, "waiting": self.waiting}

    async def generate(self, req: EngineRequest):
        self.seen.append(req)
        if self.fail:
            yield ("error", self.fail, "engine_failed"); return
        if self.running >= self.lanes and self.waiting >= self.queue_depth:
            yield ("error", "all lanes busy and the queue is full", "overloaded"); return
        self.waiting += 1
        async with self._sem:
            self.waiting -= 1
            self.running += 1
            try:
                yield ("started", len(req.prompt_tokens), 0)
                cst = None
                if req.constraint is not None:
                    cst = TokenConstraint(Schema(req.constraint), self.vocab(), self.tokenizer.eos_id)
                want = list(self.script(req.prompt_tokens)) + [self.tokenizer.eos_id]
                n = 0
                reason = "length"
                i = 0
                while n < req.max_tokens:
                    tok = want[i] if i < len(want) else self.tokenizer.eos_id
                    i += 1
                    if cst is not None:
                        if not cst.admits(tok):
                            ids = cst.allowed_ids()
                            if not ids:
                                yield ("error", "the constraint admits no token", "constraint_dead_end"); return
                            prefer = [self.tokenizer.eos_id] + [ord(ch) for ch in '"}]:,']      # steer towards closing the document
                            tok = next((t for t in prefer if t in ids), ids[0])
                        cst.advance(tok)
                    if tok == self.tokenizer.eos_id:
                        reason = "stop"; break
                    n += 1
                    if self.delay:
                        await asyncio.sleep(self.delay)
                    yield ("token", tok)
                yield ("finished", reason, {"decode_tokens": n})
            finally:
                self.running -= 1


@dataclass
class Delta:
    reasoning: str = ""
    content: str = ""
    tool: list = field(default_factory=list)


class Generation:
    """Per-request pipeline from token ids to API deltas."""

    def __init__(self, req: EngineRequest, tokenizer):
        self.req = req
        self.dec = StreamDecoder(tokenizer, req.skip_special_tokens)
        # reasoning and tool markup are spelled with special tokens: decode them even when hidden from content
        self.raw = StreamDecoder(tokenizer, False)
        self.tok = tokenizer
        self.reason = ReasoningSplitter(req.thinking)
        self.stops = StopStrings(req.stop)
        self.tools = (DsmlToolParser(req.tool_block_open) if req.tool_dialect == "dsml" else XmlToolParser()) if req.tools else None
        self.loop = LoopAbortDetector()
        self.completion_tokens = 0
        self.model_choices: list[int] | None = None     # filled from the engine's result when the request was teacher-forced
        self.finish: str | None = None
        self.text = ""
        self.reasoning_text = ""
        self.t0 = time.monotonic()
        self.t_first: float | None = None

    def _visible(self, token_id: int) -> str:
        piece = self.raw.push(token_id)
        if self.req.skip_special_tokens and self.tok.is_special(token_id):
            from .encoding import DSML, THINK_END, THINK_START
            return piece if piece in (THINK_START, THINK_END, DSML) else ""
        return piece

    def push(self, token_id: int) -> Delta:
        if self.t_first is None:
            self.t_first = time.monotonic()
        self.completion_tokens += 1
        d = self._text(self._visible(token_id), False)
        if self.loop.push_token(token_id) or self.loop.push_text(d.content):
            self.finish = "loop_abort"
        return d

    def _text(self, piece: str, final: bool) -> Delta:
        r, c = self.reason.feed(piece, final)
        d = Delta(reasoning=r)
        c = self.stops.feed(c, final)
        if self.stops.hit is not None:
            self.finish = "stop"
        if self.tools is not None:
            c, d.tool = self.tools.feed(c, final or self.stops.hit is not None)
        d.content = c
        self.text += c
        self.reasoning_text += r
        return d

    def flush(self) -> Delta:
        return self._text(self.raw.flush(), True)

    @property
    def tool_calls(self) -> list[dict]:
        return self.tools.calls if self.tools is not None else []
