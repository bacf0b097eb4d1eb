"""HTTP surface: OpenAI chat/completions/responses and Anthropic messages over one engine seam.

Routes (reference: crates/sparkflash-api/src/server.rs:262-280; behaviour docs/serving.md:79-173):
``POST /v1/chat/completions  /v1/completions  /v1/responses  /v1/messages  /tokenize  /detokenize``,
``GET /v1/models[/id]  /health  /readyz  /metrics  /v1/cluster/stats  /v1/admin/trace``, ``POST /v1/admin/trace``,
``GET /v1/admin/trace/dump``.  Optional bearer auth, model aliases.  What the engine cannot enforce is
refused with a typed error, never ignored.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, AsyncIterator

from starlette.applications import Starlette
from starlette.requests import Request
from starlette.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse
from starlette.routing import Route

from . import encoding as ENC
from .constrained import Schema, SchemaError
from .engine_api import ApiError, EngineRequest, Generation, InferenceEngine
from .metrics import Metrics

BUILD_ID = "sparkflash-b200/0.1"


def _err(status: int, message: str, code: str = "invalid_request_error", param: str | None = None, flavor: str = "openai") -> JSONResponse:
    if flavor == "anthropic":
        return JSONResponse({"type": "error", "error": {"type": code, "message": message}}, status_code=status)
    return JSONResponse({"error": {"message": message, "type": code, "param": param, "code": code}}, status_code=status)


def _sse(obj: Any, event: str | None = None) -> bytes:
    head = f"event: {event}\n" if event else ""
    return (head + "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n").encode()


def _content_text(content: Any, images: list) -> str:
    """OpenAI / Anthropic content: a string or a list of typed parts."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for p in content:
        t = p.get("type")
        if t in ("text", "input_text", "output_text"):
            out.append(p.get("text", ""))
        elif t in ("image_url", "input_image", "image"):
            images.append(p)
            out.append(ENC.IMAGE)
        elif t == "tool_result":
            out.append(_content_text(p.get("content"), images))
        elif t in ("thinking", "tool_use"):
            pass
        else:
            raise ApiError(400, f"unknown content part type {t!r}", param="messages")
    return "".join(out)


class Server:
    def __init__(self, engine: InferenceEngine, api_key: str | None = None, aliases: dict[str, str] | None = None,
                 default_thinking: bool = False, trace=None, default_max_tokens: int = 1024, vision=None):
        self.engine = engine
        self.tok = engine.tokenizer
        self.api_key = api_key
        self.aliases = aliases or {}
        self.default_thinking = default_thinking
        self.metrics = Metrics()
        self.trace = trace
        self.vision = vision          # serve/vision_glue.VisionFrontEnd, when the engine has the vision path
        self.default_max_tokens = default_max_tokens
        self.draining = False
        self.started_at = time.time()
        self.app = Starlette(routes=[
            Route("/v1/chat/completions", self._wrap(self.chat), methods=["POST"]),
            Route("/v1/completions", self._wrap(self.completions), methods=["POST"]),
            Route("/v1/responses", self._wrap(self.responses), methods=["POST"]),
            Route("/v1/messages", self._wrap(self.messages, "anthropic"), methods=["POST"]),
            Route("/v1/models", self._wrap(self.models), methods=["GET"]),
            Route("/v1/models/{model_id:path}", self._wrap(self.model), methods=["GET"]),
            Route("/tokenize", self._wrap(self.tokenize), methods=["POST"]),
            Route("/detokenize", self._wrap(self.detokenize), methods=["POST"]),
            Route("/health", self.health, methods=["GET"]),
            Route("/readyz", self.readyz, methods=["GET"]),
            Route("/metrics", self.metrics_route, methods=["GET"]),
            Route("/v1/cluster/stats", self._wrap(self.cluster_stats), methods=["GET"]),
            Route("/v1/admin/trace", self._wrap(self.admin_trace), methods=["GET", "POST"]),
            Route("/v1/admin/trace/dump", self._wrap(self.admin_trace_dump), methods=["GET"]),
        ])

    # ---- plumbing -------------------------------------------------------------------------------------
    def _wrap(self, fn, flavor: str = "openai"):
        async def handler(request: Request):
            if self.api_key:
                auth = request.headers.get("authorization", "")
                key = request.headers.get("x-api-key", "")
                if auth != f"Bearer {self.api_key}" and key != self.api_key:
                    return _err(401, "missing or wrong API key", "authentication_error", flavor=flavor)
            try:
                return await fn(request)
            except ApiError as e:
                return _err(e.status, e.message, e.code, e.param, flavor)
            except SchemaError as e:
                return _err(400, str(e), "unsupported_schema", "response_format", flavor)
            except json.JSONDecodeError as e:
                return _err(400, f"request body is not JSON: {e}", flavor=flavor)
        return handler

    async def _body(self, request: Request) -> dict:
        raw = await request.body()
        body = json.loads(raw or b"{}")
        if not isinstance(body, dict):
            raise ApiError(400, "request body must be a JSON object")
        return body

    def _model(self, name: str | None) -> str:
        if not name:
            return self.engine.model_id
        name = self.aliases.get(name, name)
        if name != self.engine.model_id:
            raise ApiError(404, f"model {name!r} is not served here (serving {self.engine.model_id!r})", "model_not_found", "model")
        return name

    def _check_serving(self):
        ok, why = self.engine.healthy()
        if not ok:
            self.metrics.set("sparkflash_serving", 0)
            raise ApiError(503, f"engine is not serving: {why}", "engine_unavailable")
        if self.draining:
            raise ApiError(503, "server is draining", "engine_unavailable")

    def _sampling(self, body: dict, req: EngineRequest, max_key: tuple[str, ...]) -> None:
        for k in max_key:
            if body.get(k) is not None:
                req.max_tokens = int(body[k]); break
        else:
            req.max_tokens = min(self.default_max_tokens, max(1, self.engine.max_context - len(req.prompt_tokens)))
        if req.max_tokens < 1:
            raise ApiError(400, "max_tokens must be at least 1", param=max_key[0])
        req.temperature = float(body.get("temperature", 1.0) if body.get("temperature") is not None else 1.0)
        req.top_p = float(body.get("top_p") if body.get("top_p") is not None else 1.0)
        req.top_k = int(body.get("top_k") if body.get("top_k") is not None else 0)
        if req.temperature < 0 or not 0 < req.top_p <= 1 or req.top_k < -1:
            raise ApiError(400, "temperature must be >= 0, top_p in (0, 1], top_k >= -1", param="temperature")
        req.seed = body.get("seed")
        stop = body.get("stop") or body.get("stop_sequences") or []
        req.stop = [stop] if isinstance(stop, str) else list(stop)
        req.repetition_penalty = float(body.get("repetition_penalty") or 1.0)
        req.presence_penalty = float(body.get("presence_penalty") or 0.0)
        req.frequency_penalty = float(body.get("frequency_penalty") or 0.0)
        lp = body.get("logprobs")
        req.logprobs = int(body.get("top_logprobs") or 1) if lp is True else int(lp or 0)
        if body.get("skip_special_tokens") is False:
            req.skip_special_tokens = False

    def _response_format(self, body: dict, req: EngineRequest) -> str | None:
        rf = body.get("response_format") or (body.get("text") or {}).get("format")
        if not rf or rf.get("type") == "text":
            return None
        if not self.engine.capabilities.constrained:
            raise ApiError(400, "response_format cannot be enforced by this engine", "unsupported_parameter", "response_format")
        if rf["type"] == "json_object":
            req.constraint = {"type": "object"}
            return "Respond with a single JSON object."
        if rf["type"] == "json_schema":
            sc = rf.get("json_schema", rf).get("schema") or rf.get("schema")
            if sc is None:
                raise ApiError(400, "json_schema needs a schema", param="response_format")
            Schema(sc)       # refuse what cannot be enforced before any token is generated
            req.constraint = sc
            return "Respond with a JSON document that satisfies this schema:\n" + json.dumps(sc, ensure_ascii=False)
        raise ApiError(400, f"unknown response_format type {rf['type']!r}", param="response_format")

    def _trace_header(self, request: Request, req: EngineRequest) -> None:
        h = request.headers.get("x-sparkflash-trace")
        if h and self.trace is not None:
            scopes, _, steps = h.partition(";")
            req.trace_scopes = self.trace.parse_scopes(scopes)
            req.trace_steps = int(steps.replace("steps=", "") or 64) if steps else 64

    async def _run(self, req: EngineRequest) -> AsyncIterator[tuple[str, Any]]:
        """Drive one request: yields ("started", p, c) | ("delta", Delta) | ("done", reason, Generation) and
        raises ApiError for engine errors before the first token."""
        self.engine.validate(req)
        gen = Generation(req, self.tok)
        self.metrics.inc("sparkflash_requests_total")
        self.metrics.inc("sparkflash_prompt_tokens_total", len(req.prompt_tokens))
        reason = "stop"
        first = True
        agen = self.engine.generate(req)
        try:
            async for ev in agen:
                if ev[0] == "started":
                    self.metrics.inc("sparkflash_global_kv_hit_tokens_total", ev[2])
                    yield ev
                elif ev[0] == "token":
                    if first:
                        first = False
                        self.metrics.observe_ttft(time.monotonic() - gen.t0)
                    d = gen.push(ev[1])
                    self.metrics.inc("sparkflash_generation_tokens_total")
                    yield ("delta", d)
                    if gen.finish is not None:
                        reason = gen.finish
                        self.engine.cancel(req.request_id)
                        break
                elif ev[0] == "finished":
                    reason = ev[1]
                    st = ev[2] or {}
                    if "model_choices" in st:
                        gen.model_choices = list(st["model_choices"])
                    if st.get("proposed"):
                        self.metrics.inc("sparkflash_draft_tokens_proposed_total", st["proposed"])
                        self.metrics.inc("vllm:spec_decode_num_draft_tokens_total", st["proposed"])
                        self.metrics.inc("sparkflash_draft_tokens_accepted_total", st.get("accepted", 0))
                        self.metrics.inc("vllm:spec_decode_num_accepted_tokens_total", st.get("accepted", 0))
                        self.metrics.inc("sparkflash_verify_steps_total", st.get("verify_steps", 0))
                        self.metrics.inc("vllm:spec_decode_num_drafts_total", st.get("verify_steps", 0))
                        self.metrics.set("sparkflash_last_acceptance_rate", st.get("accepted", 0) / st["proposed"])
                    break
                elif ev[0] == "error":
                    if ev[2] == "overloaded":
                        self.metrics.inc("sparkflash_requests_rejected_total")
                        raise ApiError(503, ev[1], "overloaded")
                    if ev[2] == "engine_failed":
                        self.metrics.set("sparkflash_serving", 0)
                        raise ApiError(503, ev[1], "engine_unavailable")
                    raise ApiError(500, ev[1], ev[2])
        finally:
            await agen.aclose()
        d = gen.flush()
        if d.reasoning or d.content or d.tool:
            yield ("delta", d)
        if gen.tool_calls and reason == "stop":
            reason = "tool_calls"
        dt = max(1e-9, time.monotonic() - (gen.t_first or gen.t0))
        self.metrics.set("sparkflash_last_decode_tokens_per_second", gen.completion_tokens / dt)
        yield ("done", reason, gen)

    @staticmethod
    def _usage(req: EngineRequest, gen: Generation, cached: int) -> dict:
        return {"prompt_tokens": len(req.prompt_tokens), "completion_tokens": gen.completion_tokens,
                "total_tokens": len(req.prompt_tokens) + gen.completion_tokens,
                "prompt_tokens_details": {"cached_tokens": cached}}

    # ---- chat completions -------------------------------------------------------------------------------
    def _chat_request(self, body: dict, request: Request, messages: list[ENC.Message], tools: list[dict] | None,
                      tool_choice: Any, max_key: tuple[str, ...]) -> EngineRequest:
        model = self._model(body.get("model"))
        thinking, effort = ENC.resolve_thinking(body.get("reasoning_effort"), body.get("thinking"), self.default_thinking)
        tools = tools or []
        required = False
        if isinstance(tool_choice, dict):      # a named function: only that tool is offered, and one call is forced
            name = (tool_choice.get("function") or tool_choice).get("name")
            tools = [t for t in tools if (t.get("function") or t).get("name") == name]
            if not tools:
                raise ApiError(400, f"tool_choice names an unknown tool {name!r}", param="tool_choice")
            required = True
        elif tool_choice == "required" or tool_choice == "any":
            required = True
        elif tool_choice == "none":
            tools = []
        elif tool_choice not in (None, "auto"):
            raise ApiError(400, f"unknown tool_choice {tool_choice!r}", param="tool_choice")
        if required and not tools:
            raise ApiError(400, "tool_choice requires tools", param="tool_choice")
        if required and thinking:
            raise ApiError(400, "a forced tool call requires thinking to be off", param="tool_choice")
        req = EngineRequest(request_id=request.headers.get("x-request-id") or "req_" + uuid.uuid4().hex[:20], model=model,
                            prompt_tokens=[], thinking=thinking, reasoning_effort=effort)
        hint = self._response_format(body, req)
        req.images = [im for m in messages for im in m.images]
        prompt = ENC.render_prompt(messages, tools, thinking, effort, required, hint)
        req.prompt_tokens = self.tok.encode(prompt)
        if req.images and self.vision is not None and self.engine.capabilities.vision:
            req.prompt_tokens, req.vision = self.vision.expand(req.prompt_tokens, req.images)
            req.images = []
        req.tools = bool(tools)
        req.tool_block_open = required
        self._sampling(body, req, max_key)
        self._trace_header(request, req)
        return req

    @staticmethod
    def _openai_messages(raw: list[dict]) -> list[ENC.Message]:
        out = []
        for m in raw:
            role = m.get("role")
            images: list = []
            if role in ("system", "developer"):
                out.append(ENC.Message("system", _content_text(m.get("content"), images)))
            elif role == "user":
                out.append(ENC.Message("user", _content_text(m.get("content"), images), images=images))
            elif role == "assistant":
                calls = [ENC.ToolCall(c.get("id", ""), c["function"]["name"], c["function"].get("arguments", "{}")) for c in m.get("tool_calls") or []]
                out.append(ENC.Message("assistant", _content_text(m.get("content"), images), reasoning=m.get("reasoning_content") or m.get("reasoning"), tool_calls=calls))
            elif role == "tool":
                out.append(ENC.Message("tool", _content_text(m.get("content"), images), tool_call_id=m.get("tool_call_id")))
            else:
                raise ApiError(400, f"unknown role {role!r}", param="messages")
        if not out:
            raise ApiError(400, "messages must not be empty", param="messages")
        return out

    async def chat(self, request: Request):
        body = await self._body(request)
        self._check_serving()
        n = int(body.get("n") or 1)
        if n < 1 or n > 8:
            raise ApiError(400, "n must lie in 1..8", param="n")
        req0 = self._chat_request(body, request, self._openai_messages(body.get("messages") or []), body.get("tools"),
                                  body.get("tool_choice"), ("max_completion_tokens", "max_tokens"))
        self.engine.validate(req0)
        reqs = [req0] + [EngineRequest(**{**req0.__dict__, "request_id": f"{req0.request_id}-{i}",
                                          "seed": None if req0.seed is None else req0.seed + i}) for i in range(1, n)]
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": req0.model, "system_fingerprint": BUILD_ID}
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

            async def stream():
                q: asyncio.Queue = asyncio.Queue()

                async def one(i: int, r: EngineRequest):
                    try:
                        async for ev in self._run(r):
                            await q.put((i, ev))
                    except ApiError as e:
                        await q.put((i, ("error", e)))
                    await q.put((i, None))
                tasks = [asyncio.create_task(one(i, r)) for i, r in enumerate(reqs)]
                live, usage = n, {"prompt_tokens": len(req0.prompt_tokens), "completion_tokens": 0, "total_tokens": 0}
                try:
                    while live:
                        i, ev = await q.get()
                        if ev is None:
                            live -= 1; continue
                        if ev[0] == "started":
                            yield _sse({**base, "choices": [{"index": i, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})
                        elif ev[0] == "delta":
                            d = ev[1]
                            delta: dict = {}
                            if d.reasoning:
                                delta["reasoning_content"] = d.reasoning
                            if d.content:
                                delta["content"] = d.content
                            if d.tool:
                                delta["tool_calls"] = [{"index": t.index, **({"id": t.id, "type": "function"} if t.id else {}),
                                                        "function": {**({"name": t.name} if t.name else {}), "arguments": t.arguments_delta}} for t in d.tool]
                            if delta:
                                yield _sse({**base, "choices": [{"index": i, "delta": delta, "finish_reason": None}]})
                        elif ev[0] == "done":
                            usage["completion_tokens"] += ev[2].completion_tokens
                            yield _sse({**base, "choices": [{"index": i, "delta": {}, "finish_reason": _finish(ev[1])}]})
                        elif ev[0] == "error":
                            e = ev[1]
                            yield _sse({"error": {"message": e.message, "type": e.code, "code": e.code}})
                    if include_usage:
                        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
                        yield _sse({**base, "choices": [], "usage": usage})
                    yield _sse("[DONE]")
                finally:
                    for t in tasks:
                        t.cancel()
            return StreamingResponse(stream(), media_type="text/event-stream")

        async def collect(i: int, r: EngineRequest):
            cached, gen, reason = 0, None, "stop"
            async for ev in self._run(r):
                if ev[0] == "started":
                    cached = ev[2]
                elif ev[0] == "done":
                    reason, gen = ev[1], ev[2]
            msg: dict = {"role": "assistant", "content": gen.text or (None if gen.tool_calls else "")}
            if gen.reasoning_text:
                msg["reasoning_content"] = gen.reasoning_text
            if gen.tool_calls:
                msg["tool_calls"] = [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": c["arguments"]}} for c in gen.tool_calls]
            return {"index": i, "message": msg, "finish_reason": _finish(reason)}, self._usage(r, gen, cached)
        results = await asyncio.gather(*[collect(i, r) for i, r in enumerate(reqs)])
        usage = results[0][1]
        usage["completion_tokens"] = sum(u["completion_tokens"] for _, u in results)
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        return JSONResponse({"id": cid, "object": "chat.completion", "created": created, "model": req0.model,
                             "system_fingerprint": BUILD_ID, "choices": [c for c, _ in results], "usage": usage})

    # ---- text completions -------------------------------------------------------------------------------
    async def completions(self, request: Request):
        body = await self._body(request)
        self._check_serving()
        model = self._model(body.get("model"))
        prompt = body.get("prompt")
        if prompt is None:
            raise ApiError(400, "prompt is required", param="prompt")
        # a string, a list of strings, a list of token ids, or a list of lists of token ids
        if isinstance(prompt, str):
            prompts = [self.tok.encode(prompt)]
        elif isinstance(prompt, list) and prompt and all(isinstance(x, int) for x in prompt):
            prompts = [list(prompt)]
        elif isinstance(prompt, list) and prompt and all(isinstance(x, str) for x in prompt):
            prompts = [self.tok.encode(x) for x in prompt]
        elif isinstance(prompt, list) and prompt and all(isinstance(x, list) for x in prompt):
            prompts = [list(x) for x in prompt]
        else:
            raise ApiError(400, "prompt must be a string, token ids, or a list of either", param="prompt")
        for p in prompts:
            if any((not isinstance(t, int)) or t < 0 or t >= self.tok.vocab_size for t in p):
                raise ApiError(400, "token id outside the vocabulary", param="prompt")
        n = int(body.get("n") or 1)
        reqs = []
        for pi, p in enumerate(prompts):
            for j in range(n):
                r = EngineRequest(request_id="cmpl_" + uuid.uuid4().hex[:20], model=model, prompt_tokens=p)
                self._sampling(body, r, ("max_tokens",))
                if body.get("max_tokens") is None:
                    r.max_tokens = min(16, r.max_tokens)
                if r.seed is not None:
                    r.seed += j
                self._response_format(body, r)
                self._trace_header(request, r)
                forced = body.get("forced_tokens")
                if forced is not None:
                    # gate extension: emit exactly these tokens and report what the model would have chosen at each position
                    if not isinstance(forced, list) or any((not isinstance(t, int)) or t < 0 or t >= self.tok.vocab_size for t in forced):
                        raise ApiError(400, "forced_tokens must be a list of token ids inside the vocabulary", param="forced_tokens")
                    r.forced_tokens = list(forced)
                    r.max_tokens = len(forced)
                self.engine.validate(r)
                reqs.append(r)
        cid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        echo = bool(body.get("echo"))
        if body.get("stream"):
            async def stream():
                for i, r in enumerate(reqs):
                    try:
                        async for ev in self._run(r):
                            if ev[0] == "delta" and ev[1].content:
                                yield _sse({"id": cid, "object": "text_completion", "created": created, "model": model,
                                            "choices": [{"index": i, "text": ev[1].content, "finish_reason": None, "logprobs": None}]})
                            elif ev[0] == "done":
                                yield _sse({"id": cid, "object": "text_completion", "created": created, "model": model,
                                            "choices": [{"index": i, "text": "", "finish_reason": _finish(ev[1]), "logprobs": None}]})
                    except ApiError as e:
                        yield _sse({"error": {"message": e.message, "type": e.code, "code": e.code}})
                yield _sse("[DONE]")
            return StreamingResponse(stream(), media_type="text/event-stream")

        async def collect(i, r):
            async for ev in self._run(r):
                if ev[0] == "done":
                    text = (self.tok.decode(r.prompt_tokens) if echo else "") + ev[2].text
                    choice = {"index": i, "text": text, "finish_reason": _finish(ev[1]), "logprobs": None}
                    if ev[2].model_choices is not None:
                        choice["model_choices"] = ev[2].model_choices
                    return choice, ev[2].completion_tokens
        results = await asyncio.gather(*[collect(i, r) for i, r in enumerate(reqs)])
        pt = sum(len(p) for p in prompts)
        ct = sum(c for _, c in results)
        return JSONResponse({"id": cid, "object": "text_completion", "created": created, "model": model,
                             "choices": [c for c, _ in results], "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}})

    # ---- OpenAI Responses ---------------------------------------------------------------------------------
    async def responses(self, request: Request):
        body = await self._body(request)
        self._check_serving()
        msgs: list[dict] = []
        if body.get("instructions"):
            msgs.append({"role": "system", "content": body["instructions"]})
        inp = body.get("input")
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        elif isinstance(inp, list):
            for it in inp:
                t = it.get("type", "message")
                if t == "message":
                    msgs.append({"role": it.get("role", "user"), "content": it.get("content")})
                elif t == "function_call":
                    msgs.append({"role": "assistant", "content": "", "tool_calls": [{"id": it.get("call_id", ""), "function": {"name": it["name"], "arguments": it.get("arguments", "{}")}}]})
                elif t == "function_call_output":
                    msgs.append({"role": "tool", "tool_call_id": it.get("call_id"), "content": it.get("output", "")})
                elif t == "reasoning":
                    pass
                else:
                    raise ApiError(400, f"unknown input item type {t!r}", param="input")
        else:
            raise ApiError(400, "input must be a string or a list of items", param="input")
        tools = [{"type": "function", "function": {k: v for k, v in t.items() if k != "type"}} for t in body.get("tools") or [] if t.get("type") == "function"]
        b2 = dict(body)
        if isinstance(body.get("reasoning"), dict) and body["reasoning"].get("effort"):
            b2["reasoning_effort"] = body["reasoning"]["effort"]
        req = self._chat_request(b2, request, self._openai_messages(msgs), tools, body.get("tool_choice"), ("max_output_tokens",))
        self.engine.validate(req)
        rid, created = "resp_" + uuid.uuid4().hex[:24], int(time.time())
        mid = "msg_" + uuid.uuid4().hex[:24]

        def envelope(status, output, usage=None):
            return {"id": rid, "object": "response", "created_at": created, "status": status, "model": req.model,
                    "output": output, "usage": usage, "error": None, "incomplete_details": None if status != "incomplete" else {"reason": "max_output_tokens"}}

        def final_output(gen: Generation):
            out = []
            if gen.reasoning_text:
                out.append({"id": "rs_" + uuid.uuid4().hex[:24], "type": "reasoning", "summary": [], "content": [{"type": "reasoning_text", "text": gen.reasoning_text}]})
            if gen.text or not gen.tool_calls:
                out.append({"id": mid, "type": "message", "role": "assistant", "status": "completed",
                            "content": [{"type": "output_text", "text": gen.text, "annotations": []}]})
            for c in gen.tool_calls:
                out.append({"id": "fc_" + c["id"][5:], "type": "function_call", "call_id": c["id"], "name": c["name"], "arguments": c["arguments"], "status": "completed"})
            return out

        def usage_of(gen, cached):
            return {"input_tokens": len(req.prompt_tokens), "input_tokens_details": {"cached_tokens": cached},
                    "output_tokens": gen.completion_tokens, "total_tokens": len(req.prompt_tokens) + gen.completion_tokens}

        if body.get("stream"):
            async def stream():
                seq = 0

                def ev(kind, **kw):
                    nonlocal seq
                    seq += 1
                    return _sse({"type": kind, "sequence_number": seq, **kw}, kind)
                yield ev("response.created", response=envelope("in_progress", []))
                yield ev("response.in_progress", response=envelope("in_progress", []))
                opened, cached, text = False, 0, ""
                try:
                    async for e in self._run(req):
                        if e[0] == "started":
                            cached = e[2]
                        elif e[0] == "delta":
                            d = e[1]
                            if d.reasoning:
                                yield ev("response.reasoning_text.delta", item_id="rs_" + rid[5:], output_index=0, content_index=0, delta=d.reasoning)
                            if d.content:
                                if not opened:
                                    opened = True
                                    yield ev("response.output_item.added", output_index=0, item={"id": mid, "type": "message", "role": "assistant", "status": "in_progress", "content": []})
                                    yield ev("response.content_part.added", item_id=mid, output_index=0, content_index=0, part={"type": "output_text", "text": "", "annotations": []})
                                text += d.content
                                yield ev("response.output_text.delta", item_id=mid, output_index=0, content_index=0, delta=d.content)
                            for t in d.tool:
                                if t.id:
                                    yield ev("response.output_item.added", output_index=1 + t.index, item={"id": "fc_" + t.id[5:], "type": "function_call", "call_id": t.id, "name": t.name, "arguments": "", "status": "in_progress"})
                                if t.arguments_delta:
                                    yield ev("response.function_call_arguments.delta", output_index=1 + t.index, delta=t.arguments_delta)
                        elif e[0] == "done":
                            gen = e[2]
                            if opened:
                                yield ev("response.output_text.done", item_id=mid, output_index=0, content_index=0, text=text)
                                yield ev("response.content_part.done", item_id=mid, output_index=0, content_index=0, part={"type": "output_text", "text": text, "annotations": []})
                                yield ev("response.output_item.done", output_index=0, item={"id": mid, "type": "message", "role": "assistant", "status": "completed", "content": [{"type": "output_text", "text": text, "annotations": []}]})
                            for c in gen.tool_calls:
                                yield ev("response.function_call_arguments.done", arguments=c["arguments"], item_id="fc_" + c["id"][5:])
                            status = "incomplete" if e[1] == "length" else "completed"
                            yield ev("response.completed" if status == "completed" else "response.incomplete", response=envelope(status, final_output(gen), usage_of(gen, cached)))
                except ApiError as err:
                    yield ev("error", code=err.code, message=err.message)
            return StreamingResponse(stream(), media_type="text/event-stream")
        cached = 0
        async for e in self._run(req):
            if e[0] == "started":
                cached = e[2]
            elif e[0] == "done":
                status = "incomplete" if e[1] == "length" else "completed"
                return JSONResponse(envelope(status, final_output(e[2]), usage_of(e[2], cached)))
        raise ApiError(500, "engine ended without a result", "engine_error")

    # ---- Anthropic messages ---------------------------------------------------------------------------------
    async def messages(self, request: Request):
        body = await self._body(request)
        self._check_serving()
        if body.get("max_tokens") is None:
            raise ApiError(400, "max_tokens is required", "invalid_request_error", "max_tokens")
        msgs: list[ENC.Message] = []
        system = body.get("system")
        if system:
            msgs.append(ENC.Message("system", _content_text(system, [])))
        for m in body.get("messages") or []:
            role, content = m.get("role"), m.get("content")
            images: list = []
            if role == "user":
                if isinstance(content, list):
                    results = [p for p in content if p.get("type") == "tool_result"]
                    rest = [p for p in content if p.get("type") != "tool_result"]
                    for p in results:
                        msgs.append(ENC.Message("tool", _content_text(p.get("content"), images), tool_call_id=p.get("tool_use_id")))
                    if rest:
                        msgs.append(ENC.Message("user", _content_text(rest, images), images=images))
                else:
                    msgs.append(ENC.Message("user", content or ""))
            elif role == "assistant":
                calls, think = [], None
                if isinstance(content, list):
                    for p in content:
                        if p.get("type") == "tool_use":
                            calls.append(ENC.ToolCall(p.get("id", ""), p["name"], json.dumps(p.get("input", {}))))
                        elif p.get("type") == "thinking":
                            think = (think or "") + p.get("thinking", "")
                msgs.append(ENC.Message("assistant", _content_text(content, images), reasoning=think, tool_calls=calls))
            else:
                raise ApiError(400, f"unknown role {role!r}", param="messages")
        if not msgs:
            raise ApiError(400, "messages must not be empty", param="messages")
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""), "parameters": t.get("input_schema", {})}} for t in body.get("tools") or []]
        tc = body.get("tool_choice") or {}
        choice = {"auto": "auto", "any": "required", "none": "none"}.get(tc.get("type"), None) if tc else None
        if tc.get("type") == "tool":
            choice = {"name": tc.get("name")}
        req = self._chat_request(body, request, msgs, tools, choice, ("max_tokens",))
        self.engine.validate(req)
        mid = "msg_" + uuid.uuid4().hex[:24]

        def stop_reason(r):
            return {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(r, "end_turn")

        if body.get("stream"):
            async def stream():
                yield _sse({"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": req.model, "content": [],
                                                                    "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": len(req.prompt_tokens), "output_tokens": 0}}}, "message_start")
                idx, kind = -1, None
                tool_block: dict[int, int] = {}

                def open_block(k, block):
                    nonlocal idx, kind
                    out = []
                    if kind is not None:
                        out.append(_sse({"type": "content_block_stop", "index": idx}, "content_block_stop"))
                    idx += 1; kind = k
                    out.append(_sse({"type": "content_block_start", "index": idx, "content_block": block}, "content_block_start"))
                    return out
                try:
                    async for e in self._run(req):
                        if e[0] == "delta":
                            d = e[1]
                            if d.reasoning:
                                if kind != "thinking":
                                    for x in open_block("thinking", {"type": "thinking", "thinking": ""}): yield x
                                yield _sse({"type": "content_block_delta", "index": idx, "delta": {"type": "thinking_delta", "thinking": d.reasoning}}, "content_block_delta")
                            if d.content:
                                if kind != "text":
                                    for x in open_block("text", {"type": "text", "text": ""}): yield x
                                yield _sse({"type": "content_block_delta", "index": idx, "delta": {"type": "text_delta", "text": d.content}}, "content_block_delta")
                            for t in d.tool:
                                if t.id:
                                    for x in open_block(f"tool{t.index}", {"type": "tool_use", "id": t.id.replace("call_", "toolu_"), "name": t.name, "input": {}}): yield x
                                if t.arguments_delta:
                                    yield _sse({"type": "content_block_delta", "index": idx, "delta": {"type": "input_json_delta", "partial_json": t.arguments_delta}}, "content_block_delta")
                        elif e[0] == "done":
                            if kind is not None:
                                yield _sse({"type": "content_block_stop", "index": idx}, "content_block_stop")
                            sr = "stop_sequence" if e[2].stops.hit else stop_reason(e[1])
                            yield _sse({"type": "message_delta", "delta": {"stop_reason": sr, "stop_sequence": e[2].stops.hit}, "usage": {"output_tokens": e[2].completion_tokens}}, "message_delta")
                            yield _sse({"type": "message_stop"}, "message_stop")
                except ApiError as err:
                    yield _sse({"type": "error", "error": {"type": err.code, "message": err.message}}, "error")
            return StreamingResponse(stream(), media_type="text/event-stream")
        async for e in self._run(req):
            if e[0] == "done":
                gen = e[2]
                content = []
                if gen.reasoning_text:
                    content.append({"type": "thinking", "thinking": gen.reasoning_text, "signature": ""})
                if gen.text:
                    content.append({"type": "text", "text": gen.text})
                for c in gen.tool_calls:
                    content.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["name"], "input": json.loads(c["arguments"] or "{}")})
                sr = "stop_sequence" if gen.stops.hit else stop_reason(e[1])
                return JSONResponse({"id": mid, "type": "message", "role": "assistant", "model": req.model, "content": content,
                                     "stop_reason": sr, "stop_sequence": gen.stops.hit,
                                     "usage": {"input_tokens": len(req.prompt_tokens), "output_tokens": gen.completion_tokens}})
        raise ApiError(500, "engine ended without a result", "engine_error")

    # ---- models, tokens, health ---------------------------------------------------------------------------------
    def _model_card(self) -> dict:
        cap = self.engine.capabilities
        return {"id": self.engine.model_id, "object": "model", "created": int(self.started_at), "owned_by": "sparkflash-b200",
                "build_id": BUILD_ID, "max_model_len": self.engine.max_context,
                "capabilities": {"constrained": cap.constrained, "vision": cap.vision, "logprobs": cap.logprobs,
                                 "penalties": cap.penalties, "speculative": cap.speculative, "tools": True, "reasoning": True},
                "aliases": sorted(k for k, v in self.aliases.items() if v == self.engine.model_id)}

    async def models(self, request: Request):
        return JSONResponse({"object": "list", "data": [self._model_card()]})

    async def model(self, request: Request):
        self._model(request.path_params["model_id"])
        return JSONResponse(self._model_card())

    async def tokenize(self, request: Request):
        body = await self._body(request)
        if "messages" in body:
            thinking, effort = ENC.resolve_thinking(body.get("reasoning_effort"), body.get("thinking"), self.default_thinking)
            text = ENC.render_prompt(self._openai_messages(body["messages"]), body.get("tools"), thinking, effort)
        else:
            text = body.get("prompt", body.get("text"))
            if not isinstance(text, str):
                raise ApiError(400, "prompt (a string) or messages is required", param="prompt")
        ids = self.tok.encode(text)
        return JSONResponse({"tokens": ids, "count": len(ids), "max_model_len": self.engine.max_context})

    async def detokenize(self, request: Request):
        body = await self._body(request)
        ids = body.get("tokens")
        if not isinstance(ids, list) or any((not isinstance(t, int)) or t < 0 or t >= self.tok.vocab_size for t in ids):
            raise ApiError(400, "tokens must be a list of ids inside the vocabulary", param="tokens")
        return JSONResponse({"prompt": self.tok.decode(ids, skip_special=bool(body.get("skip_special_tokens", False)))})

    async def health(self, request: Request):
        ok, why = self.engine.healthy()
        return JSONResponse({"status": "ok" if ok else "unhealthy", "reason": why}, status_code=200 if ok else 503)

    async def readyz(self, request: Request):
        ok, why = self.engine.healthy()
        ready = ok and not self.draining
        return JSONResponse({"ready": ready, "reason": why if not ok else ("draining" if self.draining else "ok")}, status_code=200 if ready else 503)

    async def metrics_route(self, request: Request):
        st = self.engine.stats()
        self.metrics.set("sparkflash_num_requests_running", st.get("running", 0))
        self.metrics.set("sparkflash_num_requests_waiting", st.get("waiting", 0))
        if "hbm_free_gib" in st:
            self.metrics.set("sparkflash_hbm_free_gib", st["hbm_free_gib"])
        if self.trace is not None:
            self.metrics.set("sparkflash_trace_active_scope_mask", self.trace.active_mask())
        return PlainTextResponse(self.metrics.render(), media_type="text/plain; version=0.0.4")

    async def cluster_stats(self, request: Request):
        return JSONResponse({"model": self.engine.model_id, "build_id": BUILD_ID, "uptime_s": time.time() - self.started_at,
                             "engine": self.engine.stats(), "serving": self.engine.healthy()[0]})

    async def admin_trace(self, request: Request):
        if self.trace is None:
            raise ApiError(404, "tracing is not configured", "not_found")
        if request.method == "POST":
            body = await self._body(request)
            self.trace.arm(self.trace.parse_scopes(body.get("scopes", "all")), int(body.get("steps", 64)))
        return JSONResponse(self.trace.status())

    async def admin_trace_dump(self, request: Request):
        if self.trace is None:
            raise ApiError(404, "tracing is not configured", "not_found")
        return Response(json.dumps(self.trace.export_chrome()), media_type="application/json")


def _finish(reason: str) -> str:
    return {"loop_abort": "stop"}.get(reason, reason)


def create_app(engine: InferenceEngine, **kw) -> Starlette:
    return Server(engine, **kw).app
