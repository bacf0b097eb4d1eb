"""HTTP surface against the scripted engine (reference tests: crates/sparkflash-api/tests/router.rs,
protocol_adapters.rs, encoding_golden.rs, batch_completions.rs, tokenizer_seam.rs)."""
import json

import pytest
from starlette.testclient import TestClient

from sparkflash_b200.serve import encoding as ENC
from sparkflash_b200.serve.engine_api import Capabilities, MockEngine
from sparkflash_b200.serve.reasoning import LoopAbortDetector, StopStrings
from sparkflash_b200.serve.server import Server
from sparkflash_b200.serve.tokenizer import ByteTokenizer

TOK = ByteTokenizer()


def client(script_text="Hello there.", **kw):
    eng = MockEngine(TOK, lambda p: TOK.encode(script_text), **{k: v for k, v in kw.items() if k in ("lanes", "queue", "delay", "capabilities", "max_context")})
    srv = Server(eng, **{k: v for k, v in kw.items() if k in ("api_key", "aliases", "default_thinking")})
    return TestClient(srv.app), eng, srv


def sse(resp):
    out = []
    for block in resp.text.strip().split("\n\n"):
        ev, data = None, None
        for line in block.split("\n"):
            if line.startswith("event: "): ev = line[7:]
            if line.startswith("data: "): data = line[6:]
        out.append((ev, data if data == "[DONE]" else json.loads(data)))
    return out


def test_prompt_rendering_matches_the_protocol():
    msgs = [ENC.Message("user", "hi"), ENC.Message("user", "again")]
    assert ENC.render_prompt(msgs) == ENC.BOS + ENC.USER + "hi\n\nagain" + ENC.ASSISTANT + ENC.THINK_END
    p = ENC.render_prompt([ENC.Message("user", "q")], thinking=True, effort=50)
    assert p == ENC.BOS + ENC.SYSTEM + "Reasoning Effort: 50 (range 1-100, the higher the value, the more thorough the reasoning)\n\n" + ENC.USER + "q" + ENC.ASSISTANT + ENC.THINK_START
    calls = [ENC.ToolCall("b", "f2", '{"k": [1, true, null]}'), ENC.ToolCall("a", "f1", '{"s": "x"}')]
    hist = [ENC.Message("system", "S"), ENC.Message("user", "u"), ENC.Message("assistant", "", tool_calls=calls),
            ENC.Message("tool", "r1", tool_call_id="a"), ENC.Message("tool", "r2", tool_call_id="b"), ENC.Message("system", "mid")]
    p = ENC.render_prompt(hist)
    assert '<｜DSML｜ parameter name="k" string="false">[1, True, None]</｜DSML｜ parameter>' in p
    assert '<｜DSML｜ parameter name="s" string="true">x</｜DSML｜ parameter>' in p
    assert p.index("<tool_result>r2</tool_result>") < p.index("<tool_result>r1</tool_result>")   # order of the calls
    assert p.count(ENC.SYSTEM) == 2 and p.endswith(ENC.SYSTEM + "mid" + ENC.ASSISTANT + ENC.THINK_END)
    assert ENC.resolve_thinking("none", None, True) == (False, None)
    assert ENC.resolve_thinking("low", None, False) == (True, 25)
    assert ENC.resolve_thinking(None, {"type": "enabled", "budget_tokens": 5}, False) == (True, 50)
    assert ENC.resolve_thinking("max", {"type": "disabled"}, False) == (False, None)


def test_chat_buffered_and_streamed_agree():
    c, eng, _ = client("Hello there.")
    body = {"model": "mock-model", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 64}
    r = c.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["choices"][0]["message"]["content"] == "Hello there." and j["choices"][0]["finish_reason"] == "stop"
    assert j["usage"]["completion_tokens"] == len("Hello there.") and j["usage"]["prompt_tokens"] == len(eng.seen[0].prompt_tokens)
    r = c.post("/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}})
    evs = sse(r)
    assert evs[-1][1] == "[DONE]" and evs[-2][1]["usage"]["completion_tokens"] == len("Hello there.")
    text = "".join(e[1]["choices"][0]["delta"].get("content", "") for e in evs[:-2] if e[1].get("choices"))
    assert text == "Hello there."
    assert evs[0][1]["choices"][0]["delta"]["role"] == "assistant"


def test_length_stop_strings_and_n():
    c, _, _ = client("abcdefghij")
    base = {"messages": [{"role": "user", "content": "x"}]}
    j = c.post("/v1/chat/completions", json={**base, "max_tokens": 4}).json()
    assert j["choices"][0]["message"]["content"] == "abcd" and j["choices"][0]["finish_reason"] == "length"
    j = c.post("/v1/chat/completions", json={**base, "stop": ["ef", "zz"]}).json()
    assert j["choices"][0]["message"]["content"] == "abcd" and j["choices"][0]["finish_reason"] == "stop"
    j = c.post("/v1/chat/completions", json={**base, "n": 3, "seed": 7}).json()
    assert [ch["index"] for ch in j["choices"]] == [0, 1, 2] and j["usage"]["completion_tokens"] == 30
    s = StopStrings(["END"])
    assert s.feed("abE") == "ab" and s.feed("Nx") == "ENx" and s.feed("EN") == "" and s.feed("D tail") == "" and s.hit == "END"


def test_reasoning_is_returned_separately():
    c, eng, _ = client("thinking hard" + ENC.THINK_END + "answer")
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "reasoning_effort": "high"})
    m = r.json()["choices"][0]["message"]
    assert m["reasoning_content"] == "thinking hard" and m["content"] == "answer"
    assert eng.seen[0].thinking and eng.seen[0].reasoning_effort == 50
    evs = sse(c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "thinking": {"type": "enabled"}, "stream": True}))
    rs = "".join(e[1]["choices"][0]["delta"].get("reasoning_content", "") for e in evs if e[1] != "[DONE]" and e[1].get("choices"))
    assert rs == "thinking hard"


TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]


def test_tool_calls_are_parsed_incrementally():
    call = ENC.render_tool_calls([ENC.ToolCall("x", "get_weather", '{"city": "Paris", "n": 2}')])
    c, eng, _ = client("Let me check.\n\n" + call)
    body = {"messages": [{"role": "user", "content": "weather?"}], "tools": TOOLS}
    j = c.post("/v1/chat/completions", json=body).json()
    ch = j["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["content"] == "Let me check.\n\n"
    tc = ch["message"]["tool_calls"][0]
    assert tc["function"]["name"] == "get_weather" and json.loads(tc["function"]["arguments"]) == {"city": "Paris", "n": 2}
    assert "## Tools" in TOK.decode(eng.seen[0].prompt_tokens, False)
    evs = sse(c.post("/v1/chat/completions", json={**body, "stream": True}))
    args = "".join(t["function"]["arguments"] for e in evs if e[1] != "[DONE]" for chx in e[1].get("choices", []) for t in chx["delta"].get("tool_calls", []))
    assert json.loads(args) == {"city": "Paris", "n": 2}
    # required: the prompt ends inside an opened block and the model continues from there
    inner = call.split("calls>\n", 1)[1]
    c2, eng2, _ = client(inner)
    j = c2.post("/v1/chat/completions", json={**body, "tool_choice": "required"}).json()
    assert j["choices"][0]["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert TOK.decode(eng2.seen[0].prompt_tokens, False).endswith("<｜DSML｜ calls>\n")
    r = c2.post("/v1/chat/completions", json={**body, "tool_choice": "required", "reasoning_effort": "high"})
    assert r.status_code == 400
    r = c2.post("/v1/chat/completions", json={**body, "tool_choice": {"type": "function", "function": {"name": "nope"}}})
    assert r.status_code == 400


def test_json_schema_is_enforced_and_unsupported_schemas_are_refused():
    c, _, _ = client("this is not json at all")
    sc = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer", "minimum": 3, "maximum": 5}}, "required": ["ok", "n"], "additionalProperties": False}
    body = {"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_schema", "json_schema": {"name": "t", "schema": sc}}, "max_tokens": 200}
    j = c.post("/v1/chat/completions", json=body).json()
    doc = json.loads(j["choices"][0]["message"]["content"])
    assert isinstance(doc["ok"], bool) and 3 <= doc["n"] <= 5
    j = c.post("/v1/chat/completions", json={**body, "response_format": {"type": "json_object"}}).json()
    assert isinstance(json.loads(j["choices"][0]["message"]["content"]), dict)
    bad = {**body, "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "string", "pattern": "a+"}}}}
    r = c.post("/v1/chat/completions", json=bad)
    assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported_schema"
    c2, _, _ = client("x", capabilities=Capabilities(constrained=False))
    assert c2.post("/v1/chat/completions", json=body).status_code == 400


def test_typed_refusals_and_validation():
    c, _, _ = client("x", max_context=64)
    base = {"messages": [{"role": "user", "content": "x"}]}
    for extra, param in [({"logprobs": True}, "logprobs"), ({"presence_penalty": 0.5}, "presence_penalty"), ({"repetition_penalty": 1.2}, "presence_penalty")]:
        r = c.post("/v1/chat/completions", json={**base, **extra})
        assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported_parameter" and r.json()["error"]["param"] == param
    r = c.post("/v1/chat/completions", json={**base, "max_tokens": 100000})
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"
    assert c.post("/v1/chat/completions", json={**base, "model": "other"}).status_code == 404
    assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    assert c.post("/v1/chat/completions", content=b"{not json").status_code == 400
    assert c.post("/v1/chat/completions", json={**base, "temperature": -1}).status_code == 400
    img = {"messages": [{"role": "user", "content": [{"type": "text", "text": "see"}, {"type": "image_url", "image_url": {"url": "data:..."}}]}]}
    r = c.post("/v1/chat/completions", json=img)
    assert r.status_code == 400 and r.json()["error"]["code"] == "missing_capability"


def test_completions_text_ids_batches_and_echo():
    c, eng, _ = client("xyz")
    j = c.post("/v1/completions", json={"prompt": "ab", "max_tokens": 8, "echo": True}).json()
    assert j["choices"][0]["text"] == "abxyz"
    j = c.post("/v1/completions", json={"prompt": [[97, 98], [99]], "max_tokens": 8}).json()
    assert len(j["choices"]) == 2 and j["usage"]["prompt_tokens"] == 3
    assert c.post("/v1/completions", json={"prompt": [999999]}).status_code == 400
    evs = sse(c.post("/v1/completions", json={"prompt": "ab", "stream": True}))
    assert "".join(e[1]["choices"][0]["text"] for e in evs[:-1]) == "xyz"


def test_responses_api_event_sequence():
    c, _, _ = client("think" + ENC.THINK_END + "final text")
    body = {"input": [{"type": "message", "role": "user", "content": [{"type": "input_text", "text": "q"}]}], "instructions": "be brief", "reasoning": {"effort": "low"}}
    j = c.post("/v1/responses", json=body).json()
    assert j["status"] == "completed" and [o["type"] for o in j["output"]] == ["reasoning", "message"]
    assert j["output"][1]["content"][0]["text"] == "final text" and j["usage"]["output_tokens"] > 0
    evs = sse(c.post("/v1/responses", json={**body, "stream": True}))
    kinds = [e[0] for e in evs]
    assert kinds[:2] == ["response.created", "response.in_progress"] and kinds[-1] == "response.completed"
    for k in ["response.output_item.added", "response.content_part.added", "response.output_text.delta", "response.output_text.done",
              "response.content_part.done", "response.output_item.done", "response.reasoning_text.delta"]:
        assert k in kinds, k
    assert [e[1]["sequence_number"] for e in evs] == list(range(1, len(evs) + 1))
    j = c.post("/v1/responses", json={"input": "q", "max_output_tokens": 2}).json()
    assert j["status"] == "incomplete"


def test_anthropic_messages_blocks():
    call = ENC.render_tool_calls([ENC.ToolCall("x", "get_weather", '{"city": "Oslo"}')])
    c, _, _ = client("hmm" + ENC.THINK_END + "Checking." + call)
    body = {"model": "mock-model", "max_tokens": 500, "system": "sys", "thinking": {"type": "enabled", "budget_tokens": 100},
            "messages": [{"role": "user", "content": [{"type": "text", "text": "weather"}]}],
            "tools": [{"name": "get_weather", "input_schema": {"type": "object"}}]}
    j = c.post("/v1/messages", json=body).json()
    assert [b["type"] for b in j["content"]] == ["thinking", "text", "tool_use"] and j["stop_reason"] == "tool_use"
    assert j["content"][2]["input"] == {"city": "Oslo"}
    evs = sse(c.post("/v1/messages", json={**body, "stream": True}))
    kinds = [e[0] for e in evs]
    assert kinds[0] == "message_start" and kinds[-2:] == ["message_delta", "message_stop"]
    assert kinds.count("content_block_start") == 3 == kinds.count("content_block_stop")
    dtypes = {e[1]["delta"]["type"] for e in evs if e[0] == "content_block_delta"}
    assert dtypes == {"thinking_delta", "text_delta", "input_json_delta"}
    r = c.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 400 and r.json()["type"] == "error"


def test_models_tokenize_health_metrics_auth_aliases():
    c, eng, srv = client("ok", api_key="sekret", aliases={"gpt-4o": "mock-model"})
    assert c.get("/v1/models").status_code == 401
    h = {"Authorization": "Bearer sekret"}
    j = c.get("/v1/models", headers=h).json()
    assert j["data"][0]["id"] == "mock-model" and j["data"][0]["capabilities"]["constrained"] and "gpt-4o" in j["data"][0]["aliases"]
    assert c.get("/v1/models/mock-model", headers=h).status_code == 200 and c.get("/v1/models/nope", headers=h).status_code == 404
    assert c.post("/v1/chat/completions", headers=h, json={"model": "gpt-4o", "messages": [{"role": "user", "content": "x"}]}).status_code == 200
    t = c.post("/tokenize", headers=h, json={"prompt": "héllo"}).json()
    assert t["count"] == 6 and c.post("/detokenize", headers=h, json={"tokens": t["tokens"]}).json()["prompt"] == "héllo"
    t2 = c.post("/tokenize", headers=h, json={"messages": [{"role": "user", "content": "x"}]}).json()
    assert t2["tokens"][0] == TOK.special_ids[ENC.BOS]
    assert c.get("/health").status_code == 200 and c.get("/readyz").json()["ready"]
    m = c.get("/metrics").text
    assert "sparkflash_requests_total 1" in m and "sparkflash_serving 1" in m and "sparkflash_time_to_first_token_seconds_count 1" in m
    eng.fail = "device status 12"
    assert c.get("/health").status_code == 503 and c.get("/readyz").status_code == 503
    r = c.post("/v1/chat/completions", headers=h, json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 503
    assert "sparkflash_serving 0" in c.get("/metrics").text


def test_overload_returns_503():
    import asyncio

    async def go():
        eng = MockEngine(TOK, lambda p: TOK.encode("0123456789"), lanes=1, queue=1, delay=0.01)
        srv = Server(eng)
        import httpx
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=srv.app), base_url="http://t") as ac:
            rs = await asyncio.gather(*[ac.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}) for _ in range(4)])
        return sorted(r.status_code for r in rs), srv
    codes, srv = asyncio.run(go())
    assert codes.count(200) >= 2 and codes.count(503) >= 1
    assert "sparkflash_requests_rejected_total" in srv.metrics.render()


def test_loop_abort_detector():
    d = LoopAbortDetector(ngram=3, max_repeats=4)
    fired = [d.push_token(t) for t in [1, 2, 3] * 4]
    assert fired[-1] and not any(fired[:-1])
    d = LoopAbortDetector(max_line_repeats=3, min_line_bytes=5)
    assert not d.push_text("short\nshort line one\nshort line one\n") and d.push_text("short line one\n")
    c, _, _ = client("abcdefgh" * 40)
    j = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 1000}).json()
    assert j["usage"]["completion_tokens"] == 64 and j["choices"][0]["finish_reason"] == "stop"
