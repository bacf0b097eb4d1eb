"""Serving loop over a fake rows engine: chunked prefill, continuous batching, prefix reuse, speculation
that does not change the output, constraints, cancellation, fail-stop (reference tests:
crates/sparkflash-serve/tests/{concurrency,prefix_cache,toy_host}.rs, tp4 batch tests)."""
import asyncio
import json

from starlette.testclient import TestClient

from sparkflash_b200.serve.driver import DeviceDriver, FakeRowsEngine, NgramDrafter
from sparkflash_b200.serve.engine_api import EngineRequest
from sparkflash_b200.serve.server import Server
from sparkflash_b200.serve.tokenizer import ByteTokenizer

TOK = ByteTokenizer(300)


async def collect(drv, req):
    toks, fin = [], None
    async for ev in drv.generate(req):
        if ev[0] == "token":
            toks.append(ev[1])
        elif ev[0] in ("finished", "error"):
            fin = ev
    return toks, fin


def run(drv, reqs):
    async def go():
        return await asyncio.gather(*[collect(drv, r) for r in reqs])
    drv.start()
    try:
        return asyncio.run(go())
    finally:
        drv.shutdown(1.0)


def reference_tokens(prompt, n, **kw):
    eng = FakeRowsEngine(**kw)
    for p, t in enumerate(prompt):
        eng.lane_tokens[0][p] = t
    out, pos = [], len(prompt) - 1
    for _ in range(n):
        t = eng._next(0, pos)
        if t == eng.eos_id:
            break
        out.append(t); pos += 1; eng.lane_tokens[0][pos] = t
    return out


def test_chunked_prefill_and_batching_match_the_sequential_result():
    prompts = [list(range(40, 40 + n)) for n in (37, 5, 20)]
    eng = FakeRowsEngine(max_rows=8)
    drv = DeviceDriver(eng, TOK, prefix_reuse_min=1000)
    res = run(drv, [EngineRequest(f"r{i}", "m", p, max_tokens=12, temperature=0.0) for i, p in enumerate(prompts)])
    for (toks, fin), p in zip(res, prompts):
        assert fin[0] == "finished" and fin[1] == "length" and toks == reference_tokens(p, 12)
    assert max(eng.steps) <= 8 and any(s == 3 for s in eng.steps)        # three sequences shared decode steps


def test_prefix_reuse_keeps_the_output_and_skips_rows():
    base = list(range(50, 110))
    eng = FakeRowsEngine(max_rows=16, max_lanes=1)
    drv = DeviceDriver(eng, TOK, prefix_reuse_min=8)
    drv.start()
    try:
        a = asyncio.run(collect(drv, EngineRequest("a", "m", base, max_tokens=4, temperature=0.0)))
        rows_a = sum(eng.steps)
        b = asyncio.run(collect(drv, EngineRequest("b", "m", base[:48] + [7, 8, 9], max_tokens=4, temperature=0.0)))
    finally:
        drv.shutdown(1.0)
    assert b[0] == reference_tokens(base[:48] + [7, 8, 9], 4)
    assert sum(eng.steps) - rows_a == 3 + 3 and drv.sched.stats()["prefix_rows"] == 48


def test_speculation_does_not_change_the_output():
    cyc = [65, 66, 67, 68, 69, 70]
    prompt = [cyc[i % 6] for i in range(24)]
    plain = DeviceDriver(FakeRowsEngine(cycle=cyc), TOK)
    want = run(plain, [EngineRequest("p", "m", prompt, max_tokens=30, temperature=0.0)])[0]
    eng = FakeRowsEngine(cycle=cyc)
    spec = DeviceDriver(eng, TOK, drafter=NgramDrafter(depth=4))
    got = run(spec, [EngineRequest("s", "m", prompt, max_tokens=30, temperature=0.0)])[0]
    assert got[0] == want[0] and len(got[0]) == 30
    st = got[1][2]
    assert st["accepted"] > 0 and st["accepted"] <= st["proposed"] and len([s for s in eng.steps if s > 1]) < 30


def test_constraint_masks_reach_the_sampler():
    eng = FakeRowsEngine()
    drv = DeviceDriver(eng, TOK)
    sc = {"type": "object", "properties": {"n": {"type": "integer", "minimum": 1, "maximum": 9}}, "required": ["n"], "additionalProperties": False}
    (toks, fin), = run(drv, [EngineRequest("c", "m", [1, 2, 3], max_tokens=64, temperature=0.0, constraint=sc)])
    assert fin[0] == "finished" and fin[1] == "stop"
    doc = json.loads(bytes(toks).decode())
    assert 1 <= doc["n"] <= 9


def test_http_over_the_driver_and_fail_stop():
    eng = FakeRowsEngine(eos_after=30)
    drv = DeviceDriver(eng, TOK, model_id="fake").start()
    try:
        c = TestClient(Server(drv).app)
        j = c.post("/v1/completions", json={"prompt": "hello world, this is a test", "max_tokens": 50}).json()
        assert j["choices"][0]["finish_reason"] == "stop" and j["usage"]["completion_tokens"] == 31 - len("hello world, this is a test")
        assert c.get("/readyz").status_code == 200
        eng.status_error = "device status code=3 where=7"
        r = c.post("/v1/completions", json={"prompt": "x", "max_tokens": 5})
        assert r.status_code == 503
        assert c.get("/health").status_code == 503 and "device status" in c.get("/health").json()["reason"]
        assert c.post("/v1/completions", json={"prompt": "x"}).status_code == 503
    finally:
        drv.shutdown(0.1)


def test_cancel_frees_the_lane():
    eng = FakeRowsEngine(max_lanes=1)
    drv = DeviceDriver(eng, TOK, queue_depth=0).start()

    async def go():
        agen = drv.generate(EngineRequest("x", "m", [5, 6, 7], max_tokens=400))
        n = 0
        async for ev in agen:
            if ev[0] == "token":
                n += 1
                if n == 3:
                    break
        await agen.aclose()
        await asyncio.sleep(0.1)
        return await collect(drv, EngineRequest("y", "m", [5, 6, 7], max_tokens=3))
    try:
        toks, fin = asyncio.run(go())
    finally:
        drv.shutdown(0.5)
    assert fin[0] == "finished" and len(toks) == 3


def test_image_parts_become_spans_whose_rows_carry_the_tower_output():
    import base64, io
    import torch
    from PIL import Image
    from sparkflash_b200.serve import encoding as ENC
    from sparkflash_b200.serve.vision_glue import VisionFrontEnd
    from sparkflash_b200.vision import plan as VP, tower as VT
    vc = VP.VisionConfig(n_layers=1, dim=32, n_heads=2, inter_dim=48, llm_dim=16, min_pixels=42 * 42, max_n_token=64)
    tw = VT.VisionTower(vc, VT.synthetic_vision_weights(vc))
    tok = ByteTokenizer(300)
    front = VisionFrontEnd(tw, tok.special_ids[ENC.IMAGE])
    buf = io.BytesIO(); Image.new("RGB", (60, 40), (200, 10, 10)).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    eng = FakeRowsEngine(eos_after=10 ** 6, max_rows=8)
    drv = DeviceDriver(eng, tok, model_id="fake", eos_id=10 ** 9).start()
    try:
        c = TestClient(Server(drv, vision=front).app)
        body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "look:"}, {"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "what?"}]}], "max_tokens": 3}
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        pl = VP.plan_image_grid(60, 40, vc)
        assert r.json()["usage"]["prompt_tokens"] == len(tok.encode(ENC.BOS + ENC.USER + "look:what?" + ENC.ASSISTANT + ENC.THINK_END)) + pl.n_tokens
        # every position of the span reached the engine as an embedding row, in order, exactly once
        pos = [p for _, p, _ in eng.image_log]
        assert len(pos) == pl.n_tokens and pos == list(range(pos[0], pos[0] + pl.n_tokens))
        assert c.get("/v1/models").json()["data"][0]["capabilities"]["vision"]
        bad = {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://example.com/x.png"}}]}]}
        r = c.post("/v1/chat/completions", json=bad)
        assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported_image_source"
    finally:
        drv.shutdown(0.5)


def test_top_p_top_k_reach_the_engine_only_for_sampling_rows():
    eng = FakeRowsEngine()
    drv = DeviceDriver(eng, TOK)
    reqs = [EngineRequest("a", "m", [1, 2, 3], max_tokens=3, temperature=0.8, top_p=0.9, top_k=40),
            EngineRequest("b", "m", [4, 5, 6], max_tokens=3, temperature=0.0, top_p=0.5),       # greedy: the filter is moot
            EngineRequest("c", "m", [7, 8, 9], max_tokens=3, temperature=1.0)]
    res = run(drv, reqs)
    assert all(f[0] == "finished" for _, f in res)
    assert eng.filter_log and all(f == (40, 0.9) for _, f in eng.filter_log)


def test_eight_sequences_share_one_verify_step_under_the_depth_policy():
    """Eight decoding sequences with a host drafter that is always right: the depth policy gives every sequence drafts
    while the step stays within its row cap, all of them ride in one verify step per tick, and the output is the
    sequential one (speculation invisible)."""
    from sparkflash_b200.sched.spec import SpecPolicy, StepCost
    cycle = [65, 66, 67, 68, 69, 70, 71]
    eng = FakeRowsEngine(max_rows=64, max_lanes=8, cycle=cycle)

    class OracleDrafter:
        """Knows the fake model's cycle: proposes the true continuation with high confidence."""
        depth = 5
        policy = SpecPolicy(StepCost(a0=5.0, b0=0.2, a1=5.0, b1=0.2, band=5), max_rows=64, max_depth=5)

        def propose(self, history):
            p = len(history) - 1          # position of the last token
            toks = [cycle[(p + 1 + i) % len(cycle)] for i in range(5)]
            return toks, [6.0] * 5
    drv = DeviceDriver(eng, TOK, drafter=OracleDrafter(), prefix_reuse_min=1000, eos_id=10 ** 9)
    prompts = [[40 + i, 41 + i, 42 + i] for i in range(8)]
    res = run(drv, [EngineRequest(f"r{i}", "m", p, max_tokens=24, temperature=0.0) for i, p in enumerate(prompts)])
    for (toks, fin), p in zip(res, prompts):
        assert fin[0] == "finished" and toks == reference_tokens(p, 24, cycle=cycle)
    assert max(eng.steps) <= 64
    # a shared speculative step: eight anchors plus drafts of several sequences in one rows step
    assert any(s > 16 for s in eng.steps), eng.steps
    assert drv.last_allocation.rows <= 64 and sum(drv.last_allocation.keep) > 0
    # 192 tokens in a few dozen steps (prompt steps included): the drafts were accepted
    assert len(eng.steps) < 60


def test_teacher_forcing_reports_the_models_choices_and_speculation_does_not_change_them():
    """Forced tokens are what gets emitted and fed back; the model's own choice per position is reported, and it is the same
    with and without a drafter, alone and beside other sequences (the served identity gate's property)."""
    from sparkflash_b200.gates import served
    forced = [70, 71, 33, 90, 91, 92, 40, 41, 42, 43, 60, 61]
    prompt = [50, 51, 52, 53]

    def server(drafter):
        eng = FakeRowsEngine(max_rows=16, max_lanes=6)
        drv = DeviceDriver(eng, TOK, drafter=drafter, prefix_reuse_min=1000, eos_id=10 ** 9, model_id="m").start()
        return TestClient(Server(drv).app), drv

    def fetch_with(client):
        def fetch(p, f):
            r = client.post("/v1/completions", json={"model": "m", "prompt": p, "forced_tokens": f, "temperature": 0.0})
            assert r.status_code == 200, r.text
            ch = r.json()["choices"][0]
            return ch["model_choices"]
        return fetch
    results = {}
    for name, drafter in (("plain", None), ("ngram", NgramDrafter(depth=4))):
        client, drv = server(drafter)
        try:
            with client:
                res = served.run(fetch_with(client), prompt, forced, concurrency=3)
                assert res["identical"] and res["positions"] == len(forced), res
                results[name] = res["alone"]
        finally:
            drv.shutdown(1.0)
    assert results["plain"] == results["ngram"]
    # the reported choices are the fake model's picks along the *forced* history
    eng = FakeRowsEngine()
    hist = prompt + forced
    for p, t in enumerate(hist):
        eng.lane_tokens[0][p] = t
    want = [eng._next(0, len(prompt) - 1 + i) for i in range(len(forced))]
    assert results["plain"] == want
