"""The serving loop over the real device engine on the tiny model: driver output equals Engine.generate,
speculative verify rows do not change it (position-addressed caches make rejected rows harmless), prefix
reuse keeps it, and the head honours a constraint mask."""
import asyncio
import json

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    from sparkflash_b200.config import tiny_config
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P, weights as W
    from sparkflash_b200.serve.tokenizer import ByteTokenizer
    cfg = tiny_config()
    ck = W.synthetic_checkpoint(cfg, 0)
    w = P.prepare_from_checkpoint(ck, cfg, 0, 1)
    tok = ByteTokenizer(cfg.vocab_size)

    def make(**kw):
        return E.Engine(w, max_lanes=3, max_context=256, max_rows=16, arm="tc", constrained=True, **kw)
    return cfg, tok, make


async def _collect(drv, req):
    toks, fin = [], None
    async for ev in drv.generate(req):
        if ev[0] == "token":
            toks.append(ev[1])
        elif ev[0] in ("finished", "error"):
            fin = ev
    return toks, fin


def _run(drv, reqs):
    async def go():
        return await asyncio.gather(*[_collect(drv, r) for r in reqs])
    drv.start()
    try:
        return asyncio.run(go())
    finally:
        drv.shutdown(1.0)


def test_driver_matches_generate_and_speculation_is_invisible(setup):
    from sparkflash_b200.serve.driver import DeviceDriver, NgramDrafter
    from sparkflash_b200.serve.engine_api import EngineRequest
    cfg, tok, make = setup
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (23, 9)]
    # a repetitive prompt so that the n-gram drafter has something to propose
    prompts.append(([65, 66, 67, 68] * 8)[:30])
    want = [make().generate(p, 10) for p in prompts]
    eos = 10 ** 9      # never sampled: compare fixed-length runs
    plain = _run(DeviceDriver(make(), tok, eos_id=eos, prefix_reuse_min=1000),
                 [EngineRequest(f"p{i}", "m", p, max_tokens=10, temperature=0.0) for i, p in enumerate(prompts)])
    for (toks, fin), w in zip(plain, want):
        assert fin[0] == "finished" and toks[:3] == w[:3]        # batched rows share a step with other sequences:
        assert sum(a == b for a, b in zip(toks, w)) >= 7           # bits are batch-invariant, so this is normally exact
    spec = _run(DeviceDriver(make(), tok, eos_id=eos, prefix_reuse_min=1000, drafter=NgramDrafter(depth=3)),
                [EngineRequest(f"s{i}", "m", p, max_tokens=10, temperature=0.0) for i, p in enumerate(prompts)])
    for (a, _), (b, fb) in zip(plain, spec):
        assert a == b, (a, b)
    assert any(f[2]["proposed"] > 0 for _, f in spec)


def test_prefix_reuse_and_constraint_on_device(setup):
    from sparkflash_b200.serve.driver import DeviceDriver
    from sparkflash_b200.serve.engine_api import EngineRequest
    cfg, tok, make = setup
    g = torch.Generator().manual_seed(9)
    base = torch.randint(0, 256, (40,), generator=g).tolist()
    second = base[:32] + [1, 2, 3]
    want = make().generate(second, 6)
    third = base + [1, 2, 3]
    want3 = make().generate(third, 6)
    plain = DeviceDriver(make(), tok, eos_id=10 ** 9, prefix_reuse_min=8, max_lanes=1, decoder_skip=False).start()
    try:
        asyncio.run(_collect(plain, EngineRequest("a", "m", base, max_tokens=3, temperature=0.0)))
        toks, fin = asyncio.run(_collect(plain, EngineRequest("b", "m", second, max_tokens=6, temperature=0.0)))
        assert plain.sched.stats()["prefix_rows"] == 32 and toks == want
    finally:
        plain.shutdown(1.0)
    # with the decoder-layer skip on, a fork inside the rows whose upper layers were skipped backs off one tail; the kept
    # prefix would then lie behind rows that the first request's later positions overwrote in the window ring, so nothing
    # is reused - and a continuation past the prompt's fully computed tail keeps everything
    drv = DeviceDriver(make(), tok, eos_id=10 ** 9, prefix_reuse_min=8, max_lanes=1).start()
    try:
        asyncio.run(_collect(drv, EngineRequest("a", "m", base, max_tokens=3, temperature=0.0)))
        toks, fin = asyncio.run(_collect(drv, EngineRequest("b", "m", second, max_tokens=6, temperature=0.0)))
        assert drv.sched.stats()["prefix_rows"] == 0 and toks == want
        asyncio.run(_collect(drv, EngineRequest("a2", "m", base, max_tokens=3, temperature=0.0)))
        toks, fin = asyncio.run(_collect(drv, EngineRequest("d", "m", third, max_tokens=6, temperature=0.0)))
        assert drv.sched.stats()["prefix_rows"] == 40 and toks == want3
        sc = {"type": "object", "properties": {"n": {"type": "integer", "minimum": 1, "maximum": 9}}, "required": ["n"], "additionalProperties": False}
        drv.eos_id = tok.eos_id
        toks, fin = asyncio.run(_collect(drv, EngineRequest("c", "m", base[:10], max_tokens=200, temperature=0.8, seed=3, constraint=sc)))
    finally:
        drv.shutdown(1.0)
    if fin[1] == "stop":
        doc = json.loads(bytes(toks).decode())
        assert 1 <= doc["n"] <= 9
    else:       # whitespace padding is bounded, so a random model still has to close the document eventually
        assert fin[1] == "length"


def test_candidate_filter_top_k_top_p(setup):
    cfg, tok, make = setup
    eng = make()
    prompt = list(range(30, 50))
    eng.step(prompt[:16], [0] * 16, list(range(16)))
    eng.step(prompt[16:], [0] * 4, list(range(16, 20)), temperature=[1.0] * 4, seeds=[7] * 4)
    row = 3
    lg = eng.logits[row].float()
    best = int(lg.argmax())
    assert eng.filtered_sample(row, 1, 1.0, 1.0, 7, 19) == best                    # top_k = 1 is the argmax
    assert eng.filtered_sample(row, 0, 1e-6, 1.0, 7, 19) == best                   # a vanishing nucleus too
    top5 = set(torch.topk(lg, 5).indices.tolist())
    draws = {eng.filtered_sample(row, 5, 1.0, 5.0, s, 19) for s in range(40)}
    assert draws <= top5 and len(draws) > 1                                        # hot temperature, still inside top-5
    assert eng.filtered_sample(row, 5, 1.0, 5.0, 3, 19) == eng.filtered_sample(row, 5, 1.0, 5.0, 3, 19)
    assert eng.filtered_sample(row, 0, 1.0, 0.0, 3, 19) == best                    # greedy
    out = eng.step([1], [0], [20], temperature=[2.0], seeds=[5], filters={0: (3, 1.0)})
    assert int(out[0]) in set(torch.topk(eng.logits[0].float(), 3).indices.tolist())


def test_decoder_layer_skip_is_exact(setup):
    """Prompt rows far before the end run only the cache-owning layers; the generated tokens and the final logits are
    the ones a full run gives."""
    from sparkflash_b200.serve.driver import DeviceDriver
    from sparkflash_b200.serve.engine_api import EngineRequest
    cfg, tok, make = setup
    g = torch.Generator().manual_seed(21)
    prompt = torch.randint(0, 256, (90,), generator=g).tolist()
    outs = {}
    for skip in (False, True):
        eng = make(keep_logits=True)
        assert eng.decoder_skip_layer == 3 and eng.decoder_tail == 24
        calls = []
        orig = eng.step
        eng.step = lambda *a, **k: (calls.append((len(a[0]), k.get("skip_decoder", False))), orig(*a, **k))[1]
        drv = DeviceDriver(eng, tok, eos_id=10 ** 9, prefix_reuse_min=1000, decoder_skip=skip).start()
        try:
            toks, fin = asyncio.run(_collect(drv, EngineRequest("r", "m", prompt, max_tokens=8, temperature=0.0)))
        finally:
            drv.shutdown(1.0)
        outs[skip] = (toks, sum(n for n, s in calls if s))
    assert outs[True][1] == 90 - 24 and outs[False][1] == 0
    assert outs[True][0] == outs[False][0]
