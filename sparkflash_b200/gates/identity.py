"""Identity gates: the invariances every configuration must keep, checked on a live engine through the serving
driver.  Run-to-run determinism, batch and concurrency invariance, speculation never changes the output,
chunk-width invariance, and a request resumed on a reused prefix matches a fresh one.  Reference:
docs/NUMERICS.md section 1 item 2, scripts/identity-gate.sh, scripts/batch-gate.sh.

    python -m sparkflash_b200.gates.identity            # tiny model on cuda:0
"""
from __future__ import annotations

import asyncio
import sys


async def _collect(drv, req):
    toks = []
    async for ev in drv.generate(req):
        if ev[0] == "token":
            toks.append(ev[1])
        elif ev[0] == "error":
            raise RuntimeError(ev[1])
    return toks


def _run(make_driver, reqs, **kw):
    drv = make_driver(**kw).start()
    try:
        async def go():
            return await asyncio.gather(*[_collect(drv, r) for r in reqs])
        return asyncio.run(go())
    finally:
        drv.shutdown(1.0)


def run_gates(make_driver, prompts: list[list[int]], n_new: int = 10, temperature: float = 0.7) -> dict[str, bool]:
    """``make_driver(**kw)`` builds a fresh driver+engine; kw: drafter, prefill_chunk, prefix_reuse_min, max_lanes."""
    from ..serve.driver import NgramDrafter
    from ..serve.engine_api import EngineRequest

    def reqs(tag):
        return [EngineRequest(f"{tag}{i}", "m", p, max_tokens=n_new, temperature=temperature, seed=11 + i) for i, p in enumerate(prompts)]
    out = {}
    alone = [_run(make_driver, [r], prefix_reuse_min=10 ** 9)[0] for r in reqs("a")]
    again = [_run(make_driver, [r], prefix_reuse_min=10 ** 9)[0] for r in reqs("b")]
    out["run_to_run"] = alone == again
    out["batch_invariance"] = _run(make_driver, reqs("c"), prefix_reuse_min=10 ** 9) == alone
    out["speculation_invisible"] = _run(make_driver, reqs("d"), prefix_reuse_min=10 ** 9, drafter=NgramDrafter(3)) == alone
    out["chunk_width"] = [_run(make_driver, [r], prefix_reuse_min=10 ** 9, prefill_chunk=5)[0] for r in reqs("e")] == alone
    # resume: the same prompt twice on one lane, the second adopts the first's prefix
    drv = make_driver(prefix_reuse_min=4, max_lanes=1).start()
    try:
        first = asyncio.run(_collect(drv, reqs("f")[0]))
        second = asyncio.run(_collect(drv, reqs("g")[0]))
        out["resume_matches_fresh"] = first == second == alone[0] and drv.sched.stats()["prefix_hits"] >= 1
    finally:
        drv.shutdown(1.0)
    return out


def main() -> int:
    import torch
    from ..config import tiny_config
    from ..models.deepseek_v41 import engine as E, prepare as P, weights as W
    from ..serve.driver import DeviceDriver
    from ..serve.tokenizer import ByteTokenizer
    cfg = tiny_config()
    w = P.prepare_from_checkpoint(W.synthetic_checkpoint(cfg, 0), cfg, 0, 1)
    tok = ByteTokenizer(cfg.vocab_size)

    def make(**kw):
        lanes = kw.pop("max_lanes", 4)
        eng = E.Engine(w, max_lanes=lanes, max_context=512, max_rows=16, arm="tc")
        return DeviceDriver(eng, tok, eos_id=10 ** 9, max_lanes=lanes, **kw)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (19, 33)] + [([65, 66, 67] * 12)[:30]]
    res = run_gates(make, prompts)
    for k, v in res.items():
        print(f"identity: {k:24s} {'ok' if v else 'FAIL'}")
    return 0 if all(res.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
