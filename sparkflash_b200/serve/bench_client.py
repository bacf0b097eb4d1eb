"""Served benchmark: N concurrent streaming chat requests against a running server; reports aggregate
decode tok/s, TTFT percentiles and per-request rates.  Reference: scripts/bench_serving.py, scripts/served-gate.py."""
from __future__ import annotations

import asyncio
import json
import time


async def _one(client, url, headers, prompt, max_tokens, i):
    t0 = time.monotonic()
    first, n = None, 0
    body = {"messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens, "stream": True, "temperature": 0.0,
            "stream_options": {"include_usage": True}}
    usage = None
    async with client.stream("POST", url + "/v1/chat/completions", json=body, headers=headers) as r:
        if r.status_code != 200:
            await r.aread()
            return {"ok": False, "status": r.status_code}
        async for line in r.aiter_lines():
            if not line.startswith("data: ") or line == "data: [DONE]":
                continue
            ev = json.loads(line[6:])
            if ev.get("usage"):
                usage = ev["usage"]
            for ch in ev.get("choices", []):
                if ch["delta"].get("content") or ch["delta"].get("reasoning_content"):
                    n += 1
                    if first is None:
                        first = time.monotonic()
    t1 = time.monotonic()
    toks = (usage or {}).get("completion_tokens", n)
    return {"ok": True, "ttft": (first or t1) - t0, "tokens": toks, "seconds": t1 - t0, "decode_tok_s": toks / max(1e-9, t1 - (first or t0))}


async def run_async(url, concurrency, requests, prompt_tokens, max_tokens, api_key=None, transport=None):
    import httpx
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    prompt = "benchmark " * max(1, prompt_tokens // 10)
    sem = asyncio.Semaphore(concurrency)
    async with httpx.AsyncClient(timeout=600, transport=transport) as client:
        async def guarded(i):
            async with sem:
                return await _one(client, url, headers, f"[{i}] " + prompt, max_tokens, i)
        t0 = time.monotonic()
        res = await asyncio.gather(*[guarded(i) for i in range(requests)])
        wall = time.monotonic() - t0
    ok = [r for r in res if r["ok"]]
    ttft = sorted(r["ttft"] for r in ok)
    pick = lambda p: ttft[min(len(ttft) - 1, int(p * len(ttft)))] if ttft else 0.0
    return {"requests": requests, "ok": len(ok), "rejected": len(res) - len(ok), "concurrency": concurrency, "wall_s": wall,
            "aggregate_tok_s": sum(r["tokens"] for r in ok) / max(1e-9, wall), "ttft_p50_s": pick(0.5), "ttft_p99_s": pick(0.99),
            "per_request_tok_s": sum(r["decode_tok_s"] for r in ok) / max(1, len(ok))}


def run(args) -> int:
    out = asyncio.run(run_async(args.url.rstrip("/"), args.concurrency, args.requests, args.prompt_tokens, args.max_tokens, args.api_key))
    print(json.dumps(out))
    return 0 if out["ok"] else 1
