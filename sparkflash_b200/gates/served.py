"""Served identity gate: the same teacher-forced sequence through a running server under different serving
conditions must give the same model choices at every position.

The request names the tokens to emit (``forced_tokens``, an extension of ``/v1/completions``); the server emits them and
reports, per position, the token the model would have chosen.  Conditions compared: alone vs. beside concurrent traffic,
and (by running the gate against servers started with different settings) speculation on/off, chunk width, graphs on/off.

    python -m sparkflash_b200.gates.served --url http://127.0.0.1:8000 [--concurrency 4] [--tokens 48]

Reference: scripts/served-gate.py, scripts/identity-gate.sh, docs/NUMERICS.md:104-188,245-301 of the reference.
"""
from __future__ import annotations

import argparse
import json
import random
import threading
import urllib.request


def complete(url: str, prompt: list[int], forced: list[int], api_key: str | None = None, temperature: float = 0.0, seed: int = 0,
             timeout: float = 120.0) -> list[int]:
    body = {"model": "default", "prompt": prompt, "forced_tokens": forced, "temperature": temperature, "seed": seed}
    hdr = {"Content-Type": "application/json"}
    if api_key:
        hdr["Authorization"] = f"Bearer {api_key}"
    req = urllib.request.Request(url.rstrip("/") + "/v1/completions", data=json.dumps(body).encode(), headers=hdr)
    with urllib.request.urlopen(req, timeout=timeout) as r:
        out = json.loads(r.read())
    ch = out["choices"][0]
    if "model_choices" not in ch:
        raise RuntimeError("the server does not report model_choices (no teacher forcing)")
    return ch["model_choices"]


def run(fetch, prompt: list[int], forced: list[int], concurrency: int = 4, noise_prompts: list[list[int]] | None = None) -> dict:
    """``fetch(prompt, forced) -> model choices``.  Runs the probe alone, then beside ``concurrency`` other requests, and
    compares.  Returns {"identical": bool, "first_difference": index or None, ...}."""
    alone = fetch(prompt, forced)
    noise_prompts = noise_prompts or [[(7 * i + 3 * j) % 200 + 10 for j in range(5 + 3 * i)] for i in range(concurrency)]
    busy: dict = {}

    def probe():
        busy["probe"] = fetch(prompt, forced)

    def noise(i):
        busy[i] = fetch(noise_prompts[i], forced[:max(4, len(forced) // 2)])
    ts = [threading.Thread(target=noise, args=(i,)) for i in range(min(concurrency, len(noise_prompts)))] + [threading.Thread(target=probe)]
    [t.start() for t in ts]; [t.join() for t in ts]
    crowded = busy["probe"]
    diff = next((i for i, (a, b) in enumerate(zip(alone, crowded)) if a != b), None)
    if diff is None and len(alone) != len(crowded):
        diff = min(len(alone), len(crowded))
    return {"identical": diff is None, "first_difference": diff, "positions": len(alone), "alone": alone, "beside_traffic": crowded}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--api-key")
    ap.add_argument("--tokens", type=int, default=48)
    ap.add_argument("--prompt-tokens", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    rng = random.Random(a.seed)
    prompt = [rng.randrange(10, a.vocab) for _ in range(a.prompt_tokens)]
    forced = [rng.randrange(10, a.vocab) for _ in range(a.tokens)]
    res = run(lambda p, f: complete(a.url, p, f, a.api_key), prompt, forced, a.concurrency)
    print(json.dumps({k: v for k, v in res.items() if k not in ("alone", "beside_traffic")}))
    return 0 if res["identical"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
