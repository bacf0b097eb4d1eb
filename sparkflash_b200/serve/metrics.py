"""Prometheus text exposition of the serving counters (reference: crates/sparkflash-api/src/metrics.rs:116-242;
the metric names are the wire contract, `hbm_free_gib` replaces the unified-memory gauge)."""
from __future__ import annotations

import threading

COUNTERS = [
    ("sparkflash_requests_total", "Requests accepted by the router."),
    ("sparkflash_requests_rejected_total", "Requests refused because lanes and queue were full."),
    ("sparkflash_prompt_tokens_total", "Prompt tokens processed."),
    ("sparkflash_generation_tokens_total", "Tokens generated."),
    ("sparkflash_global_kv_hit_tokens_total", "Prompt tokens served from a reused lane prefix."),
    ("sparkflash_draft_tokens_accepted_total", "Draft tokens accepted by verification."),
    ("sparkflash_draft_tokens_proposed_total", "Draft tokens proposed."),
    ("sparkflash_verify_steps_total", "Speculative verify steps."),
    ("vllm:spec_decode_num_accepted_tokens_total", "Accepted draft tokens (vLLM-compatible name)."),
    ("vllm:spec_decode_num_draft_tokens_total", "Proposed draft tokens (vLLM-compatible name)."),
    ("vllm:spec_decode_num_drafts_total", "Draft passes (vLLM-compatible name)."),
    ("sparkflash_engram_lookups_total", "Engram table lookups."),
]
GAUGES = [
    ("sparkflash_last_decode_tokens_per_second", "Decode rate of the last finished request."),
    ("sparkflash_last_prefill_tokens_per_second", "Prefill rate of the last finished request."),
    ("sparkflash_last_acceptance_rate", "Draft acceptance rate of the last finished request."),
    ("sparkflash_last_time_to_first_token_seconds", "TTFT of the last finished request."),
    ("sparkflash_engram_hit_rate", "Engram cache hit rate."),
    ("sparkflash_trace_active_scope_mask", "Currently armed trace scopes."),
    ("sparkflash_hbm_free_gib", "Free device memory on this rank."),
    ("sparkflash_num_requests_running", "Sequences holding a lane."),
    ("sparkflash_num_requests_waiting", "Sequences queued."),
    ("sparkflash_serving", "1 while the engine accepts work, 0 after a fail-stop or stall."),
]
TTFT_BUCKETS = [0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30, 60]


class Metrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.c = {n: 0.0 for n, _ in COUNTERS}
        self.g = {n: 0.0 for n, _ in GAUGES}
        self.g["sparkflash_serving"] = 1.0
        self.ttft_counts = [0] * (len(TTFT_BUCKETS) + 1)
        self.ttft_sum = 0.0

    def inc(self, name: str, v: float = 1.0) -> None:
        with self._lock:
            self.c[name] += v

    def set(self, name: str, v: float) -> None:
        with self._lock:
            self.g[name] = float(v)

    def observe_ttft(self, seconds: float) -> None:
        with self._lock:
            self.ttft_sum += seconds
            for i, b in enumerate(TTFT_BUCKETS):
                if seconds <= b:
                    self.ttft_counts[i] += 1
                    break
            else:
                self.ttft_counts[-1] += 1
            self.g["sparkflash_last_time_to_first_token_seconds"] = seconds

    def render(self) -> str:
        with self._lock:
            out = []
            for n, h in COUNTERS:
                out += [f"# HELP {n} {h}", f"# TYPE {n} counter", f"{n} {self.c[n]:g}"]
            for n, h in GAUGES:
                out += [f"# HELP {n} {h}", f"# TYPE {n} gauge", f"{n} {self.g[n]:g}"]
            n = "sparkflash_time_to_first_token_seconds"
            out += [f"# HELP {n} Time to first token.", f"# TYPE {n} histogram"]
            acc = 0
            for b, c in zip(TTFT_BUCKETS, self.ttft_counts):
                acc += c
                out.append(f'{n}_bucket{{le="{b:g}"}} {acc}')
            acc += self.ttft_counts[-1]
            out += [f'{n}_bucket{{le="+Inf"}} {acc}', f"{n}_sum {self.ttft_sum:g}", f"{n}_count {acc}"]
            return "\n".join(out) + "\n"
