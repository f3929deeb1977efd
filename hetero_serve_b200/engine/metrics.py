"""Per-request records and a run summary, in the manner of the reference's
``RequestRecord`` / ``summarise`` (heteroserve/metrics.py:17-87, 123-180):
time to first token, time per output token, end-to-end latency."""

from __future__ import annotations

import math
from dataclasses import dataclass, field


def percentile(values: list[float], p: float) -> float:
    """Linear interpolation between closest ranks (heteroserve/metrics.py:17-28)."""
    if not values:
        return float("nan")
    s = sorted(values)
    if len(s) == 1:
        return s[0]
    k = (len(s) - 1) * p
    lo, hi = math.floor(k), math.ceil(k)
    if lo == hi:
        return s[int(k)]
    return s[lo] * (hi - k) + s[hi] * (k - lo)


@dataclass
class RequestRecord:
    req_id: object
    prompt_tokens: int = 0
    generated_tokens: int = 0
    cached_prefix_tokens: int = 0
    prefill_tokens_computed: int = 0
    preemptions: int = 0
    finish_reason: str = ""
    output_ids: list[int] = field(default_factory=list)
    t_submit: float = 0.0
    t_admit: float = 0.0
    t_first_token: float = 0.0
    t_done: float = 0.0

    @property
    def ttft(self) -> float:
        return self.t_first_token - self.t_submit if self.t_first_token else float("nan")

    @property
    def e2e(self) -> float:
        return self.t_done - self.t_submit if self.t_done else float("nan")

    @property
    def tpot(self) -> float:
        n = self.generated_tokens - 1
        if n <= 0 or not self.t_first_token or not self.t_done:
            return float("nan")
        return (self.t_done - self.t_first_token) / n

    @property
    def cache_hit_rate(self) -> float:
        return self.cached_prefix_tokens / self.prompt_tokens if self.prompt_tokens else 0.0

    def as_dict(self) -> dict:
        return {
            "req_id": self.req_id, "prompt_tokens": self.prompt_tokens,
            "generated_tokens": self.generated_tokens,
            "cached_prefix_tokens": self.cached_prefix_tokens,
            "prefill_tokens_computed": self.prefill_tokens_computed,
            "preemptions": self.preemptions, "finish_reason": self.finish_reason,
            "ttft": round(self.ttft, 5), "tpot": round(self.tpot, 6), "e2e": round(self.e2e, 5),
            "cache_hit_rate": round(self.cache_hit_rate, 4), "output_ids": list(self.output_ids),
        }

    @classmethod
    def of(cls, seq) -> "RequestRecord":
        return cls(req_id=seq.req_id, prompt_tokens=len(seq.request.prompt_ids),
                   generated_tokens=len(seq.output_ids),
                   cached_prefix_tokens=seq.cached_prefix_tokens,
                   prefill_tokens_computed=seq.prefill_tokens_computed,
                   preemptions=seq.preemptions, finish_reason=seq.finish_reason,
                   output_ids=list(seq.output_ids), t_submit=seq.t_submit, t_admit=seq.t_admit,
                   t_first_token=seq.t_first_token, t_done=seq.t_done)


def summarise(records: list[RequestRecord], wall_s: float) -> dict:
    ok = [r for r in records if r.t_done]
    gen = sum(r.generated_tokens for r in ok)
    ttft = [r.ttft for r in ok if not math.isnan(r.ttft)]
    tpot = [r.tpot for r in ok if not math.isnan(r.tpot)]
    e2e = [r.e2e for r in ok]
    prompt = sum(r.prompt_tokens for r in ok)
    return {
        "n_requests": len(ok), "wall_s": round(wall_s, 4),
        "throughput_tok_s": round(gen / wall_s, 2) if wall_s > 0 else 0.0,
        "request_throughput": round(len(ok) / wall_s, 3) if wall_s > 0 else 0.0,
        "ttft_p50": percentile(ttft, 0.5), "ttft_p95": percentile(ttft, 0.95),
        "tpot_p50": percentile(tpot, 0.5), "e2e_p50": percentile(e2e, 0.5),
        "e2e_p95": percentile(e2e, 0.95),
        "cache_hit_rate": round(sum(r.cached_prefix_tokens for r in ok) / prompt, 4) if prompt else 0.0,
        "prefill_tokens_saved": sum(r.cached_prefix_tokens for r in ok),
        "preemptions": sum(r.preemptions for r in ok),
    }
