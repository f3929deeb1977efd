"""What the engine reports about finished requests: one :class:`RequestRecord` per request
and a summary of a run.

The field and key names are the reference's (heteroserve/metrics.py:31-87 ``RequestRecord``,
:123-180 ``summarise``), so that its dashboards and result files read the same: ``ttft`` is
the time from submission to the first generated token, ``tpot`` the mean time per generated
token after the first, ``e2e`` the time from submission to the end.  Times are seconds on the
scheduler's clock; a span with a missing end is NaN.
"""

from __future__ import annotations

from dataclasses import dataclass, field

NAN = float("nan")


def _span(start: float, end: float) -> float:
    """end - start, or NaN while the end has not happened (its stamp is still 0)."""
    return end - start if end else NAN


def percentile(values, p: float) -> float:
    """The p-quantile (0 <= p <= 1) with linear interpolation between the two nearest order
    statistics; NaN for no values."""
    ordered = sorted(values)
    if not ordered:
        return NAN
    rank = p * (len(ordered) - 1)
    below = int(rank)
    above = min(below + 1, len(ordered) - 1)
    weight = rank - below
    return ordered[below] + (ordered[above] - ordered[below]) * weight


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
        return _span(self.t_submit, self.t_first_token)

    @property
    def e2e(self) -> float:
        return _span(self.t_submit, self.t_done)

    @property
    def tpot(self) -> float:
        later = self.generated_tokens - 1           # tokens after the first
        if later < 1 or not self.t_first_token:
            return NAN
        return _span(self.t_first_token, self.t_done) / later

    @property
    def cache_hit_rate(self) -> float:
        return self.cached_prefix_tokens / max(1, self.prompt_tokens)

    def as_dict(self) -> dict:
        out = {name: getattr(self, name) for name in (
            "req_id", "prompt_tokens", "generated_tokens", "cached_prefix_tokens",
            "prefill_tokens_computed", "preemptions", "finish_reason")}
        out.update(ttft=round(self.ttft, 5), tpot=round(self.tpot, 6), e2e=round(self.e2e, 5),
                   cache_hit_rate=round(self.cache_hit_rate, 4), output_ids=list(self.output_ids))
        return out

    @classmethod
    def of(cls, seq) -> "RequestRecord":
        """The record of a scheduler's sequence state."""
        return cls(req_id=seq.req_id, prompt_tokens=len(seq.request.prompt_ids),
                   generated_tokens=len(seq.output_ids),
                   cached_prefix_tokens=seq.cached_prefix_tokens,
                   prefill_tokens_computed=seq.prefill_tokens_computed,
                   preemptions=seq.preemptions, finish_reason=seq.finish_reason,
                   output_ids=list(seq.output_ids), t_submit=seq.t_submit, t_admit=seq.t_admit,
                   t_first_token=seq.t_first_token, t_done=seq.t_done)


def summarise(records: list[RequestRecord], wall_s: float) -> dict:
    """Totals and latency quantiles over the requests that finished within ``wall_s`` seconds."""
    done = [r for r in records if r.t_done]
    per_second = (lambda n: n / wall_s) if wall_s > 0 else (lambda n: 0.0)
    known = lambda xs: [x for x in xs if x == x]            # noqa: E731  (drops NaN)
    ttft, tpot, e2e = (known(getattr(r, name) for r in done) for name in ("ttft", "tpot", "e2e"))
    prompt = sum(r.prompt_tokens for r in done)
    saved = sum(r.cached_prefix_tokens for r in done)
    return {
        "n_requests": len(done),
        "wall_s": round(wall_s, 4),
        "throughput_tok_s": round(per_second(sum(r.generated_tokens for r in done)), 2),
        "request_throughput": round(per_second(len(done)), 3),
        "ttft_p50": percentile(ttft, 0.5), "ttft_p95": percentile(ttft, 0.95),
        "tpot_p50": percentile(tpot, 0.5),
        "e2e_p50": percentile(e2e, 0.5), "e2e_p95": percentile(e2e, 0.95),
        "cache_hit_rate": round(saved / prompt, 4) if prompt else 0.0,
        "prefill_tokens_saved": saved,
        "preemptions": sum(r.preemptions for r in done),
    }
