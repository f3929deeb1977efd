"""The Python entry point: a model folder in, generated token ids out.

    engine = LLMEngine("path/to/model", dtype="bfloat16", num_blocks=512)
    record = engine.submit(Request(prompt_ids=[...], max_new_tokens=32))
    outputs = engine.generate([[...], [...]], max_new_tokens=16, temperature=0.8, seed=1)

``Request`` and ``RequestRecord`` carry the reference's names
(heteroserve/sched/router.py:36-44, heteroserve/metrics.py:31-68); ``submit`` is the
reference's ``Router.submit(Request) -> RequestRecord`` (router.py:404-406) without the
processes and sockets in between.  ``submit_nowait`` / ``step`` / ``has_work`` expose the
continuous-batching loop for callers that feed requests while others run.
"""

from __future__ import annotations

import tempfile
from dataclasses import replace
from pathlib import Path
from typing import Sequence

from ..config import EngineConfig, preset
from ..weights import write_model_dir
from .loading import TORCH_DTYPES, load_model
from .metrics import RequestRecord, summarise
from .scheduler import Request, Scheduler, SequenceState
from .step import Runner, StepEntry


class LLMEngine:
    def __init__(self, model_dir: str | Path, config: EngineConfig | None = None, *, ops=None,
                 **overrides):
        cfg = config or EngineConfig()
        if overrides:
            cfg = replace(cfg, **overrides)
        self.config = cfg
        self.model, self.model_config = load_model(model_dir, cfg.dtype, cfg.device)
        spec = self.model.spec
        self.runner = Runner(
            self.model, num_pages=cfg.num_blocks, page_size=cfg.block_size,
            max_requests=cfg.live_requests, dtype=TORCH_DTYPES[cfg.dtype], device=cfg.device,
            ops=ops, prefix_cache=cfg.prefix_cache, cuda_graphs=cfg.cuda_graphs,
            fused_decode=cfg.fused_decode)
        max_ctx = min(cfg.max_ctx or spec.max_positions, spec.max_positions)
        self.scheduler = Scheduler(
            self.runner.manager, self._run_step, max_batch=cfg.max_batch,
            max_prefill_tokens=cfg.max_prefill_tokens, max_ctx=max_ctx,
            eos_token_id=spec.eos_token_id, policy=cfg.policy, vocab_size=spec.vocab_size,
            pipeline=cfg.pipeline)
        self._tmp = None

    # -- construction --------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir, **kw) -> "LLMEngine":
        return cls(model_dir, **kw)

    @classmethod
    def random(cls, model: str | dict, seed: int = 0, *, store_dtype: str | None = None,
               **kw) -> "LLMEngine":
        """Random-weights mode: write a model folder for a preset name or a config.json
        dictionary (``model``) and a seed into a temporary folder, then load it like any other;
        ``config=EngineConfig(...)`` or single engine options go through as for the constructor."""
        raw = preset(model) if isinstance(model, str) else dict(model)
        tmp = tempfile.TemporaryDirectory(prefix="hetero_serve_b200-")
        dtype = kw.get("dtype", (kw.get("config") or EngineConfig()).dtype)
        write_model_dir(tmp.name, raw, seed, store_dtype or ("bfloat16" if str(dtype).startswith("b") else "float32"))
        eng = cls(tmp.name, **kw)
        eng._tmp = tmp
        return eng

    # -- the loop -------------------------------------------------------------------
    def _run_step(self, entries: list[StepEntry]):
        """Launch a step with device sampling.  The copy of its tokens to the host is enqueued
        behind it; the scheduler asks for them (``tokens_host``) when it needs them — with
        ``pipeline``, after it has launched the following step."""
        res = self.runner.step(entries, sample=True)
        res.start_fetch()
        return res

    def submit_nowait(self, request: Request) -> SequenceState:
        return self.scheduler.add(request)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> list[RequestRecord]:
        """One scheduler iteration; returns the records of requests whose end became known in
        it (with ``pipeline`` that is one call after the step that produced their last token)."""
        return [RequestRecord.of(s) for s in self.scheduler.step()]

    def run_until_done(self) -> list[RequestRecord]:
        out: list[RequestRecord] = []
        while self.scheduler.has_work():
            out.extend(self.step())
        return out

    def submit(self, request: Request) -> RequestRecord:
        """Run until this request has finished (others in flight advance too)."""
        seq = self.submit_nowait(request)
        while seq.state != "done":
            self.step()
        return RequestRecord.of(seq)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 32,
                 temperature: float = 0.0, top_k: int = 0, seed: int = 0,
                 stop_at_eos: bool = True) -> list[list[int]]:
        """Generate for several prompts at once; returns the new token ids of each."""
        seqs = [self.submit_nowait(Request(list(p), max_new_tokens, temperature, top_k,
                                           seed + i, stop_at_eos))
                for i, p in enumerate(prompts)]
        self.run_until_done()
        return [list(s.output_ids) for s in seqs]

    def state_message(self) -> dict:
        msg = self.scheduler.state_message()
        msg["engine"] = f"hetero_serve_b200/{self.config.dtype}"
        msg["device"] = self.config.device
        return msg

    def summarise(self, records: list[RequestRecord], wall_s: float) -> dict:
        return summarise(records, wall_s)
