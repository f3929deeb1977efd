"""Trace replay: feeds given token ids through the step function and writes logits.

It has no forward pass, cache or loader of its own: the model comes from
:func:`load_model`, the batch runs through :meth:`Runner.step`, the pages come from the
runner's cache manager — the objects generation uses.  Prefix reuse is off, so every
token a step brings is actually run.
"""

from __future__ import annotations

import json
import os
from typing import IO, Iterable

import torch

from .loading import TORCH_DTYPES, load_model
from .step import Runner, StepEntry

MAX_LIVE_REQUESTS = 8


def replay(*, model_dir, dtype: str, out_dir, max_tokens: int, lines: Iterable[str],
           report: IO[str], page_size: int = 16, device="cuda:0", ops=None) -> int:
    model, _cfg = load_model(model_dir, dtype, device)
    num_pages = max(1, -(-int(max_tokens) // page_size))
    runner = Runner(model, num_pages=num_pages, page_size=page_size,
                    max_requests=MAX_LIVE_REQUESTS, dtype=TORCH_DTYPES[dtype], device=device,
                    ops=ops, prefix_cache=False, cuda_graphs=False)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ()))
                   for e in rec.get("entries", ())]
        if entries:
            res = runner.step(entries)
            if res.logits is not None and res.logits.shape[0]:
                data = res.logits.to(torch.float32).cpu().contiguous().numpy()
                path = os.path.join(out_dir, f"{step}.f32")
                with open(path + ".tmp", "wb") as fh:
                    fh.write(data.astype("<f4", copy=False).tobytes())
                os.replace(path + ".tmp", path)
            elif runner.cuda:
                runner.check_status()
        for rid in rec.get("end", ()):
            if rid in runner.manager:
                runner.close(rid)
        report.write(f"done {step}\n")
        report.flush()
    return 0
