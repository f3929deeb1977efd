"""Trace replay: feeds given token ids through the step function and writes logits.

It has no forward pass, cache or loader of its own: the model comes from
:func:`load_model`, the batch runs through :meth:`Runner.step`, the pages come from the
runner's cache manager — the objects generation uses.

By default prefix reuse is off, so every token a step brings is actually run.  With
``prefix_cache`` the replay does what the scheduler does around the step function
(heteroserve/worker/worker.py:378-416, 635-645, 738-757): a request's first entry is
matched against the published pages and only the tokens behind the match are run; after
every step the full pages of the requests in it are published; a request named in a step's
``drop`` list is preempted — its full pages stay findable, everything it holds is given
back, and the trace feeds it again from its first token later.
"""

from __future__ import annotations

import json
import os
from typing import IO, Iterable

import torch

from .loading import TORCH_DTYPES, load_model
from .step import Runner, StepEntry, StepError

DEFAULT_LIVE_REQUESTS = 8


def replay(*, model_dir, dtype: str, out_dir, max_tokens: int, lines: Iterable[str],
           report: IO[str], page_size: int = 16, device="cuda:0", ops=None,
           prefix_cache: bool = False, max_requests: int = DEFAULT_LIVE_REQUESTS) -> int:
    model, _cfg = load_model(model_dir, dtype, device)
    num_pages = max(1, -(-int(max_tokens) // page_size))
    runner = Runner(model, num_pages=num_pages, page_size=page_size,
                    max_requests=max_requests, dtype=TORCH_DTYPES[dtype], device=device,
                    ops=ops, prefix_cache=prefix_cache, cuda_graphs=False)
    mgr = runner.manager
    fed: dict = {}                      # request -> every token fed so far (for publishing)
    stats = {"hit_tokens": 0, "run_tokens": 0, "dropped": 0}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", ()):
            rid, tokens, want = e["id"], list(e["tokens"]), list(e.get("want", ()))
            skip = 0
            if rid not in mgr:
                fed[rid] = []
                if prefix_cache:
                    skip = runner.open(rid, tokens)
                    if any(w < skip for w in want):
                        raise StepError(
                            f"step {step}, request {rid!r}: place {min(want)} lies in the "
                            f"{skip} tokens served from the prefix cache; nothing is run there")
                    stats["hit_tokens"] += skip
            fed[rid].extend(tokens)
            stats["run_tokens"] += len(tokens) - skip
            entries.append(StepEntry(rid, tokens[skip:], [w - skip for w in want]))
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
            if prefix_cache:
                for e in entries:
                    mgr.publish(e.req_id, fed[e.req_id])
        for rid in rec.get("drop", ()):
            if rid not in mgr:
                raise StepError(f"step {step}: request {rid!r} is dropped but not live")
            mgr.publish(rid, fed[rid])
            runner.close(rid)
            fed.pop(rid, None)
            stats["dropped"] += 1
        for rid in rec.get("end", ()):
            if rid in mgr:
                mgr.publish(rid, fed.get(rid, ()))
                runner.close(rid)
            fed.pop(rid, None)
        report.write(f"done {step}\n")
        report.flush()
    if prefix_cache:
        with open(os.path.join(out_dir, "replay_stats.json"), "w") as fh:
            json.dump(stats, fh)
    return 0
