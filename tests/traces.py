"""Builds replay traces for the ways of cutting the same requests into steps, and checks a
replay's output files against the plain implementation.

A trace is a list of step records as ``bin/trace_run`` reads them.  Every driver returns
``(steps, index)`` where ``index[step] = [(request, position), ...]`` names the rows of that
step's output file.
"""

from __future__ import annotations

import io
import json
from pathlib import Path

import numpy as np
import torch


def whole(requests: dict[str, list[int]]):
    """Each request alone and whole: one step, every position wanted."""
    steps, index = [], {}
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
        index[i] = [(rid, p) for p in range(len(toks))]
    return steps, index


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps, index = [], {}
    n = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head],
                                              "want": [head - 1]}], "end": []})
        index[n] = [(rid, head - 1)]
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            index[n] = [(rid, p)]
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps, index


def portions(requests, sizes=(24, 7, 2, 16, 3, 2, 31, 5, 2, 9)):
    """Portions of changing size, down to two tokens; first and last place of each wanted."""
    steps, index = [], {}
    n = 0
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            size = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            want = sorted({0, size - 1})
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + size],
                                                  "want": want}],
                          "end": [rid] if at + size == len(toks) else []})
            index[n] = [(rid, at + w) for w in want]
            at += size
            n += 1
    return steps, index


def mixed(requests, seed=0, max_live=4, sizes=(1, 1, 2, 5, 1, 17, 3, 1, 9, 2, 30)):
    """Up to ``max_live`` requests live at a time: portions of some beside single tokens of
    others; a request may sit a step out; finished requests give their pages back and the
    next ones take them.  Returns also the peak of live tokens (rounded up per request to
    64), the pool size that forces reuse."""
    rng = np.random.default_rng(seed)
    order = list(requests)
    waiting = list(order)
    live: dict[str, int] = {}
    steps, index = [], {}
    n, peak = 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, rows, end = [], [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue                                  # sits this step out
            toks, at = requests[rid], live[rid]
            size = min(int(sizes[int(rng.integers(len(sizes)))]), len(toks) - at)
            want = sorted({0, size - 1}) if rng.random() < 0.8 else []
            entries.append({"id": rid, "tokens": toks[at:at + size], "want": want})
            rows += [(rid, at + w) for w in want]
            live[rid] = at + size
            if live[rid] == len(toks):
                end.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(-(-v // 64) * 64 for v in live.values()))
        steps.append({"step": n, "entries": entries, "end": end})
        if rows:
            index[n] = rows
        for rid in end:
            del live[rid]
        n += 1
    return steps, index, peak


def shared_prefix(requests, first: str, second: str, shared: int, portion=24):
    """``second`` begins with the first ``shared`` tokens of ``first`` (a multiple of the page
    size).  ``first`` runs whole and ends; ``second`` then comes in portions of ``portion``:
    with prefix reuse its first ``shared`` tokens are served from the pages ``first`` left, so
    only places behind them are wanted.  A third request, if any, runs beside it."""
    a, b = requests[first], requests[second]
    assert a[:shared] == b[:shared]
    steps = [{"step": 0, "entries": [{"id": first, "tokens": a, "want": list(range(len(a)))}],
              "end": [first]}]
    index = {0: [(first, p) for p in range(len(a))]}
    others = [r for r in requests if r not in (first, second)]
    at, n = 0, 1
    while at < len(b):
        size = min(portion, len(b) - at)
        want = [w for w in range(size) if at + w >= shared]
        entries = [{"id": second, "tokens": b[at:at + size], "want": want}]
        rows = [(second, at + w) for w in want]
        for r in others:                                  # a neighbour decoding token by token
            k = n - 1
            if k < len(requests[r]):
                entries.append({"id": r, "tokens": [requests[r][k]], "want": [0]})
                rows.append((r, k))
        steps.append({"step": n, "entries": entries, "end": []})
        index[n] = rows
        at += size
        n += 1
    steps.append({"step": n, "entries": [], "end": [second] + others})
    return steps, index


def drop_and_recompute(requests, victim: str, drop_after=2, portion=24):
    """Every request is prefilled in portions side by side; after ``drop_after`` steps the
    victim is dropped (preempted) and, one step later, fed again from its first token while
    the others go on: its pages were given back and are taken again."""
    at = {r: 0 for r in requests}
    steps, index = [], {}
    n = 0
    dropped = False
    while any(at[r] < len(t) for r, t in requests.items()):
        entries, rows = [], []
        sit_out = victim if (dropped and n == drop_after + 1) else None
        for r, toks in requests.items():
            if at[r] >= len(toks) or r == sit_out:
                continue
            size = min(portion if r != victim else portion // 2 + 1, len(toks) - at[r])
            want = sorted({0, size - 1})
            entries.append({"id": r, "tokens": toks[at[r]:at[r] + size], "want": want})
            rows += [(r, at[r] + w) for w in want]
            at[r] += size
        rec = {"step": n, "entries": entries, "end": []}
        if n == drop_after and not dropped:
            rec["drop"] = [victim]
            at[victim] = 0
            dropped = True
        steps.append(rec)
        if rows:
            index[n] = rows
        n += 1
    steps.append({"step": n, "entries": [], "end": list(requests)})
    return steps, index


def lines_of(steps) -> io.StringIO:
    return io.StringIO("".join(json.dumps(s) + "\n" for s in steps))


def collect(out_dir, index, vocab) -> dict[tuple[str, int], np.ndarray]:
    """Read the ``<step>.f32`` files back as {(request, position): logits}."""
    got = {}
    for step, rows in index.items():
        data = np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {step}: {data.size} floats for {len(rows)} rows"
        data = data.reshape(len(rows), vocab)
        for i, key in enumerate(rows):
            got[key] = data[i]
    return got


def worst_error(got, plain_logits: dict[str, torch.Tensor]):
    """Largest absolute difference to the plain logits, and where it is."""
    worst, where = 0.0, None
    for (rid, pos), row in sorted(got.items()):
        ref = plain_logits[rid][pos].numpy()
        err = float(np.abs(row.astype(np.float64) - ref).max())
        if not np.isfinite(row).all():
            err = float("inf")
        if err > worst:
            worst, where = err, (rid, pos)
    return worst, where
