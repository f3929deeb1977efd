"""Trace replay on the GPU, in 32-bit and in bfloat16, against the plain implementation:
each request whole; most of it in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; and up to four live requests mixed, with so few pages
that they are used again.  Also: every cut gives the same logits as the whole request."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import traces
from conftest import ROOT, TOL
from hetero_serve_b200.engine.replay import replay

pytestmark = pytest.mark.gpu


def _requests(tiny, base=100):
    lens = {"tiny_a": (5, 17, 33, 70, 128), "tiny_b": (1, 16, 31, 70, 200)}[tiny.name]
    return {f"r{i}": tiny.tokens(n, base + i) for i, n in enumerate(lens)}


def _replay(tiny, dtype, steps, out, max_tokens, **kw):
    import io
    out.mkdir(parents=True, exist_ok=True)
    rep = io.StringIO()
    assert replay(model_dir=tiny.dir, dtype=dtype, out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=rep, **kw) == 0
    assert rep.getvalue().count("done ") == len(steps)
    return out


def _plain(tiny, reqs, dtype):
    return {r: tiny.logits(t, dtype) for r, t in reqs.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_agrees_with_the_plain_model_and_with_the_whole_request(tiny, tmp_path, dtype):
    reqs = _requests(tiny)
    V = tiny.config["vocab_size"]
    plain = _plain(tiny, reqs, dtype)
    results = {}
    for name, make in (("whole", traces.whole), ("tail", traces.tail_one_by_one),
                       ("portions", traces.portions)):
        steps, index = make(reqs)
        out = _replay(tiny, dtype, steps, tmp_path / name, max_tokens=256)
        got = traces.collect(out, index, V)
        err, where = traces.worst_error(got, plain)
        assert err < TOL[dtype], (name, err, where)
        results[name] = got
    # The logits at a position do not depend on how the tokens were cut into steps.  In 32-bit
    # every kernel's order of summation depends on the element alone (k order in the linears,
    # key order in the attention), so the cuts agree bit for bit; in bfloat16 the few-row and
    # the tensor-core kernels order their sums differently, so they agree to rounding.
    for name in ("tail", "portions"):
        for key, row in results[name].items():
            if dtype == "float32":
                assert np.array_equal(row, results["whole"][key]), (name, key)
            else:
                assert np.abs(row - results["whole"][key]).max() <= 2e-2, (name, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_requests_with_reused_pages(tiny, tmp_path, dtype):
    lens = (40, 9, 64, 23, 70, 3, 55, 31, 100, 12)
    reqs = {f"m{i}": tiny.tokens(n, 300 + i) for i, n in enumerate(lens)}
    steps, index, peak = traces.mixed(reqs, seed=2)
    out = _replay(tiny, dtype, steps, tmp_path / "mixed", max_tokens=peak)
    got = traces.collect(out, index, tiny.config["vocab_size"])
    assert len(got) > 60
    err, where = traces.worst_error(got, _plain(tiny, reqs, dtype))
    assert err < TOL[dtype], (err, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_hit_changes_no_logit(tiny_models, tmp_path, dtype):
    """Tiny B's prompts of 16 and 70 tokens share their first 16 tokens: with prefix reuse the
    second one's first page is the first one's, and every logit behind it equals the plain
    model's (the reference's counterpart: tests/test_model.py:173-193)."""
    tiny = tiny_models["tiny_b"]
    p2 = tiny.tokens(16, 31)
    reqs = {"p2": p2, "p4": p2 + tiny.tokens(54, 32), "n": tiny.tokens(9, 33)}
    steps, index = traces.shared_prefix(reqs, "p2", "p4", 16)
    plain = _plain(tiny, reqs, dtype)
    rows = {}
    for cache in (True, False):
        out = _replay(tiny, dtype, steps, tmp_path / f"hit{int(cache)}", max_tokens=192,
                      prefix_cache=cache)
        if cache:
            stats = json.loads((out / "replay_stats.json").read_text())
            assert stats["hit_tokens"] == 16
        rows[cache] = traces.collect(out, index, tiny.config["vocab_size"])
        err, where = traces.worst_error(rows[cache], plain)
        assert err < TOL[dtype], (cache, err, where)
    if dtype == "float32":          # served from the cache or computed: the same bits
        for key, row in rows[True].items():
            assert np.array_equal(row, rows[False][key]), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_dropped_request_is_recomputed(tiny, tmp_path, dtype):
    """A live request is preempted in the middle of its prompt (pages given back) and fed
    again from its first token beside the others (the reference's counterpart:
    heteroserve/worker/worker.py:738-757)."""
    reqs = {"a": tiny.tokens(60, 41), "v": tiny.tokens(50, 42), "c": tiny.tokens(33, 43)}
    steps, index = traces.drop_and_recompute(reqs, "v")
    plain = _plain(tiny, reqs, dtype)
    for cache in (False, True):
        out = _replay(tiny, dtype, steps, tmp_path / f"drop{int(cache)}", max_tokens=192,
                      prefix_cache=cache)
        got = traces.collect(out, index, tiny.config["vocab_size"])
        err, where = traces.worst_error(got, plain)
        assert err < TOL[dtype], (cache, err, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny_models, tmp_path, dtype):
    """One token at a time from the very first position to the end of the table: every page
    edge, every position of the table."""
    tiny = tiny_models["tiny_b"]
    toks = tiny.tokens(256, 7)
    reqs = {"long": toks}
    steps, index = traces.tail_one_by_one(reqs, tail=255)
    out = _replay(tiny, dtype, steps, tmp_path / "long", max_tokens=256)
    got = traces.collect(out, index, 1000)
    assert sorted(p for _, p in got) == list(range(256))
    err, where = traces.worst_error(got, _plain(tiny, reqs, dtype))
    assert err < TOL[dtype], (err, where)


def test_trace_run_program_as_a_user_calls_it(tiny_models, tmp_path):
    """The executable itself, fed through a pipe step by step, waiting for `done`."""
    tiny = tiny_models["tiny_a"]
    reqs = {"a": tiny.tokens(37, 1), "b": tiny.tokens(20, 2)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": reqs["a"][30:32], "want": [1]},
                                {"id": "b", "tokens": reqs["b"], "want": [19]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": reqs["a"][32:], "want": []}], "end": []},
        {"step": 3, "entries": [], "end": ["a"]},
    ]
    out = tmp_path / "o"
    env = dict(os.environ, PYTHONUNBUFFERED="1")
    proc = subprocess.Popen(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", tiny.dir, "--dtype",
         "float32", "--out", str(out), "--max-tokens", "128"],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for s in steps:
        proc.stdin.write(json.dumps(s) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {s['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32"]
    index = {0: [("a", 0), ("a", 29)], 1: [("a", 31), ("b", 19)]}
    got = traces.collect(out, index, 512)
    err, where = traces.worst_error(got, _plain(tiny, reqs, "float32"))
    assert err < TOL["float32"], (err, where)
