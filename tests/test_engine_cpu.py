"""The step function, the cache and the replay driver without a GPU: the kernels are
replaced by their plain PyTorch twins (tests/plain_ops.py) on CPU tensors, everything
else — model assembly, metadata, pages, block tables — is the product's own code."""

import pytest
import torch

import plain_ops
import traces
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry, StepError
from hetero_serve_b200.cache import OutOfPages

TOL = 2e-5


def _requests(tiny):
    lens = {"tiny_a": (5, 17, 33, 70), "tiny_b": (1, 16, 31, 70, 45)}[tiny.name]
    return {f"r{i}": tiny.tokens(n, 100 + i) for i, n in enumerate(lens)}


def _replay(tiny, steps, tmp_path, max_tokens, **kw):
    out = tmp_path / "out"
    out.mkdir(exist_ok=True)
    import io
    rep = io.StringIO()
    assert replay(model_dir=tiny.dir, dtype="float32", out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=rep, device="cpu",
                  ops=plain_ops.PlainOps(), **kw) == 0
    assert rep.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    return out


@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(tiny, tmp_path, driver):
    reqs = _requests(tiny)
    make = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions}
    steps, index = make[driver](reqs)
    out = _replay(tiny, steps, tmp_path, max_tokens=128)
    got = traces.collect(out, index, tiny.config["vocab_size"])
    err, where = traces.worst_error(got, {r: tiny.logits(t) for r, t in reqs.items()})
    assert err < TOL, (err, where)


def test_mixed_batches_with_page_reuse(tiny, tmp_path):
    reqs = {f"r{i}": tiny.tokens(n, 200 + i) for i, n in
            enumerate((40, 9, 64, 23, 70, 3, 55, 31))}
    steps, index, peak = traces.mixed(reqs, seed=1)
    assert peak <= 4 * 128
    out = _replay(tiny, steps, tmp_path, max_tokens=peak)      # so few pages that they are reused
    got = traces.collect(out, index, tiny.config["vocab_size"])
    assert len(got) > 40
    err, where = traces.worst_error(got, {r: tiny.logits(t) for r, t in reqs.items()})
    assert err < TOL, (err, where)


def test_prefix_hit_in_a_replay_changes_no_logit(tiny_models, tmp_path):
    """Tiny B's prompts of 16 and 70 tokens share their first 16: the second request's first
    page comes from the cache, and every logit behind it equals the plain model's."""
    import json
    tiny = tiny_models["tiny_b"]
    p2 = tiny.tokens(16, 31)
    reqs = {"p2": p2, "p4": p2 + tiny.tokens(54, 32), "n": tiny.tokens(9, 33)}
    steps, index = traces.shared_prefix(reqs, "p2", "p4", 16)
    out = _replay(tiny, steps, tmp_path, max_tokens=192, prefix_cache=True)
    stats = json.loads((out / "replay_stats.json").read_text())
    assert stats["hit_tokens"] == 16 and stats["run_tokens"] == 16 + 54 + 3
    got = traces.collect(out, index, tiny.config["vocab_size"])
    err, where = traces.worst_error(got, {r: tiny.logits(t) for r, t in reqs.items()})
    assert err < TOL, (err, where)


def test_dropped_request_is_recomputed_in_a_replay(tiny, tmp_path):
    reqs = {"a": tiny.tokens(60, 41), "v": tiny.tokens(50, 42), "c": tiny.tokens(33, 43)}
    steps, index = traces.drop_and_recompute(reqs, "v")
    assert any("drop" in s for s in steps)
    for cache in (False, True):
        out = _replay(tiny, steps, tmp_path, max_tokens=192, prefix_cache=cache)
        got = traces.collect(out, index, tiny.config["vocab_size"])
        err, where = traces.worst_error(got, {r: tiny.logits(t) for r, t in reqs.items()})
        assert err < TOL, (cache, err, where)


def _runner(tiny, pages=8, **kw):
    model, _ = load_model(tiny.dir, "float32", "cpu")
    return Runner(model, num_pages=pages, page_size=16, max_requests=4, dtype=torch.float32,
                  device="cpu", ops=plain_ops.PlainOps(), **kw)


def test_step_refuses_what_it_cannot_run(tiny_models):
    tiny = tiny_models["tiny_a"]
    rn = _runner(tiny, pages=2)
    with pytest.raises(StepError, match="twice"):
        rn.step([StepEntry("a", [1]), StepEntry("a", [2])])
    with pytest.raises(StepError, match="outside"):
        rn.step([StepEntry("a", [1, 2], want=[2])])
    with pytest.raises(StepError, match="token id"):
        rn.step([StepEntry("a", [512])])
    with pytest.raises(StepError, match="no tokens"):
        rn.step([StepEntry("a", [])])
    with pytest.raises(OutOfPages):
        rn.step([StepEntry("b", [1] * 33)])
    rn2 = _runner(tiny, pages=16)
    with pytest.raises(StepError, match="exceed"):
        rn2.step([StepEntry("a", [1] * 129)])
    rn.manager.check()


def test_pages_are_reused_with_stale_contents(tiny_models):
    """A page that held another request's keys must not leak into the next one."""
    tiny = tiny_models["tiny_b"]
    rn = _runner(tiny, pages=3)
    a, b = tiny.tokens(40, 1), tiny.tokens(37, 2)
    rn.step([StepEntry("a", a)])
    rn.close("a")
    res = rn.step([StepEntry("b", b, want=[36])])
    assert (res.logits[0].double() - tiny.logits(b)[36]).abs().max() < TOL


def test_sampling_through_the_step_matches_the_plain_sampler(tiny_models):
    import plain_gpt2
    tiny = tiny_models["tiny_b"]
    rn = _runner(tiny)
    toks = tiny.tokens(12, 9)
    res = rn.step([StepEntry("a", toks, want=[11], temperature=0.8, top_k=40, seed=77),
                   StepEntry("b", toks[:5], want=[4], temperature=0.0)], sample=True)
    got = res.tokens_host()
    u = plain_gpt2.uniform_for(77, 12)
    assert got[0] == plain_gpt2.sample_token(tiny.logits(toks)[11], 0.8, 40, u)
    assert got[1] == int(torch.argmax(tiny.logits(toks[:5])[4]))


def test_a_token_can_be_taken_from_the_device_copy(tiny_models):
    """FROM_DEVICE as the first token of an entry stands for the token the latest sampling step
    left on the device for that request: two requests decode three steps each without the host
    feeding their tokens back, and get the logits of a replay that knows the tokens."""
    from hetero_serve_b200.engine.step import FROM_DEVICE
    tiny = tiny_models["tiny_b"]
    rn = _runner(tiny, pages=12)
    a, b = tiny.tokens(9, 4), tiny.tokens(20, 5)
    first = rn.step([StepEntry("a", a, want=[8]), StepEntry("b", b, want=[19], temperature=0.7,
                                                           seed=3)], sample=True)
    ctx = {"a": list(a) + [first.tokens_host()[0]], "b": list(b) + [first.tokens_host()[1]]}
    for _ in range(3):
        res = rn.step([StepEntry("b", [FROM_DEVICE], want=[0], temperature=0.7, seed=3),
                       StepEntry("a", [FROM_DEVICE], want=[0])], sample=True)
        lg = res.logits.double().clone()
        tb, ta = res.tokens_host()
        assert (lg[0] - tiny.logits(ctx["b"])[-1]).abs().max() < TOL
        assert (lg[1] - tiny.logits(ctx["a"])[-1]).abs().max() < TOL
        ctx["a"].append(ta)
        ctx["b"].append(tb)
    # known tokens may follow the device token in the same entry; a device token elsewhere is refused
    res = rn.step([StepEntry("a", [FROM_DEVICE, 7, 9], want=[2])])
    assert (res.logits[0].double() - tiny.logits(ctx["a"] + [7, 9])[-1]).abs().max() < TOL
    with pytest.raises(StepError, match="token id"):
        rn.step([StepEntry("b", [3, FROM_DEVICE])])
    rn.manager.check()


def test_size_classes_bound_the_padding():
    """Counts are rounded up to size classes where shapes must repeat: never below the count,
    monotone, powers of two up to 8, then four classes per doubling (padding under a quarter)."""
    from hetero_serve_b200.kernels.ops import size_class
    assert [size_class(n) for n in (1, 2, 3, 5, 8)] == [1, 2, 4, 8, 8]
    assert [size_class(n) for n in (9, 16, 17, 33, 48, 49, 64, 65, 2048, 2049)] == \
        [10, 16, 20, 40, 48, 56, 64, 80, 2048, 2560]
    last = 0
    classes = set()
    for n in range(1, 5000):
        c = size_class(n)
        assert c >= n and c >= last
        assert c == size_class(c)                  # a class is its own class
        if n > 8:
            assert (c - n) / n < 0.25
        last = c
        classes.add(c)
    assert len(classes) <= 4 + 4 * 10              # 8 .. 8192: ten doublings


def test_a_refused_step_leaves_the_cache_as_it_found_it(tiny_models):
    """Pages run out at the THIRD entry of a step: what the first two took is given back, the
    request the step opened on its own is closed again, and the step can be run in two."""
    tiny = tiny_models["tiny_a"]
    rn = _runner(tiny, pages=5)
    a = tiny.tokens(40, 1)
    rn.step([StepEntry("a", a[:20])])                         # a holds 2 pages
    free, live = rn.manager.pages_free(), set(rn.manager.live())
    with pytest.raises(OutOfPages):
        rn.step([StepEntry("a", a[20:40]), StepEntry("b", [1] * 30), StepEntry("c", [2] * 20)])
    assert rn.manager.pages_free() == free and set(rn.manager.live()) == live
    assert rn.manager.length("a") == 20 and rn.manager.table_lengths("a") == [2]
    rn.manager.check()
    with pytest.raises(StepError, match="token id"):          # refused before anything is taken
        rn.step([StepEntry("a", a[20:40]), StepEntry("d", [1, 999])])
    assert rn.manager.pages_free() == free and "d" not in rn.manager
    res = rn.step([StepEntry("a", a[20:40], want=[19])])
    assert (res.logits[0].double() - tiny.logits(a)[39]).abs().max() < TOL
    rn.manager.check()
