"""The scheduler's decisions (no GPU): admission, portions under a token budget, decoding,
finishing and freeing, and what happens when pages run out.  The step function is replaced
by a fake that reserves and commits pages like the real one and returns tokens that depend
only on (last token fed, position, seed), so any batching must give the same outputs."""

import pytest

from hetero_serve_b200.cache import CacheManager, GroupSpec
from hetero_serve_b200.engine.scheduler import Request, RequestRefused, Scheduler, SeqState

VOCAB = 97


class FakeStep:
    def __init__(self, manager):
        self.manager = manager
        self.log = []            # per step: [(req_id, start, n_tokens, wants)]

    def __call__(self, entries):
        out, rec = [], []
        for e in entries:
            start = self.manager.length(e.req_id)
            self.manager.reserve(e.req_id, start + len(e.tokens))
            self.manager.commit(e.req_id, start + len(e.tokens))
            rec.append((e.req_id, start, len(e.tokens), bool(e.want)))
            for w in e.want:
                out.append((e.tokens[w] * 7 + (start + w + 1) * 13 + e.seed) % VOCAB)
        self.log.append(rec)
        return out


def make(num_pages=64, page_size=4, max_requests=8, policy="prefill_first", max_batch=8,
         budget=24, max_ctx=200, eos=None, prefix_cache=True):
    mgr = CacheManager([GroupSpec()], num_pages, page_size, max_requests, prefix_cache)
    fake = FakeStep(mgr)
    sch = Scheduler(mgr, fake, max_batch=max_batch, max_prefill_tokens=budget, max_ctx=max_ctx,
                    eos_token_id=eos, policy=policy, vocab_size=VOCAB)
    return sch, fake, mgr


def run(sch, mgr, limit=10_000):
    n = 0
    while sch.has_work():
        sch.step()
        mgr.check()
        n += 1
        assert n < limit
    return n


def expected_outputs(prompt, n_new, seed=0, eos=None, max_ctx=10 ** 9):
    ctx, out = list(prompt), []
    while len(out) < n_new:
        tok = (ctx[-1] * 7 + len(ctx) * 13 + seed) % VOCAB
        out.append(tok); ctx.append(tok)
        if (eos is not None and tok == eos) or len(ctx) >= max_ctx:
            break
    return out


def prompt(n, base=1):
    return [(base + 3 * i) % VOCAB for i in range(n)]


def test_prompt_is_cut_into_portions_then_decoded():
    sch, fake, mgr = make(budget=24)
    seq = sch.add(Request(prompt(70), max_new_tokens=4))
    run(sch, mgr)
    shape = [[(s, n, w) for _, s, n, w in step] for step in fake.log]
    assert shape[:3] == [[(0, 24, False)], [(24, 24, False)], [(48, 22, True)]]
    assert shape[3:] == [[(70, 1, True)], [(71, 1, True)], [(72, 1, True)]]
    assert seq.output_ids == expected_outputs(prompt(70), 4)
    assert seq.state == SeqState.DONE and seq.finish_reason == "max_new_tokens"
    assert sch.stats.prefill_steps == 3 and sch.stats.decode_steps == 3
    assert mgr.pages_free() == 64 and mgr.free_slots() == 8     # everything given back


def test_prefill_first_gives_unfinished_prompts_priority():
    sch, fake, mgr = make(budget=16)
    a = sch.add(Request(prompt(10), max_new_tokens=6))
    sch.step(); sch.step()                       # a: prefill, one decode
    b = sch.add(Request(prompt(40, 5), max_new_tokens=2, seed=3))
    sch.step()
    assert [r for r, *_ in fake.log[-1]] == [b.req_id]           # b's portion, a waits
    sch.step(); sch.step()
    assert fake.log[-1][0][:3] == (b.req_id, 32, 8)
    sch.step()
    assert sorted(r for r, *_ in fake.log[-1]) == sorted([a.req_id, b.req_id])  # one decode batch
    run(sch, mgr)
    assert a.output_ids == expected_outputs(prompt(10), 6)
    assert b.output_ids == expected_outputs(prompt(40, 5), 2, seed=3)


def test_mixed_policy_puts_decodes_and_portions_in_one_step():
    sch, fake, mgr = make(budget=16, policy="mixed")
    a = sch.add(Request(prompt(10), max_new_tokens=8))
    sch.step()
    b = sch.add(Request(prompt(40, 5), max_new_tokens=2))
    sch.step()
    step = fake.log[-1]
    assert (a.req_id, 10, 1, True) in step                      # a's decoded token ...
    assert (b.req_id, 0, 15, False) in step                     # ... beside b's portion: 16 in all
    assert sum(n for _, _, n, _ in step) == 16
    run(sch, mgr)
    assert sch.stats.mixed_steps >= 2
    assert a.output_ids == expected_outputs(prompt(10), 8)
    assert b.output_ids == expected_outputs(prompt(40, 5), 2)


def test_max_batch_caps_a_decode_step():
    sch, fake, mgr = make(max_batch=2, budget=64)
    seqs = [sch.add(Request(prompt(5, i), max_new_tokens=3)) for i in range(3)]
    run(sch, mgr)
    assert max(len(step) for step in fake.log) <= 2
    for i, s in enumerate(seqs):
        assert s.output_ids == expected_outputs(prompt(5, i), 3)


def test_admission_waits_for_pages_in_arrival_order():
    sch, fake, mgr = make(num_pages=8, page_size=4, budget=64, prefix_cache=False)
    a = sch.add(Request(prompt(20), max_new_tokens=3))          # 5 pages, grows to 6
    b = sch.add(Request(prompt(14, 9), max_new_tokens=2))       # 4 pages: must wait
    c = sch.add(Request(prompt(3, 30), max_new_tokens=2))       # would fit, but is behind b
    sch.step()
    assert a.admitted and not b.admitted and not c.admitted
    run(sch, mgr)
    order = [r for step in fake.log for r, s, n, w in step if s == 0]
    assert order == [a.req_id, b.req_id, c.req_id]
    assert b.output_ids == expected_outputs(prompt(14, 9), 2)
    assert mgr.pages_free() == 8


def test_pages_run_out_newest_is_preempted_and_recomputed():
    kw = dict(page_size=4, budget=64, max_batch=4, prefix_cache=False)
    big, _, bm = make(num_pages=64, **kw)
    small, fake, sm = make(num_pages=8, **kw)                   # 32 token slots
    outs = {}
    for sch, mgr in ((big, bm), (small, sm)):
        a = sch.add(Request(prompt(10), max_new_tokens=12, seed=1))
        b = sch.add(Request(prompt(9, 4), max_new_tokens=12, seed=2))
        run(sch, mgr)
        outs[sch] = (a, b)
    a, b = outs[small]
    assert small.stats.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    # the newest (b) was the victim; it was prefilled again over prompt + outputs - 1
    again = [(r, s, n) for step in fake.log for r, s, n, w in step if r == b.req_id and s == 0]
    assert len(again) == 1 + b.preemptions and again[1][2] > 9
    for x, y in zip(outs[small], outs[big]):
        assert x.output_ids == y.output_ids and len(x.output_ids) == 12
    assert sm.pages_free() == 8


def test_preempted_request_goes_to_the_front():
    sch, fake, mgr = make(num_pages=6, page_size=4, budget=64, prefix_cache=False)
    a = sch.add(Request(prompt(8), max_new_tokens=12))
    b = sch.add(Request(prompt(8, 2), max_new_tokens=12))
    c = sch.add(Request(prompt(4, 7), max_new_tokens=2))
    seen_waiting_front = False
    while sch.has_work():
        sch.step(); mgr.check()
        if b.preemptions and b.state == SeqState.WAITING:
            assert sch.waiting[0] is b
            seen_waiting_front = True
    assert seen_waiting_front
    assert a.output_ids == expected_outputs(prompt(8), 12)
    assert b.output_ids == expected_outputs(prompt(8, 2), 12)
    assert c.output_ids == expected_outputs(prompt(4, 7), 2)


def test_request_that_outgrows_the_pool_ends_with_what_it_has():
    sch, _, mgr = make(num_pages=3, page_size=4, budget=64, prefix_cache=False)
    a = sch.add(Request(prompt(6), max_new_tokens=50))
    run(sch, mgr)
    assert a.finish_reason == "out_of_pages" and a.state == SeqState.DONE
    # 12 slots: positions 0..11 were resident, so tokens up to position 12 were sampled
    assert a.output_ids == expected_outputs(prompt(6), 7)
    assert mgr.pages_free() == 3 and mgr.free_slots() == 8


def test_finish_at_eos_and_at_the_context_limit():
    p = prompt(6)
    eos = expected_outputs(p, 3)[2]
    sch, _, mgr = make(eos=eos)
    s1 = sch.add(Request(p, max_new_tokens=10))
    s2 = sch.add(Request(p, max_new_tokens=10, stop_at_eos=False))
    run(sch, mgr)
    assert s1.output_ids == expected_outputs(p, 10, eos=eos) and s1.finish_reason == "eos"
    assert len(s1.output_ids) == 3 and len(s2.output_ids) == 10
    sch, _, mgr = make(max_ctx=12)
    s3 = sch.add(Request(p, max_new_tokens=50))
    run(sch, mgr)
    assert len(p) + len(s3.output_ids) == 12 and s3.finish_reason == "max_ctx"


def test_requests_that_can_never_run_are_refused():
    sch, _, _ = make(num_pages=4, page_size=4, max_ctx=32)
    with pytest.raises(RequestRefused, match="empty"):
        sch.add(Request([]))
    with pytest.raises(RequestRefused, match="context limit"):
        sch.add(Request(prompt(32)))
    with pytest.raises(RequestRefused, match="pages"):
        sch.add(Request(prompt(16)))            # 17 positions need 5 pages, the pool has 4
    with pytest.raises(RequestRefused, match="outside"):
        sch.add(Request([1, VOCAB]))
    with pytest.raises(RequestRefused, match="max_new_tokens"):
        sch.add(Request([1], max_new_tokens=0))


def test_prefix_reuse_skips_prefill_and_changes_nothing():
    sch, fake, mgr = make(page_size=4, budget=64)
    shared = prompt(22)
    a = sch.add(Request(shared + [5, 6], max_new_tokens=3))
    run(sch, mgr)
    b = sch.add(Request(shared + [9], max_new_tokens=3))
    run(sch, mgr)
    assert a.cached_prefix_tokens == 0 and b.cached_prefix_tokens == 20
    assert b.prefill_tokens_computed == 3
    assert b.output_ids == expected_outputs(shared + [9], 3)
    assert sch.state_message()["tokens_saved_by_cache"] == 20
    # an identical prompt: everything but its last page is reused, the last token is computed
    c = sch.add(Request(shared + [5, 6], max_new_tokens=3))
    run(sch, mgr)
    assert c.cached_prefix_tokens == 20 and c.output_ids == a.output_ids


def test_abort_gives_everything_back():
    sch, _, mgr = make()
    a = sch.add(Request(prompt(30), max_new_tokens=50))
    b = sch.add(Request(prompt(5), max_new_tokens=50))
    sch.step(); sch.step()
    assert sch.abort(a.req_id) and sch.abort(b.req_id) and not sch.abort("nobody")
    mgr.check()
    assert not sch.has_work() and mgr.free_slots() == 8


# ------------------------------------------------------------------ pipelined steps
class LazyFakeStep(FakeStep):
    """Like FakeStep, but the tokens come as an object that is read later, and an entry may
    bring FROM_DEVICE: the fake keeps "device memory" of the last token per request."""

    def __init__(self, manager):
        super().__init__(manager)
        self.device_last = {}
        self.unread = 0           # results handed out whose tokens have not been asked for
        self.max_unread = 0

    def __call__(self, entries):
        from hetero_serve_b200.engine.step import FROM_DEVICE
        fed = []
        for e in entries:
            toks = list(e.tokens)
            if toks[0] == FROM_DEVICE:
                toks[0] = self.device_last[e.req_id]
            assert all(0 <= t < VOCAB for t in toks)
            fed.append(type(e)(e.req_id, toks, e.want, e.temperature, e.top_k, e.seed))
        out = super().__call__(fed)
        it = iter(out)
        for e in entries:
            for w in e.want:
                tok = next(it)
                if w == len(e.tokens) - 1:
                    self.device_last[e.req_id] = tok
        fake = self
        fake.unread += 1
        fake.max_unread = max(fake.max_unread, fake.unread)

        class Later:
            def tokens_host(self_inner):
                fake.unread -= 1
                return out
        return Later()


def make_pipelined(pipeline, **kw):
    num_pages, page_size = kw.pop("num_pages", 64), kw.pop("page_size", 4)
    mgr = CacheManager([GroupSpec()], num_pages, page_size, kw.pop("max_requests", 8),
                       kw.pop("prefix_cache", True))
    fake = LazyFakeStep(mgr)
    sch = Scheduler(mgr, fake, max_batch=kw.pop("max_batch", 8),
                    max_prefill_tokens=kw.pop("budget", 24), max_ctx=kw.pop("max_ctx", 200),
                    eos_token_id=kw.pop("eos", None), policy=kw.pop("policy", "prefill_first"),
                    vocab_size=VOCAB, pipeline=pipeline)
    assert not kw
    return sch, fake, mgr


def test_pipelined_decoding_launches_before_it_reads():
    sch, fake, mgr = make_pipelined(True)
    seq = sch.add(Request(prompt(10), max_new_tokens=6))
    run(sch, mgr)
    assert seq.output_ids == expected_outputs(prompt(10), 6)
    assert fake.max_unread == 2          # a step was launched while the previous one was unread
    # the prompt, then five decode steps: the last token's end is known by counting, so no
    # step is launched for it
    assert [len(step) for step in fake.log] == [1] * 6
    assert mgr.pages_free() == 64 and mgr.free_slots() == 8
    sync, fake2, _ = make_pipelined(False)
    sync.add(Request(prompt(10), max_new_tokens=6))
    run(sync, _)
    shape = lambda log: [[r[1:] for r in step] for step in log]
    assert fake2.max_unread == 1 and shape(fake2.log) == shape(fake.log)


def test_pipelined_sees_eos_one_step_late_and_discards_the_extra_step():
    want = expected_outputs(prompt(9, base=5), 30)
    eos = want[3]
    assert eos not in want[:3]
    sch, fake, mgr = make_pipelined(True, eos=eos)
    seq = sch.add(Request(prompt(9, base=5), max_new_tokens=30))
    other = sch.add(Request(prompt(7, base=2), max_new_tokens=12))
    run(sch, mgr)
    assert seq.output_ids == want[:4] and seq.finish_reason == "eos"
    assert other.output_ids == expected_outputs(prompt(7, base=2), 12, eos=eos)
    # one more step than it needed ran for the request that met eos
    assert sum(1 for step in fake.log for r in step if r[0] == seq.req_id) == 1 + 4
    assert mgr.pages_free() == 64 and mgr.free_slots() == 8


@pytest.mark.parametrize("policy", ["prefill_first", "mixed"])
@pytest.mark.parametrize("seed", range(6))
def test_pipelined_and_plain_scheduling_give_the_same_tokens(policy, seed):
    """Random workloads with too few pages (preemption), eos and the context limit: the
    pipelined scheduler gives every request the tokens the plain one gives it."""
    import random
    rng = random.Random(seed)
    reqs = []
    for i in range(10):
        n = rng.randint(1, 40)
        reqs.append(dict(prompt_ids=[rng.randrange(VOCAB) for _ in range(n)],
                         max_new_tokens=rng.randint(1, 30), seed=rng.randrange(100),
                         stop_at_eos=rng.random() < 0.7))
    outs = {}
    for pipeline in (False, True):
        sch, fake, mgr = make_pipelined(pipeline, num_pages=24, page_size=4, max_requests=4,
                                        max_batch=4, budget=16, max_ctx=60, eos=11,
                                        policy=policy)
        seqs = []
        pending = list(reqs)
        steps = 0
        while pending or sch.has_work():
            # requests arrive while others run
            for _ in range(rng.randint(0, 2) if pending else 0):
                if pending:
                    seqs.append(sch.add(Request(**pending.pop(0))))
            if sch.has_work():
                sch.step()
                mgr.check()
            steps += 1
            assert steps < 5000
        outs[pipeline] = [(s.output_ids, s.finish_reason) for s in seqs]
        assert mgr.pages_free() == 24 and mgr.free_slots() == 4
        for s, r in zip(seqs, reqs):
            full = expected_outputs(r["prompt_ids"], r["max_new_tokens"], r["seed"],
                                    eos=11 if r["stop_at_eos"] else None, max_ctx=60)
            if s.finish_reason != "out_of_pages":
                assert s.output_ids == full
            else:
                assert s.output_ids == full[:len(s.output_ids)]
        assert sch.stats.preemptions > 0          # the pool is small on purpose


def test_abort_while_a_token_is_in_flight():
    sch, fake, mgr = make_pipelined(True)
    a = sch.add(Request(prompt(6), max_new_tokens=20))
    b = sch.add(Request(prompt(5, base=9), max_new_tokens=5))
    for _ in range(4):
        sch.step()
    assert a.pending
    assert sch.abort(a.req_id)
    run(sch, mgr)
    assert a.finish_reason == "aborted"
    assert b.output_ids == expected_outputs(prompt(5, base=9), 5)
    assert mgr.pages_free() == 64 and mgr.free_slots() == 8


@pytest.mark.parametrize("policy", ["prefill_first", "mixed"])
def test_requests_admitted_together_still_share_a_prefix(policy):
    """Three requests with the same first 12 tokens are submitted at once: nothing is published
    when they are admitted, so admission finds no match; the first one's prompt pages are
    published when its prefill ends, and the others pick them up before they run anything."""
    sch, fake, mgr = make(page_size=4, budget=24, policy=policy)
    shared = prompt(12, base=5)
    reqs = [shared + prompt(9, base=40 + 7 * i) for i in range(3)]
    seqs = [sch.add(Request(p, max_new_tokens=3)) for p in reqs]
    run(sch, mgr)
    assert seqs[0].cached_prefix_tokens == 0
    if policy == "prefill_first":           # one prompt a step: the later ones see the first's pages
        assert [s.cached_prefix_tokens for s in seqs[1:]] == [12, 12]
        assert [s.prefill_tokens_computed for s in seqs] == [21, 9, 9]
    for s, p in zip(seqs, reqs):
        assert s.output_ids == expected_outputs(p, 3)
    assert sch.stats.tokens_saved_by_cache == sum(s.cached_prefix_tokens for s in seqs)
    mgr.check()
