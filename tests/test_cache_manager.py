"""The cache manager (no GPU): pages are never lost, held twice or freed twice, under
random orders of requests; prefix reuse; LRU eviction; windowed groups; state slots."""

import random

import pytest

from hetero_serve_b200.cache import (CacheError, CacheManager, GroupSpec, OutOfPages,
                                     chain_hashes, hash_page)


def test_chain_hash_matches_the_reference_vector():
    # produced by heteroserve/kv/blocks.py chain_hashes(list(range(32)), 16)
    assert chain_hashes(list(range(32)), 16) == [10251598853290956434, 14413796365232270483]
    assert chain_hashes(list(range(31)), 16) == [10251598853290956434]     # full pages only
    a = chain_hashes([1] * 16 + [2] * 16, 16)
    b = chain_hashes([3] * 16 + [2] * 16, 16)
    assert a[1] != b[1]                       # same second page, different prefix
    assert hash_page(None, [5, 6]) != hash_page(1, [5, 6])


def test_reserve_commit_close_roundtrip():
    m = CacheManager([GroupSpec()], num_pages=8, page_size=16, max_requests=2)
    m.open("a")
    m.reserve("a", 33)
    assert m.table("a") == [0, 1, 2] and m.pages_free() == 5      # lowest numbers first
    m.commit("a", 33)
    assert m.length("a") == 33
    m.reserve("a", 48)                                          # already covered
    assert len(m.table("a")) == 3
    m.close("a")
    assert m.pages_free() == 8
    m.check()
    with pytest.raises(CacheError, match="not open"):
        m.close("a")                                            # freed twice


def test_reserve_is_all_or_nothing():
    m = CacheManager([GroupSpec()], num_pages=4, page_size=16, max_requests=3)
    m.open("a"); m.reserve("a", 48)
    m.open("b"); m.reserve("b", 16)
    with pytest.raises(OutOfPages):
        m.reserve("b", 64)                     # needs 3 more, 0 free
    assert len(m.table("b")) == 1 and m.pages_free() == 0
    assert not m.can_reserve("b", 17) and m.can_reserve("b", 16)
    m.check()


def test_prefix_sharing_refcounts_and_no_write_into_shared_pages():
    m = CacheManager([GroupSpec()], num_pages=8, page_size=16, max_requests=4)
    prompt = list(range(40))
    assert m.open("a", prompt).cached_tokens == 0
    m.reserve("a", 40); m.commit("a", 40); m.publish("a", prompt)
    o = m.open("b", prompt)                    # same prompt: 2 full pages are shared
    assert o.cached_tokens == 32 and m.table("b") == m.table("a")[:2]
    assert m.pools[0].refcount(m.table("a")[0]) == 2
    m.reserve("b", 40)
    assert m.table("b")[2] != m.table("a")[2]  # the partial page is private
    # a prompt that IS the published pages still recomputes its last page: the last token's
    # key/value is never written into a page someone else holds
    o = m.open("c", prompt[:32])
    assert o.cached_tokens == 16
    m.check()
    for r in "abc":
        m.close(r)
    m.check()
    assert m.pages_free() == 8 and m.snapshot()["groups"][0]["evictable"] == 2


def test_lru_eviction_oldest_released_first():
    m = CacheManager([GroupSpec()], num_pages=3, page_size=4, max_requests=4)
    for name, base in (("a", 0), ("b", 100), ("c", 200)):
        toks = list(range(base, base + 4))
        m.open(name, toks); m.reserve(name, 4); m.commit(name, 4); m.publish(name, toks)
    m.close("b"); m.close("a"); m.close("c")           # release order: b, a, c
    assert m.pages_free() == 3
    m.open("d"); m.reserve("d", 4)                     # evicts b's page (oldest release)
    assert m.pools[0].evictions == 1
    assert m.open("e", list(range(100, 108))).cached_tokens == 0     # b is gone
    assert m.open("f", list(range(0, 8))).cached_tokens == 4         # a is still cached
    m.check()


def test_published_page_is_not_evicted_while_held():
    m = CacheManager([GroupSpec()], num_pages=2, page_size=4, max_requests=4)
    toks = list(range(8))
    m.open("a", toks); m.reserve("a", 8); m.commit("a", 8); m.publish("a", toks)
    m.open("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 4)
    m.close("a")
    m.reserve("b", 8)                                   # both evicted now
    assert m.pools[0].evictions == 2
    m.check()


def test_windowed_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([GroupSpec(window=0), GroupSpec(window=20)], num_pages=16, page_size=16,
                     max_requests=2)
    assert not m.prefix_cache                           # a window rules prefix reuse out
    m.open("a")
    m.reserve("a", 100); m.commit("a", 100)
    full, win = m.table("a", 0), m.table("a", 1)
    assert all(p >= 0 for p in full) and len(full) == 7
    # next query at position >= 100 reads keys >= 81: pages 0..4 (positions < 80) are back
    assert win[:5] == [-1] * 5 and all(p >= 0 for p in win[5:])
    assert m.pages_free(1) == 16 - 2 and m.pages_free(0) == 16 - 7
    m.reserve("a", 130); m.commit("a", 130)
    assert m.table("a", 1)[:6] == [-1] * 6
    m.check()
    m.close("a")
    assert m.pages_free(0) == 16 and m.pages_free(1) == 16
    m.check()


def test_state_slots():
    m = CacheManager([GroupSpec()], num_pages=4, page_size=16, max_requests=2)
    a, b = m.open("a").slot, m.open("b").slot
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages, match="slot"):
        m.open("c")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    m.close("a")
    assert m.open("c").slot == a
    m.check()


def test_state_rules_out_prefix_reuse():
    m = CacheManager([GroupSpec()], 4, 16, 2, prefix_cache=True, has_state=True)
    assert not m.prefix_cache
    toks = list(range(32))
    m.open("a", toks); m.reserve("a", 32); m.commit("a", 32)
    assert m.publish("a", toks) == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    windows = [0] if seed % 2 == 0 else [0, 24]
    m = CacheManager([GroupSpec(window=w) for w in windows], num_pages=24, page_size=8,
                     max_requests=5, prefix_cache=True)
    prompts = [[rng.randrange(4) for _ in range(rng.randrange(1, 60))] for _ in range(6)]
    live: dict[str, list[int]] = {}
    n = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{n}"; n += 1
            toks = list(rng.choice(prompts)) + [rng.randrange(4) for _ in range(rng.randrange(4))]
            o = m.open(rid, toks)
            assert o.cached_tokens % 8 == 0 and o.cached_tokens < len(toks)
            live[rid] = toks
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            cur = m.length(rid)
            new = min(cur + rng.choice([1, 1, 1, 2, 7, 19]), 120)
            while len(live[rid]) < new:
                live[rid].append(rng.randrange(4))
            try:
                m.reserve(rid, new)
            except OutOfPages:
                before = [list(m.table(rid, g)) for g in range(len(windows))]
                assert before == [list(m.table(rid, g)) for g in range(len(windows))]
                victim = rng.choice(list(live))
                m.close(victim); del live[victim]
                m.check()
                continue
            m.commit(rid, new)
            if rng.random() < 0.5:
                m.publish(rid, live[rid])
        elif live:
            rid = rng.choice(list(live))
            if rng.random() < 0.5:
                m.publish(rid, live[rid])
            m.close(rid); del live[rid]
        m.check()
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(m.pages_free(g) == 24 for g in range(len(windows)))
    assert m.free_slots() == 5


def test_rematch_picks_up_pages_published_after_admission():
    """Two requests with the same first 32 tokens are admitted together (nothing published yet,
    so neither matches); the first is prefilled and publishes; the second, before it runs
    anything, matches again and trades its fresh pages for the published ones."""
    from hetero_serve_b200.cache import CacheManager, GroupSpec
    m = CacheManager([GroupSpec()], num_pages=12, page_size=16, max_requests=4, prefix_cache=True)
    a = list(range(40))
    b = list(range(32)) + [99] * 20
    for rid, toks in (("a", a), ("b", b)):
        assert m.open(rid, toks).cached_tokens == 0
        m.reserve(rid, len(toks))
    free = m.pages_free()
    m.commit("a", len(a))
    m.publish("a", a)
    old_table = list(m.table("b"))
    assert m.rematch("b", b) == 32
    assert m.table("b")[:2] == m.table("a")[:2] and m.table("b")[2:] == old_table[2:]
    assert m.length("b") == 32 and m.pages_free() == free + 2      # two fresh pages came back
    assert m.rematch("b", b) == 32                                  # nothing more to gain
    m.check()
    m.commit("b", len(b))
    assert m.rematch("b", b) == 32                                  # it has run: no rematch
    m.close("a"); m.close("b")
    m.check()
