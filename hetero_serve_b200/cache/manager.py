"""The cache manager: pages for keys and values, a block table per request, prefix
reuse, and slots for per-request state of fixed size.  Pure host code: it hands out
page numbers; the tensors live in :mod:`hetero_serve_b200.cache.storage`.

Pages are grouped.  Layers whose mixers have the same needs (head count, head size,
"all keys" or "a window of them") share a *page group*: one pool of pages, one block
table per request.  GPT-2 has a single group that keeps every key; a model with
windowed layers would add a group whose pages are given back as soon as the window
has passed them.  Every group has pages of its own.

The page life cycle follows the reference's ``BlockAllocator`` (heteroserve/kv/blocks.py):

* free pages are handed out lowest number first (blocks.py:83,116-118);
* full pages of a prompt are *published* under a chain hash — blake2b over the previous
  hash and the page's token ids (blocks.py:29-46) — so that a later request with the same
  prefix reuses them (``match``, blocks.py:153-166) with a reference count (blocks.py:128-145);
* a published page whose count drops to zero stays findable until the pool runs dry, and
  is then evicted oldest first (blocks.py:116-126, 135-145).

Differences, decided here: reservation is all-or-nothing (the reference's ``grow`` keeps the
pages it got before failing, blocks.py:203-209); a prefix match never covers the last token
of a prompt — at most ``(len - 1) // page_size`` pages are reused — so a shared page is never
written again (the reference caps the count at ``len - 1`` but then rewrites the last token
into the shared block, heteroserve/worker/worker.py:401-402).
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Hashable, Iterable, Sequence


class OutOfPages(RuntimeError):
    """The pool cannot supply the pages asked for; nothing was taken."""


class CacheError(RuntimeError):
    """The manager was used inconsistently (unknown request, double close, ...)."""


def hash_page(prev_hash: int | None, token_ids: Sequence[int]) -> int:
    """64-bit chain hash of one full page: blake2b-8 over the previous hash (8 zero bytes
    for the first page) and the token ids as little-endian int32
    (heteroserve/kv/blocks.py:29-34)."""
    h = hashlib.blake2b(digest_size=8)
    h.update(b"\x00" * 8 if prev_hash is None else prev_hash.to_bytes(8, "little"))
    h.update(struct.pack(f"<{len(token_ids)}i", *token_ids))
    return int.from_bytes(h.digest(), "little")


def chain_hashes(token_ids: Sequence[int], page_size: int) -> list[int]:
    """Chain hash of every *full* page of a token sequence (heteroserve/kv/blocks.py:37-46)."""
    out: list[int] = []
    prev: int | None = None
    for i in range(len(token_ids) // page_size):
        prev = hash_page(prev, token_ids[i * page_size:(i + 1) * page_size])
        out.append(prev)
    return out


@dataclass(frozen=True)
class GroupSpec:
    """One page group: ``window == 0`` keeps every position, ``window == w`` the last w."""

    window: int = 0
    num_pages: int | None = None      # None → the manager's default


class PagePool:
    """Pages of one group: free list, reference counts, published pages, LRU."""

    def __init__(self, num_pages: int, allow_publish: bool):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self.allow_publish = allow_publish
        self._free = list(range(num_pages - 1, -1, -1))     # pop() → lowest number
        self._ref = [0] * num_pages
        self._hash_to_page: dict[int, int] = {}
        self._page_to_hash: dict[int, int] = {}
        self._evictable: OrderedDict[int, None] = OrderedDict()   # hash → None, oldest first
        self.evictions = 0

    # capacity ------------------------------------------------------------
    @property
    def num_free(self) -> int:
        """Pages obtainable right now: unused ones and published ones nobody holds."""
        return len(self._free) + len(self._evictable)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    # life cycle ----------------------------------------------------------
    def take(self, n: int) -> list[int]:
        """``n`` fresh pages with count 1, or :class:`OutOfPages` and nothing taken."""
        if n > self.num_free:
            raise OutOfPages(f"{n} pages wanted, {self.num_free} obtainable "
                             f"of {self.num_pages}")
        out = []
        for _ in range(n):
            if self._free:
                page = self._free.pop()
            else:
                h, _ = self._evictable.popitem(last=False)
                page = self._hash_to_page.pop(h)
                del self._page_to_hash[page]
                self.evictions += 1
            self._ref[page] = 1
            out.append(page)
        return out

    def hold(self, page: int) -> None:
        """One more holder of a published page."""
        if self._ref[page] == 0:
            h = self._page_to_hash.get(page)
            if h is None or h not in self._evictable:
                raise CacheError(f"page {page} is free: it cannot be held")
            del self._evictable[h]
        self._ref[page] += 1

    def drop(self, page: int) -> None:
        if self._ref[page] <= 0:
            raise CacheError(f"page {page} is given back twice")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            h = self._page_to_hash.get(page)
            if h is not None and self._hash_to_page.get(h) == page:
                self._evictable[h] = None          # most recently released at the end
            else:
                self._free.append(page)

    # prefix reuse --------------------------------------------------------
    def match(self, hashes: Iterable[int]) -> list[int]:
        """Pages of the longest published prefix; stops at the first miss."""
        out = []
        for h in hashes:
            page = self._hash_to_page.get(h)
            if page is None:
                break
            out.append(page)
        return out

    def publish(self, h: int, page: int) -> bool:
        """Make a full page findable.  Equal content published earlier wins."""
        if not self.allow_publish or h in self._hash_to_page or page in self._page_to_hash:
            return False
        if self._ref[page] <= 0:
            raise CacheError(f"page {page} is not held: it cannot be published")
        self._hash_to_page[h] = page
        self._page_to_hash[page] = h
        return True

    def refcount(self, page: int) -> int:
        return self._ref[page]

    def check(self, held: dict[int, int]) -> None:
        """Invariant: every page is exactly one of free / evictable / held, and the count of
        a held page equals the number of tables that list it (``held``: page → holders)."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is twice in the free list")
        evictable = {self._hash_to_page[h] for h in self._evictable}
        if len(evictable) != len(self._evictable):
            raise AssertionError("two evictable hashes name one page")
        in_use = {p for p in range(self.num_pages) if self._ref[p] > 0}
        if free & evictable or free & in_use or evictable & in_use:
            raise AssertionError("a page is in two states at once")
        if len(free) + len(evictable) + len(in_use) != self.num_pages:
            lost = set(range(self.num_pages)) - free - evictable - in_use
            raise AssertionError(f"pages lost: {sorted(lost)}")
        for p in in_use:
            if held.get(p, 0) != self._ref[p]:
                raise AssertionError(f"page {p}: count {self._ref[p]}, holders {held.get(p, 0)}")
        for p in held:
            if p not in in_use:
                raise AssertionError(f"page {p} is in a table but not held")
        for h, p in self._hash_to_page.items():
            if self._page_to_hash.get(p) != h:
                raise AssertionError("hash maps disagree")


@dataclass
class _Request:
    slot: int
    length: int = 0                              # positions whose keys/values are resident
    tables: list[list[int]] = field(default_factory=list)     # per group; -1 = given back
    first_live: list[int] = field(default_factory=list)       # per group: first page kept
    cached_tokens: int = 0
    published: int = 0                           # full pages already published


@dataclass(frozen=True)
class Opened:
    slot: int
    cached_tokens: int


class CacheManager:
    """Pages and state slots of every live request."""

    def __init__(self, groups: Sequence[GroupSpec], num_pages: int, page_size: int,
                 max_requests: int, prefix_cache: bool = True, has_state: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if not groups:
            groups = ()
        self.page_size = page_size
        self.groups = tuple(groups)
        # a shared prefix is only sound when every group still holds it and no mixer keeps
        # state beside the pages
        self.prefix_cache = (prefix_cache and not has_state and len(self.groups) > 0
                             and all(g.window == 0 for g in self.groups))
        self.pools = [PagePool(g.num_pages or num_pages, self.prefix_cache) for g in self.groups]
        self.max_requests = max_requests
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._requests: dict[Hashable, _Request] = {}
        self.hit_tokens = 0
        self.miss_tokens = 0
        # called with the state slot of every request that is opened, whoever opens it (the
        # step function, the scheduler): the owner of the state tensors clears the slot here,
        # so that a request never starts on what the slot's previous owner left
        self.on_open: Callable[[int], None] | None = None

    # -- queries ------------------------------------------------------------
    def __contains__(self, req_id) -> bool:
        return req_id in self._requests

    def _get(self, req_id) -> _Request:
        try:
            return self._requests[req_id]
        except KeyError:
            raise CacheError(f"request {req_id!r} is not open") from None

    def live(self) -> list:
        return list(self._requests)

    def length(self, req_id) -> int:
        return self._get(req_id).length

    def slot(self, req_id) -> int:
        return self._get(req_id).slot

    def table(self, req_id, group: int = 0) -> list[int]:
        return self._get(req_id).tables[group]

    def free_slots(self) -> int:
        return len(self._free_slots)

    def pages_free(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def max_pages_per_request(self, max_positions: int) -> int:
        return self.pages_for(max_positions)

    # -- life of a request -----------------------------------------------------
    def open(self, req_id, token_ids: Sequence[int] | None = None) -> Opened:
        """Start a request: a state slot, and (if prefix reuse is on and ``token_ids`` is
        given) the pages of the longest published prefix, at most ``(len-1)//page_size``."""
        if req_id in self._requests:
            raise CacheError(f"request {req_id!r} is already open")
        if not self._free_slots:
            raise OutOfPages("no state slot free")
        req = _Request(slot=self._free_slots.pop(),
                       tables=[[] for _ in self.groups], first_live=[0] * len(self.groups))
        if self.prefix_cache and token_ids is not None and len(token_ids) > 1:
            usable = (len(token_ids) - 1) // self.page_size
            hashes = chain_hashes(token_ids[:usable * self.page_size], self.page_size)
            matches = [pool.match(hashes) for pool in self.pools]
            n = min(len(m) for m in matches)
            for gi, pool in enumerate(self.pools):
                for page in matches[gi][:n]:
                    pool.hold(page)
                req.tables[gi] = list(matches[gi][:n])
            req.cached_tokens = n * self.page_size
            req.length = req.cached_tokens
            req.published = n
        if token_ids is not None:
            self.hit_tokens += req.cached_tokens
            self.miss_tokens += len(token_ids) - req.cached_tokens
        self._requests[req_id] = req
        if self.on_open is not None:
            self.on_open(req.slot)
        return Opened(req.slot, req.cached_tokens)

    def rematch(self, req_id, token_ids: Sequence[int]) -> int:
        """Try the prefix match again for a request that has computed nothing since it was
        opened: pages published meanwhile (by requests admitted with it that were prefilled
        first) replace the fresh pages reserved for the same positions.  Returns the number of
        leading tokens now served from the cache."""
        req = self._get(req_id)
        if not self.prefix_cache or req.length != req.cached_tokens or len(token_ids) < 2:
            return req.cached_tokens
        usable = (len(token_ids) - 1) // self.page_size
        have = req.cached_tokens // self.page_size
        if usable <= have:
            return req.cached_tokens
        hashes = chain_hashes(token_ids[:usable * self.page_size], self.page_size)
        n = min(len(pool.match(hashes)) for pool in self.pools)
        if n <= have:
            return req.cached_tokens
        for gi, pool in enumerate(self.pools):
            found = pool.match(hashes)
            table = req.tables[gi]
            for i in range(have, n):
                pool.hold(found[i])
                if i < len(table):
                    pool.drop(table[i])          # the fresh page reserved for this position
                    table[i] = found[i]
                else:
                    table.append(found[i])
        gained = (n - have) * self.page_size
        req.cached_tokens = req.length = n * self.page_size
        req.published = max(req.published, n)
        self.hit_tokens += gained
        self.miss_tokens -= gained
        return req.cached_tokens

    def pages_needed(self, req_id, new_len: int) -> list[int]:
        """Fresh pages each group must supply so that positions < new_len have a page."""
        req = self._get(req_id)
        want = self.pages_for(new_len)
        return [max(0, want - len(t)) for t in req.tables]

    def can_reserve(self, req_id, new_len: int) -> bool:
        need = self.pages_needed(req_id, new_len)
        return all(n <= pool.num_free for n, pool in zip(need, self.pools))

    def reserve(self, req_id, new_len: int) -> None:
        """Give the request pages for positions < new_len in every group, or raise
        :class:`OutOfPages` having taken none."""
        req = self._get(req_id)
        need = self.pages_needed(req_id, new_len)
        for n, pool in zip(need, self.pools):
            if n > pool.num_free:
                raise OutOfPages(f"{n} pages wanted, {pool.num_free} obtainable")
        for gi, (n, pool) in enumerate(zip(need, self.pools)):
            if n:
                req.tables[gi].extend(pool.take(n))

    def table_lengths(self, req_id) -> list[int]:
        return [len(t) for t in self._get(req_id).tables]

    def unreserve(self, req_id, lengths: Sequence[int]) -> None:
        """Give back the pages reserved beyond ``lengths`` (what :meth:`table_lengths` said
        before the reservation): undoes a :meth:`reserve` whose step did not run."""
        req = self._get(req_id)
        for gi, (n, pool) in enumerate(zip(lengths, self.pools)):
            if self.pages_for(req.length) > n:
                raise CacheError("unreserve below the resident positions")
            table = req.tables[gi]
            while len(table) > n:
                page = table.pop()
                if page >= 0:
                    pool.drop(page)

    def commit(self, req_id, new_len: int) -> None:
        """Positions < new_len are now resident.  Pages of a windowed group that no later
        query can reach are given back at once."""
        req = self._get(req_id)
        if new_len < req.length:
            raise CacheError("a request's length cannot shrink")
        if any(self.pages_for(new_len) > len(t) for t in req.tables):
            raise CacheError("commit beyond the reserved pages")
        req.length = new_len
        for gi, g in enumerate(self.groups):
            if g.window <= 0:
                continue
            # the next query sits at position >= new_len and reads keys > new_len - window
            first_needed = max(0, new_len - g.window + 1)
            keep_from = first_needed // self.page_size
            table = req.tables[gi]
            for i in range(req.first_live[gi], min(keep_from, len(table))):
                if table[i] >= 0:
                    self.pools[gi].drop(table[i])
                    table[i] = -1
            req.first_live[gi] = max(req.first_live[gi], min(keep_from, len(table)))

    def publish(self, req_id, token_ids: Sequence[int]) -> int:
        """Make the full pages of ``token_ids[:length]`` findable by later requests
        (heteroserve/kv/blocks.py:211-230).  Returns how many were newly published."""
        if not self.prefix_cache:
            return 0
        req = self._get(req_id)
        n_tok = min(len(token_ids), req.length)
        hashes = chain_hashes(token_ids[:n_tok], self.page_size)
        new = 0
        for i in range(req.published, len(hashes)):
            for gi, pool in enumerate(self.pools):
                if pool.publish(hashes[i], req.tables[gi][i]):
                    new += 1
        req.published = max(req.published, len(hashes))
        return new

    def close(self, req_id) -> None:
        """End a request: every page and the state slot are given back."""
        req = self._requests.pop(req_id, None)
        if req is None:
            raise CacheError(f"request {req_id!r} is not open (closed twice?)")
        for gi, pool in enumerate(self.pools):
            for page in req.tables[gi]:
                if page >= 0:
                    pool.drop(page)
        self._free_slots.append(req.slot)

    # -- checks and counters --------------------------------------------------------
    def check(self) -> None:
        """Raise AssertionError if a page or a slot is lost, held twice or freed twice."""
        for gi, pool in enumerate(self.pools):
            held: dict[int, int] = {}
            for req in self._requests.values():
                for page in req.tables[gi]:
                    if page >= 0:
                        held[page] = held.get(page, 0) + 1
            pool.check(held)
        slots = [r.slot for r in self._requests.values()] + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise AssertionError(f"state slots lost or doubled: {sorted(slots)}")

    def snapshot(self) -> dict:
        """Counters in the manner of the reference's ``snapshot`` (heteroserve/kv/blocks.py:339-351)."""
        out = {"page_size": self.page_size, "live_requests": len(self._requests),
               "hits": self.hit_tokens, "misses": self.miss_tokens, "groups": []}
        for g, pool in zip(self.groups, self.pools):
            out["groups"].append({
                "window": g.window, "num_blocks": pool.num_pages, "used": pool.num_used,
                "free": pool.num_free, "cached_blocks": len(pool._hash_to_page),
                "evictable": len(pool._evictable), "evictions": pool.evictions,
                "utilisation": round(pool.num_used / pool.num_pages, 4)})
        return out
