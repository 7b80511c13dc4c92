"""The cache manager on the host: no page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from mini_engine_b200.cache import CacheHolder, CacheManager, GroupSpec, PagePoolError, StateSlotPool, compute_hash

FULL = GroupSpec(None, 2, 16, (0, 1))
WIN = GroupSpec(24, 2, 16, (2,))


class Req(CacheHolder):
    def __init__(self, tokens):
        super().__init__()
        self.tokens = tokens


def test_allocate_is_all_or_nothing():
    m = CacheManager([FULL], 4, 16)
    a, b = Req([1] * 40), Req([2] * 40)
    assert m.allocate(a, 40) and m.num_free_pages == [1]
    assert not m.allocate(b, 40)                       # needs 3, has 1: nothing changes
    assert m.num_free_pages == [1] and b.block_tables == [[]]
    m.free(a)
    assert m.num_free_pages == [4] and m.allocate(b, 40)
    m.check([b])


def test_decode_takes_a_page_only_at_a_page_boundary():
    m = CacheManager([FULL], 4, 16)
    a = Req([])
    assert m.allocate(a, 16)
    a.num_computed_tokens = 16
    assert len(a.block_tables[0]) == 1
    assert m.allocate(a, 1) and len(a.block_tables[0]) == 2
    a.num_computed_tokens = 17
    assert m.allocate(a, 1) and len(a.block_tables[0]) == 2


def test_double_free_is_caught():
    m = CacheManager([FULL], 2, 16)
    a = Req([])
    m.allocate(a, 5)
    page = a.block_tables[0][0]
    m.free(a)
    with pytest.raises(PagePoolError):
        m.pools[0].release(page)


def test_pages_are_used_again_in_release_order():
    m = CacheManager([FULL], 3, 16)
    a = Req([])
    m.allocate(a, 48)
    assert a.block_tables[0] == [0, 1, 2]
    m.free(a)                                           # last page first onto the back of the free list
    b = Req([])
    m.allocate(b, 48)
    assert b.block_tables[0] == [2, 1, 0]


def test_prefix_hits_share_pages_and_never_cover_the_last_token():
    m = CacheManager([FULL], 8, 4)
    toks = list(range(100, 112))                        # 12 tokens = 3 full pages
    a = Req(toks)
    assert m.find_prefix_hit(toks) == [[]]
    m.allocate(a, 12)
    a.num_computed_tokens = 12
    m.hash_full_pages(a, toks)
    assert a.num_hashed_blocks == 3
    hits = m.find_prefix_hit(toks)                      # same 12 tokens: at most (12-1)//4 = 2 pages
    assert hits == [a.block_tables[0][:2]]
    b = Req(toks)
    assert m.allocate(b, 12 - 8, hits)
    assert b.num_computed_tokens == 8 and b.num_cached_tokens == 8
    assert b.block_tables[0][:2] == a.block_tables[0][:2] and b.block_tables[0][2] != a.block_tables[0][2]
    assert m.pools[0].ref_count[a.block_tables[0][0]] == 2
    m.check([a, b])
    m.free(a)
    m.check([b])
    m.free(b)
    # freed pages keep their hashes until they are taken for new content
    assert m.find_prefix_hit(toks + [1]) == [hits[0] + [m.pools[0].hash_to_page[compute_hash(toks[8:12], compute_hash(toks[4:8], compute_hash(toks[:4])))]]]
    c = Req(toks)
    assert m.allocate(c, 4, m.find_prefix_hit(toks))
    m.check([c])
    other = Req([])
    assert m.allocate(other, 20)                         # takes all free pages: their old hashes are dropped
    assert m.num_free_pages == [0]
    assert m.find_prefix_hit(toks + [1]) == [c.block_tables[0][:2]]   # the third page's content is gone
    m.check([c, other])


def test_hash_chain_depends_on_the_prefix():
    assert compute_hash([1, 2, 3]) != compute_hash([1, 2, 3], prefix=5)
    assert compute_hash([1, 2, 3], 5) == compute_hash([1, 2, 3], 5)


def test_collision_is_checked_against_tokens():
    m = CacheManager([FULL], 4, 2)
    a = Req([5, 6, 7])
    m.allocate(a, 3)
    a.num_computed_tokens = 3
    m.hash_full_pages(a, a.tokens)
    page = a.block_tables[0][0]
    m.pools[0].page_tokens[page] = [9, 9]                # pretend another content has this hash
    assert m.find_prefix_hit([5, 6, 7]) == [[]]


def test_window_group_gives_pages_back_and_full_group_keeps_them():
    m = CacheManager([FULL, WIN], 8, 16)
    assert not m.prefix_caching                          # a page given back cannot be found again
    a = Req([])
    pos = 0
    for n in (40, 1, 1, 30, 1):
        assert m.allocate(a, n)
        pos += n
        a.num_computed_tokens = pos
        m.release_behind_window(a)
        m.check([a])
        first_needed = pos - 24 + 1
        for i, p in enumerate(a.block_tables[1]):
            assert (p == -1) == ((i + 1) * 16 <= first_needed)
        assert all(p >= 0 for p in a.block_tables[0])
    assert a.block_tables[1][:3] == [-1, -1, -1] and m.num_free_pages == [3, 6]
    m.free(a)
    assert m.num_free_pages == [8, 8]
    m.check([])


def test_state_slots():
    m = CacheManager([FULL], 8, 16, num_state_slots=2, has_state=True)
    assert not m.prefix_caching
    a, b, c = Req([]), Req([]), Req([])
    assert m.allocate(a, 1) and m.allocate(b, 1)
    assert {a.state_slot, b.state_slot} == {0, 1}
    assert not m.allocate(c, 1) and c.state_slot == -1 and m.num_free_pages == [6]
    m.free(a)
    assert a.state_slot == -1 and m.allocate(c, 1) and c.state_slot in (0, 1)
    m.check([b, c])
    p = StateSlotPool(1)
    s = p.acquire()
    p.release(s)
    with pytest.raises(RuntimeError):
        p.release(s)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_keep_the_invariants(seed):
    rng = random.Random(seed)
    groups = [FULL] if seed % 2 == 0 else [FULL, WIN]
    m = CacheManager(groups, rng.randint(6, 20), rng.choice([4, 8, 16]), num_state_slots=5 if seed % 3 == 0 else 0,
                     has_state=seed % 3 == 0)
    shared = [rng.randrange(50) for _ in range(64)]
    live: list[Req] = []
    for _ in range(400):
        op = rng.random()
        if op < 0.35 and len(live) < 6:
            n = rng.randint(1, 70)
            toks = (shared[:rng.randint(0, 64)] + [rng.randrange(50) for _ in range(n)])[:n]
            r = Req(toks)
            hits = m.find_prefix_hit(toks)
            portion = rng.randint(1, len(toks) - len(hits[0]) * m.page_size)
            if m.allocate(r, portion, hits):
                r.num_computed_tokens += portion
                m.hash_full_pages(r, r.tokens)
                m.release_behind_window(r)
                live.append(r)
            else:
                assert r.block_tables == [[] for _ in groups] or all(not t for t in r.block_tables)
                assert r.state_slot == -1
        elif op < 0.8 and live:
            r = rng.choice(live)
            owed = len(r.tokens) - r.num_computed_tokens
            n = rng.randint(1, owed) if owed > 0 else 1
            if owed <= 0:
                r.tokens.append(rng.randrange(50))
            before = [list(t) for t in r.block_tables]
            if m.allocate(r, n):
                r.num_computed_tokens += n
                m.hash_full_pages(r, r.tokens)
                m.release_behind_window(r)
            else:
                assert r.block_tables == before
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.free(r)
            assert all(not t for t in r.block_tables)
        m.check(live)
        for g, pool in enumerate(m.pools):
            held = sum(1 for r in live for p in r.block_tables[g] if p >= 0)
            assert held >= len(pool.used)                # shared pages are counted once in `used`
            for r in live:                               # every token still visible has a page
                lo = 0 if groups[g].window is None else max(0, r.num_computed_tokens - groups[g].window + 1)
                for pos in range(lo, r.num_computed_tokens):
                    assert r.block_tables[g][pos // m.page_size] >= 0
    for r in live:
        m.free(r)
    m.check([])
    assert m.num_free_pages == [p.num_pages for p in m.pools]
