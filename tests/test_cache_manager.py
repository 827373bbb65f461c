"""The cache manager alone, on the CPU: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; slots."""
import random

import pytest

from torchlet_b200.cache import CacheError, CacheManager, GroupSpec, PagePool


def make(num_pages=12, page=4, slots=3, window=None, max_seq=64, two_groups=False):
    groups = [GroupSpec(2, 16, None, (0, 1), num_pages)]
    if two_groups or window:
        groups.append(GroupSpec(2, 16, window, (2,), num_pages))
    return CacheManager(groups, page, slots, max_seq)


def test_pool_refuses_double_free_and_overdraw():
    pool = PagePool(4)
    pages = pool.take(3)
    assert sorted(pages) == [1, 2, 3] and pool.num_free == 0
    with pytest.raises(CacheError):
        pool.take(1)
    pool.give_back([pages[0]])
    with pytest.raises(CacheError):
        pool.give_back([pages[0]])
    with pytest.raises(CacheError):
        pool.give_back([7])
    pool.give_back([0])  # the null page is never held; giving it back is a no-op
    assert pool.num_free == 1


def test_extend_is_all_or_nothing_and_pages_are_used_again():
    m = make(num_pages=5, page=4)  # 4 usable pages
    m.admit("a"); m.admit("b")
    assert m.extend("a", 9)  # 3 pages
    assert not m.can_extend("b", 8) and not m.extend("b", 8)
    assert m.table("b", 0) == [] and m.pools[0].num_free == 1
    assert m.extend("b", 4)
    a_pages = list(m.table("a", 0))
    m.advance("a", 9)
    m.finish("a")
    m.check()
    m.admit("c")
    assert m.extend("c", 12)
    assert set(m.table("c", 0)) == set(a_pages)
    m.check()
    with pytest.raises(CacheError):
        m.advance("b", 5)  # no page for token 5


def test_window_group_gives_pages_back_when_passed():
    m = make(num_pages=20, page=4, window=6)
    m.admit("a")
    assert m.extend("a", 10)
    assert m.advance("a", 10) == 1  # next query at 10 sees keys >= 5: page 0 (0..3) is passed
    assert m.table("a", 1)[0] == 0 and m.table("a", 1)[1] != 0
    assert m.table("a", 0)[0] != 0  # the group without window keeps everything
    m.extend("a", 11); assert m.advance("a", 11) == 0  # keys >= 6: page 1 (4..7) still needed
    m.extend("a", 14); assert m.advance("a", 14) == 1  # keys >= 9: page 1 passed
    m.check()
    held_window = [p for p in m.table("a", 1) if p]
    assert len(held_window) == 2
    m.finish("a"); m.check()
    assert m.pools[1].num_free == 19


def test_slots():
    m = make(slots=2)
    s0, s1 = m.admit("a"), m.admit("b")
    assert {s0, s1} == {0, 1} and m.num_free_slots == 0
    with pytest.raises(CacheError):
        m.admit("c")
    with pytest.raises(CacheError):
        m.admit("a")
    assert m.finish("a") == s0
    assert m.admit("c") == s0
    m.check()


def test_length_limit():
    m = make(max_seq=16)
    m.admit("a")
    with pytest.raises(CacheError):
        m.extend("a", 17)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = make(num_pages=rng.choice([6, 9, 17]), page=rng.choice([2, 4, 8]), slots=4,
             window=rng.choice([None, 5, 11]), max_seq=80)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.num_free_slots:
            rid = f"r{counter}"; counter += 1
            m.admit(rid); live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            new_len = min(80, live[rid] + rng.choice([1, 1, 1, 2, 5, 13]))
            if m.extend(rid, new_len):
                m.advance(rid, new_len); live[rid] = new_len
            else:
                before = [list(m.table(rid, g)) for g in range(len(m.groups))]
                assert before == [list(m.table(rid, g)) for g in range(len(m.groups))]
        elif live:
            rid = rng.choice(list(live))
            m.finish(rid); del live[rid]
        m.check()
        for rid, length in live.items():
            assert m.num_tokens(rid) == length
            for g, group in enumerate(m.groups):
                table = m.table(rid, g)
                lo = 0 if group.window is None else max(0, length - group.window + 1)
                for pos in range(lo, length):  # every position the next token can see has a page
                    assert table[pos // m.page_size] != 0
    m.reset(); m.check()
    assert all(pool.num_free == pool.num_pages - 1 for pool in m.pools)


def test_decode_pass_matches_single_calls():
    """begin_decode / end_decode do for a batch what extend / advance do one by one,
    the length limit included."""
    from torchlet_b200.cache.manager import CacheError, CacheManager, GroupSpec

    def fresh():
        manager = CacheManager([GroupSpec(2, 16, None, (0,), 40), GroupSpec(2, 16, 20, (1,), 40)], page_size=8, max_slots=4,
                               max_seq_len=50)
        for rid, length in (("a", 7), ("b", 16), ("c", 30)):
            manager.admit(rid)
            assert manager.extend(rid, length)
            manager.advance(rid, length)
        return manager

    one, batch = fresh(), fresh()
    ids = ["a", "b", "c"]
    for _ in range(20):
        for rid in ids:
            length = one.num_tokens(rid)
            assert one.extend(rid, length + 1)
            one.advance(rid, length + 1)
        before, slots = batch.begin_decode(ids)
        batch.end_decode(ids)
        assert [batch.num_tokens(r) for r in ids] == [one.num_tokens(r) for r in ids]
        assert before.tolist() == [n - 1 for n in (batch.num_tokens(r) for r in ids)]
        assert slots.tolist() == [batch.slot_of(r) for r in ids]
        for g in range(2):
            # the same logical pages are held (which physical ones depends on the order of the calls)
            assert all([p != 0 for p in batch.table(r, g)] == [p != 0 for p in one.table(r, g)] for r in ids)
        batch.check()
    # request "c" is at the limit of 50 tokens now
    assert batch.num_tokens("c") == 50
    try:
        batch.begin_decode(["c"])
    except CacheError:
        pass
    else:
        raise AssertionError("the length limit was not enforced")
    # a pool that runs dry is reported by index
    small = CacheManager([GroupSpec(2, 16, None, (0,), 3)], page_size=8, max_slots=2, max_seq_len=64)
    for rid in ("x", "y"):
        small.admit(rid)
        assert small.extend(rid, 8)
        small.advance(rid, 8)
    assert small.begin_decode(["x", "y"]) == 0  # two pages, both taken


def test_a_model_without_paged_history_needs_no_pages():
    """Every mixer keeps fixed-size state only: no group, no pool; slots and lengths still work."""
    manager = CacheManager([], page_size=16, max_slots=2, max_seq_len=128)
    slot = manager.admit("a")
    assert manager.extend("a", 5) and manager.can_extend("a", 128)
    manager.advance("a", 5)
    assert manager.num_tokens("a") == 5
    before, slots = manager.begin_decode(["a"])
    assert before.tolist() == [5] and slots.tolist() == [slot]
    manager.end_decode(["a"])
    assert manager.num_tokens("a") == 6
    manager.admit("b")
    with pytest.raises(CacheError):
        manager.admit("c")  # slots are what runs out
    with pytest.raises(CacheError):
        manager.extend("a", 129)  # the length limit still holds
    manager.check()
    assert manager.finish("a") == slot
    assert manager.admit("c") == slot  # the slot is used again
    manager.reset()
    manager.check()
    assert manager.num_free_slots == 2


def test_check_finds_what_it_is_there_to_find():
    """``check()`` is what the other tests lean on: every kind of damage, done to the bookkeeping by
    hand, makes it raise and name the damage."""
    def fresh():
        m = CacheManager([GroupSpec(1, 8, None, (0,), 9)], 4, 3, 64)
        m.admit("a"); m.admit("b")
        assert m.extend("a", 9) and m.extend("b", 5)
        m.check()
        return m

    m = fresh()
    m._requests["b"].tables[0][0] = m._requests["a"].tables[0][0]
    with pytest.raises(CacheError, match="held twice|differs"):
        m.check()
    m = fresh()
    m.pools[0]._free.append(m.pools[0]._free[0])
    with pytest.raises(CacheError, match="free twice"):
        m.check()
    m = fresh()
    m.pools[0]._free.append(m._requests["a"].tables[0][1])
    with pytest.raises(CacheError, match="both free and held"):
        m.check()
    m = fresh()
    m.pools[0]._free.pop()
    with pytest.raises(CacheError, match="pages lost"):
        m.check()
    m = fresh()
    m.pools[0]._free[0] = 0
    with pytest.raises(CacheError, match="page 0|lost|twice"):
        m.check()
    m = fresh()
    m.table_arrays[0][m.slot_of("a"), 1] = 7 if m._requests["a"].tables[0][1] != 7 else 6
    with pytest.raises(CacheError, match="table array differs"):
        m.check()
    m = fresh()
    m._requests["b"].slot = m._requests["a"].slot
    with pytest.raises(CacheError, match="slot|differs"):
        m.check()
    m = fresh()
    m._free_slots.pop()
    with pytest.raises(CacheError, match="slot is lost"):
        m.check()
