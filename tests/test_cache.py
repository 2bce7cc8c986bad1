"""Slots and pages: nothing lost, held twice or freed twice; windows give pages back; a refused
step changes nothing. Runs on the CPU (the cache's storage is allocated there)."""
import random

import numpy as np
import pytest
import torch

from xpu_serve_b200.cache import Cache, CacheError, CacheFull, IndexPool
from xpu_serve_b200.parts.base import KVNeed, StateNeed


def make(max_tokens=1024, window=0, max_slots=None, max_seq=None):
    needs = [StateNeed((2, 8)), KVNeed(2, 16, 0), StateNeed((2, 8)), KVNeed(2, 16, window), None, KVNeed(1, 32, 0)]
    shares = [None, None, None, None, None, None]
    return Cache(needs, shares, max_tokens, max_slots=max_slots, max_seq_tokens=max_seq, dtype=torch.float32,
                 device="cpu")


def test_index_pool_accounting():
    p = IndexPool(4, "slot")
    a = p.take(3)
    assert a == [0, 1, 2] and p.free_count == 1
    with pytest.raises(CacheFull):
        p.take(2)
    p.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back([0, 0])
    assert p.is_held(0)                       # the refused call changed nothing
    with pytest.raises(CacheError, match="does not exist"):
        p.give_back([7])
    assert p.take(1) == [1]                   # the lowest free index is used again first
    p.check()


def test_groups_by_need():
    c = make()
    kinds = [type(g).__name__ for g in c.groups]
    assert kinds.count("StateGroup") == 1 and kinds.count("KVGroup") == 2      # window 0: calls 1 and 3 share a group
    c2 = make(window=100)
    assert [type(g).__name__ for g in c2.groups].count("KVGroup") == 3        # the window makes its own group
    assert c2.views[4].storage is None
    assert c.views[1].storage.shape == (16 + 1, 2, 2, 64, 16) and c.views[0].storage.shape[1:] == (2, 8)   # + the spare page
    assert c.views[1].storage.data_ptr() != c.views[3].storage.data_ptr()


def test_steps_reserve_pages_and_lengths_advance():
    c = make()
    s = c.open(2)
    starts = c.begin_step(s, [70, 5])
    assert list(starts) == [0, 0]
    c.end_step(s, [70, 5])
    assert list(c.lens[s]) == [70, 5] and c.tokens_held() == 3 * 64
    assert list(c.begin_step(s, [1, 1])) == [70, 5]
    c.end_step(s, [1, 1])
    t = c.page_table(c.kv_groups[0], s)
    assert t.shape == (2, 2) and t[0, 0] != t[0, 1] and t[1, 1] == -1
    c.check()
    c.close([s[1]])
    assert c.tokens_held() == 2 * 64
    c.close([s[0]])
    assert c.tokens_held() == 0 and c.slots.held_count == 0
    c.check()


def test_refused_step_changes_nothing():
    c = make(max_tokens=256)
    s = c.open(3)
    c.begin_step(s[:2], [100, 60])
    c.end_step(s[:2], [100, 60])
    before = (c.lens.copy(), [g.pages.free_count for g in c.groups if hasattr(g, "pages")])
    with pytest.raises(CacheFull):
        c.begin_step(s, [1, 1, 129])          # needs 3 more pages, 1 is free
    with pytest.raises(CacheError, match="not held"):
        c.begin_step([s[0], 3], [1, 1])
    with pytest.raises(CacheError, match="twice"):
        c.begin_step([s[0], s[0]], [1, 1])
    with pytest.raises(CacheError, match="at least one token"):
        c.begin_step([s[0]], [0])
    after = (c.lens.copy(), [g.pages.free_count for g in c.groups if hasattr(g, "pages")])
    assert np.array_equal(before[0], after[0]) and before[1] == after[1]
    c.check()


def test_close_twice_is_refused():
    c = make()
    s = c.open(2)
    c.close([s[0]])
    with pytest.raises(CacheError, match="freed twice"):
        c.close([s[0]])
    with pytest.raises(CacheError, match="freed twice"):
        c.close([s[1], s[1]])
    c.close([s[1]])
    c.check()


def test_sequence_limit():
    c = make(max_tokens=1024, max_seq=100)
    s = c.open(1)
    with pytest.raises(CacheError, match="exceed the limit of 100"):
        c.begin_step(s, [101])
    c.begin_step(s, [100])


def test_window_group_gives_pages_back():
    c = make(max_tokens=2048, window=70)
    win = [i for i in c.kv_groups if c.groups[i].need.window == 70][0]
    full = [i for i in c.kv_groups if c.groups[i].need.window == 0][0]
    (s,) = c.open(1)
    c.begin_step([s], [300])
    c.end_step([s], [300])
    # the next query stands at 300 and sees keys from 231 on: pages 0..2 (positions < 192) are free again
    assert c.groups[win].pages.held_count == 2 and c.groups[full].pages.held_count == 5
    t = c.page_table(win, [s])
    assert list(t[0, :3]) == [-1, -1, -1] and t[0, 3] >= 0 and t[0, 4] >= 0
    for _ in range(200):
        c.begin_step([s], [1])
        c.end_step([s], [1])
    assert c.groups[win].pages.held_count <= 3 and c.groups[full].pages.held_count == 8
    c.check()
    c.close([s])
    assert c.groups[win].pages.held_count == 0
    c.check()


def test_fixed_size_state_is_zeroed_on_open():
    c = make()
    s = c.open(2)
    state = c.views[0].storage
    state[s[0]] = 3.0
    state[s[1]] = 4.0
    c.close(s)
    s2 = c.open(1)
    assert s2 == [s[0]] and float(state[s2[0]].abs().sum()) == 0.0 and float(state[s[1]].abs().sum()) > 0


def test_shared_cache_view():
    needs = [KVNeed(2, 16, 0), KVNeed(2, 16, 0), StateNeed((1, 4))]
    c = Cache(needs, [None, 0, None], 256, dtype=torch.float32, device="cpu")
    assert c.views[1].storage.data_ptr() == c.views[0].storage.data_ptr()
    assert c.views[0].owner and not c.views[1].owner and len(c.groups) == 2
    assert c.groups[c.views[0].group].calls == [(0, 0)]


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make(max_tokens=64 * 40, window=90, max_slots=12)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and c.slots.free_count:
            for s in c.open(rng.randint(1, min(3, c.slots.free_count))):
                live[s] = 0
        elif r < 0.4 and live:
            gone = rng.sample(sorted(live), rng.randint(1, min(3, len(live))))
            c.close(gone)
            for s in gone:
                del live[s]
        elif live:
            batch = rng.sample(sorted(live), rng.randint(1, len(live)))
            q = [rng.choice([1, 1, 1, 7, 64, 65, 130]) for _ in batch]
            try:
                c.begin_step(batch, q)
            except CacheError:
                continue
            c.end_step(batch, q)
            for s, n in zip(batch, q):
                live[s] += n
        c.check()
        assert {s: int(c.lens[s]) for s in live} == live
    c.close(sorted(live))
    c.check()
    assert c.tokens_held() == 0 and c.slots.held_count == 0


@pytest.mark.parametrize("window", [0, 100])
def test_decoding_the_same_batch_step_after_step(window):
    """The short cut for "the last step's batch again, one token each" reserves pages exactly where the full
    path would, notices a sequence that ends, a slot that is closed, and the context's end."""
    c = make(max_tokens=2048, window=window, max_slots=4, max_seq=400)
    slots = c.open(3)
    first = [5, 64, 190]
    c.begin_step(slots, first)
    c.end_step(slots, first)
    lens = list(first)
    versions = c.tables_version()
    for step in range(150):
        starts = c.begin_step(slots, [1, 1, 1])
        assert list(starts) == lens
        for gi in c.kv_groups:
            g = c.groups[gi]
            for s, n in zip(slots, lens):
                assert int(g.end_held[s]) == -(-(n + 1) // 64)         # the page the new position lies in is held
                assert g.table[s, n // 64] >= 0
        crossed = any(n % 64 == 0 for n in lens)
        assert (c.tables_version() != versions) == crossed or window > 0
        c.end_step(slots, [1, 1, 1])
        versions = c.tables_version()
        lens = [n + 1 for n in lens]
        c.check()
    # the third sequence stands at 340: 60 more positions fit, the 61st does not
    for _ in range(60):
        c.begin_step(slots, [1, 1, 1])
        c.end_step(slots, [1, 1, 1])
    with pytest.raises(CacheError, match="exceed the limit"):
        c.begin_step(slots, [1, 1, 1])
    c.close([slots[2]])
    with pytest.raises(CacheError, match="not held"):
        c.begin_step(slots, [1, 1, 1])
    c.begin_step(slots[:2], [1, 1])
    c.end_step(slots[:2], [1, 1])
    c.check()


@pytest.mark.parametrize("window", [0, 70])
def test_a_failed_step_gives_its_pages_back(window):
    """`begin_step` reserved, then a kernel failed: `abort_step` puts the books back (pages, tables, lengths),
    also for a window group that has given pages back before, and the slots can step again or be closed."""
    c = make(max_tokens=2048, window=window)
    a, b = c.open(2)
    c.begin_step([a, b], [200, 10])
    c.end_step([a, b], [200, 10])

    def books():
        return ([int(c.groups[g].pages.held_count) for g in c.kv_groups], [c.groups[g].table.copy() for g in c.kv_groups],
                c.lens.copy(), c.tokens_held())

    before = books()
    versions = c.tables_version()
    c.begin_step([a, b], [130, 60])                 # both cross page boundaries
    assert books()[0] != before[0]
    c.abort_step([a, b])
    after = books()
    assert after[0] == before[0] and all((x == y).all() for x, y in zip(after[1], before[1]))
    assert (after[2] == before[2]).all() and after[3] == before[3]
    assert c.tables_version() != versions            # a staged copy of the tables is stale
    c.check()
    c.begin_step([a], [1])                           # a step inside the pages already held: nothing to undo
    c.abort_step([a])
    assert books()[0] == before[0]
    starts = c.begin_step([a, b], [130, 60])
    assert list(starts) == [200, 10]
    c.end_step([a, b], [130, 60])
    c.check()
    c.close([a, b])
    c.check()
    assert c.tokens_held() == 0


def test_a_call_with_several_needs():
    """A mixer may keep several things per sequence (say a window of inputs, a running state and keys/values).
    Each need lies in the group of its kind and geometry, beside other calls' equal needs, and the call's view
    hands them out in declaration order; a reader of that call's cache sees the same storage."""
    both = (StateNeed((2, 8)), StateNeed((8,), "float32"), KVNeed(2, 16, 0))
    needs = [both, StateNeed((2, 8)), KVNeed(2, 16, 0), both, None]
    c = Cache(needs, [None, None, None, None, 0], 512, dtype=torch.bfloat16, device="cpu")
    assert len(c.groups) == 3 and len(c.kv_groups) == 1
    v = c.views[0]
    assert len(v) == 3 and v.storage is v[0].storage and v.owner
    assert tuple(v[0].storage.shape[1:]) == (2, 8) and v[0].storage.dtype == torch.bfloat16
    assert tuple(v[1].storage.shape[1:]) == (8,) and v[1].storage.dtype == torch.float32
    assert tuple(v[2].storage.shape[1:]) == (2, 2, 64, 16) and v[2].group == c.kv_groups[0]
    assert v[0].group == c.views[1].group and v[0].storage.data_ptr() != c.views[1].storage.data_ptr()
    assert v[2].group == c.views[2].group and len(c.views[1]) == 1 and c.views[1][0] is c.views[1]
    ptrs = {c.views[i][k].storage.data_ptr() for i in (0, 3) for k in range(3)}
    assert len(ptrs) == 6                                            # two calls of the same kind: storage of their own
    assert len(c.views[4]) == 0 and c.views[4].storage is None       # declares nothing: reads nothing
    shared = Cache([both, both], [None, 0], 512, dtype=torch.bfloat16, device="cpu")
    r = shared.views[1]
    assert not r.owner and [r[k].storage.data_ptr() for k in range(3)] == [shared.views[0][k].storage.data_ptr() for k in range(3)]
    # every state is zeroed when a slot is opened, pages are counted once per group
    (s,) = c.open(1)
    c.begin_step([s], [70])
    c.end_step([s], [70])
    assert c.groups[c.kv_groups[0]].pages.held_count == 2
    for k in (0, 1):
        v[k].storage[s] = 7
    c.close([s])
    (s2,) = c.open(1)
    assert s2 == s and all(float(v[k].storage[s].abs().sum()) == 0 for k in (0, 1))
    c.check()
    # the calls of a state group are pieces of one allocation: opening a slot zeroes its row in every call's
    # piece and no other row, and every piece is contiguous and starts on a 16-byte boundary
    c.close([s2])
    states = [c.views[i][k].storage for i, k in ((0, 0), (1, 0), (3, 0), (0, 1), (3, 1))]
    for t in states:
        t.fill_(5)
        assert t.is_contiguous() and t.data_ptr() % 16 == 0
    got = c.open(2)
    for t in states:
        rows = t.reshape(t.shape[0], -1).float().abs().sum(1)
        assert all(float(rows[i]) == 0 for i in got)
        assert all(float(rows[i]) > 0 for i in range(t.shape[0]) if i not in got)
