"""Cache bookkeeping: slots, pages, groups, windows, state (CPU tensors, no GPU)."""
import random

import pytest
import torch

from mdma_b200.cache import CacheFull, FreeList, KVNeed, SequenceCache, StateNeed


def test_free_list_refuses_double_free_and_overdraw():
    fl = FreeList(3, "slot")
    a, b, c = fl.acquire(), fl.acquire(), fl.acquire()
    assert {a, b, c} == {0, 1, 2}
    with pytest.raises(CacheFull):
        fl.acquire()
    fl.release(b)
    with pytest.raises(ValueError):
        fl.release(b)                  # freed twice
    with pytest.raises(ValueError):
        fl.release(7)                  # never given out
    assert fl.acquire() == b           # used again
    fl.check()


def make_cache(window=0, max_tokens=64 * 12, slots=4, ctx=512):
    needs = [KVNeed(2, 16, 0), KVNeed(2, 16, 0), KVNeed(1, 32, window) if window else KVNeed(2, 16, 0)]
    states = [None, StateNeed((4,), torch.float32), None]
    return SequenceCache(needs, states, max_tokens, slots, ctx, torch.float32, "cpu", page_size=64)


def test_groups_have_storage_of_their_own():
    c = make_cache(window=100)
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.sites == [0, 1] and win.sites == [2]
    assert full.k.shape == (2, 12, 64, 2, 16) and win.k.shape == (1, 12, 64, 1, 32)
    assert c.view(0).k.data_ptr() != c.view(1).k.data_ptr()
    assert c.view(2).window == 100 and c.view(0).window == 0
    assert c.view(1).state.shape == (4, 4) and c.view(0).state is None


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    c = make_cache()
    live = {}
    for _ in range(400):
        if live and rng.random() < 0.3:
            slot = rng.choice(list(live))
            c.release(slot)
            del live[slot]
        elif len(live) < 4 and rng.random() < 0.5:
            slot = c.acquire()
            assert slot not in live
            live[slot] = 0
        elif live:
            ext = {s: rng.randint(1, 90) for s in rng.sample(list(live), rng.randint(1, len(live)))}
            why = c.can_extend(ext)
            if why is None:
                c.extend(ext)
                c.commit(ext)
                for s, n in ext.items():
                    live[s] += n
            else:
                before = {g.pages.free_count for g in c.groups}
                with pytest.raises(CacheFull):
                    c.extend(ext)
                assert before == {g.pages.free_count for g in c.groups}     # all or nothing
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            for g in c.groups:
                assert len(g.seq_pages.get(s, {})) == -(-n // 64)
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pages.free_count == g.n_pages for g in c.groups) and c.slots.free_count == 4


def test_pages_of_a_finished_sequence_are_used_again():
    c = make_cache(max_tokens=64 * 3, slots=2)
    a = c.acquire()
    c.extend({a: 150}); c.commit({a: 150})
    b = c.acquire()
    assert c.can_extend({b: 10}) is not None            # 3 pages, all held by a
    c.release(a)
    assert c.can_extend({b: 10}) is None
    c.extend({b: 10}); c.commit({b: 10})
    c.check()


def test_state_is_zeroed_when_a_slot_is_taken():
    c = make_cache()
    s = c.acquire()
    c.view(1).state[s] += 5.0
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and torch.all(c.view(1).state[s2] == 0)


def test_window_group_gives_pages_back():
    c = make_cache(window=100, max_tokens=64 * 40, slots=2, ctx=2048)
    s = c.acquire()
    full, win = c.groups
    total = 0
    for n in [300] + [1] * 200:
        c.extend({s: n}); c.commit({s: n})
        total += n
        c.check()
        assert len(full.seq_pages[s]) == -(-total // 64)
        first_needed = max(0, total + 1 - 100) // 64
        assert min(win.seq_pages[s]) == first_needed           # older pages were released
        assert len(win.seq_pages[s]) <= 100 // 64 + 2
    c.release(s)
    c.check()


def test_context_limit():
    c = make_cache(ctx=128)
    s = c.acquire()
    assert "context" in c.can_extend({s: 129})
    assert c.can_extend({s: 128}) is None


def test_truncate_gives_pages_back_and_refuses_what_cannot_be_rewound():
    needs = [KVNeed(2, 16, 0)]
    c = SequenceCache(needs, [None], 64 * 8, 2, 512, torch.float32, "cpu", page_size=64)
    s = c.acquire()
    c.extend({s: 300}); c.commit({s: 300})
    free = c.groups[0].pages.free_count
    c.truncate(s, 70)
    assert c.length(s) == 70 and c.groups[0].pages.free_count == free + 3      # pages 2..4 returned
    c.check()
    c.extend({s: 100}); c.commit({s: 100})                                     # and it can grow again
    assert c.length(s) == 170
    with pytest.raises(ValueError):
        c.truncate(s, 171)
    stateful = make_cache()
    t = stateful.acquire()
    with pytest.raises(ValueError, match="state"):
        stateful.truncate(t, 0)


def test_token_by_token_growth_holds_exactly_the_pages_it_needs():
    """A sequence that grows one token a step (decoding) looks only at its newest page each step; the pages it
    ends up with are the ones a single extension to the same length would take, also with a window and
    after a rewind."""
    for window in (0, 100):
        c = make_cache(window=window, max_tokens=64 * 24, slots=2, ctx=700)
        a, b = c.acquire(), c.acquire()
        c.extend({a: 130}); c.commit({a: 130})
        for _ in range(300):
            c.extend({a: 1}); c.commit({a: 1})
        c.extend({b: 430}); c.commit({b: 430})
        c.check()
        for g in c.groups:
            pages_a, pages_b = set(g.seq_pages[a]), set(g.seq_pages[b])
            if g.need.window:
                # what has left the window is given back; what is kept covers the window and the newest page
                first_live = max(0, 430 + 1 - g.need.window) // 64
                assert pages_a == set(range(first_live, (430 - 1) // 64 + 1))
                assert pages_b >= pages_a
            else:
                assert pages_a == pages_b == set(range((430 - 1) // 64 + 1))
    c = SequenceCache([KVNeed(2, 16, 0)], [None], 64 * 24, 1, 700, torch.float32, "cpu", page_size=64)    # no state: may rewind
    a = c.acquire()
    c.extend({a: 200}); c.commit({a: 200})
    c.truncate(a, 70)
    for _ in range(100):
        c.extend({a: 1}); c.commit({a: 1})
    c.check()
    assert all(set(g.seq_pages[a]) == {0, 1, 2} for g in c.groups)
