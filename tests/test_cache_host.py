"""The cache's bookkeeping on the host: no slot or page lost, held twice or
freed twice; requests that cannot be met change nothing (no GPU)."""
import random

import pytest
import torch

from nnis_b200.cache import (PAGE_SIZE, CacheFull, CacheManager, FreeList, KVRequest, SlotError,
                             StateRequest)


def make(max_tokens=64 * 8, max_slots=4, requests=None, max_positions=10_000):
    requests = requests if requests is not None else [KVRequest(2, 16), KVRequest(2, 16)]
    return CacheManager(requests, torch.float32, torch.device("cpu"), max_tokens, max_slots,
                        max_positions)


def test_free_list_never_hands_out_twice_and_reuses_lowest():
    f = FreeList(3, "slot")
    a, b, c = f.take(), f.take(), f.take()
    assert sorted((a, b, c)) == [0, 1, 2]
    with pytest.raises(CacheFull):
        f.take()
    f.give(1)
    with pytest.raises(SlotError):
        f.give(1)
    with pytest.raises(SlotError):
        f.give(9)
    assert f.take() == 1
    f.check()


def test_slots_are_given_back_and_used_again():
    c = make()
    held = [c.acquire() for _ in range(4)]
    assert sorted(held) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        c.acquire()
    c.release(2)
    with pytest.raises(SlotError):
        c.release(2)
    assert c.acquire() == 2
    c.check()


def test_pages_follow_lengths_and_return_on_release():
    c = make()
    s = c.acquire()
    c.reserve([s], [1])
    c.commit([s], [1])
    assert len(c.page_table(0, s)) == 1
    c.reserve([s], [PAGE_SIZE])
    assert len(c.page_table(0, s)) == 1
    c.reserve([s], [PAGE_SIZE + 1])
    c.commit([s], [PAGE_SIZE + 1])
    assert len(c.page_table(0, s)) == 2 and c.length(s) == PAGE_SIZE + 1
    assert c.usage()["pages_held"] == [2]
    c.release(s)
    assert c.usage()["pages_held"] == [0]
    c.check()


def test_layers_of_one_shape_share_a_group_and_others_have_their_own():
    c = make(requests=[KVRequest(2, 16), KVRequest(2, 16), KVRequest(1, 32), KVRequest(2, 16, 128),
                       None, StateRequest((3, 5))])
    assert len(c.groups) == 3
    assert c.view(0).group == c.view(1).group != c.view(2).group
    assert c.view(3).group not in (c.view(0).group, c.view(2).group) and c.view(3).window == 128
    assert c.view(0).k.data_ptr() != c.view(1).k.data_ptr()
    assert c.view(4) is None
    assert tuple(c.view(5).state.shape) == (4, 3, 5)
    assert tuple(c.view(2).k.shape) == (8, 1, PAGE_SIZE, 32)


def test_failed_reserve_changes_nothing():
    c = make(max_tokens=PAGE_SIZE * 3)
    a, b = c.acquire(), c.acquire()
    c.reserve([a], [PAGE_SIZE * 2])
    c.commit([a], [PAGE_SIZE * 2])
    before = (list(c.page_table(0, a)), list(c.page_table(0, b)), c.usage()["pages_held"])
    with pytest.raises(CacheFull):
        c.reserve([a, b], [PAGE_SIZE * 2 + 1, PAGE_SIZE + 1])
    assert before == (list(c.page_table(0, a)), list(c.page_table(0, b)), c.usage()["pages_held"])
    with pytest.raises(SlotError):
        c.reserve([a, a], [PAGE_SIZE * 2, PAGE_SIZE * 2])
    with pytest.raises(SlotError):
        c.reserve([3], [1])
    with pytest.raises(SlotError):
        c.reserve([a], [5])  # shrinking
    c.check()


def test_positions_beyond_the_model_are_refused():
    c = make(max_positions=100)
    s = c.acquire()
    with pytest.raises(CacheFull, match="100"):
        c.reserve([s], [101])


def test_window_group_gives_back_pages_behind_the_window():
    c = make(max_tokens=PAGE_SIZE * 8, requests=[KVRequest(1, 16, 70)])
    s = c.acquire()
    c.reserve([s], [300])
    assert c.usage()["pages_held"] == [5]
    c.commit([s], [300])
    # next query at 300 sees keys 231..300: pages 0..2 (keys 0..191) are free again
    assert c.page_table(0, s)[:3] == [-1, -1, -1] and c.usage()["pages_held"] == [2]
    c.release(s)
    c.check()
    assert c.usage()["pages_held"] == [0]


def test_state_rows_are_zeroed_when_a_slot_is_taken():
    c = make(requests=[StateRequest((4,))])
    s = c.acquire()
    c.view(0).state[s] += 3.0
    c.release(s)
    assert c.acquire() == s
    assert float(c.view(0).state[s].abs().sum()) == 0.0


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    c = make(max_tokens=PAGE_SIZE * 40, max_slots=6)
    live = {}
    for _ in range(2000):
        r = rng.random()
        if r < 0.3 and len(live) < 6:
            live[c.acquire()] = 0
        elif r < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.randrange(1, 90)
            try:
                c.reserve([s], [n])
                c.commit([s], [n])
                live[s] = n
            except CacheFull:
                pass
        elif r < 0.9 and live:
            s = rng.choice(list(live))
            live[s] = rng.randrange(0, live[s] + 1)
            c.truncate(s, live[s])
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        assert c.usage()["pages_held"] == [sum(-(-n // PAGE_SIZE) for n in live.values())]
        assert c.usage()["live_tokens"] == sum(live.values())


def test_truncate_gives_pages_back_and_refuses_what_cannot_be_undone():
    c = make(max_tokens=PAGE_SIZE * 8)
    s = c.acquire()
    c.reserve([s], [200])
    c.commit([s], [200])
    kept = list(c.page_table(0, s)[:2])
    with pytest.raises(SlotError, match="cannot truncate"):
        c.truncate(s, 201)
    with pytest.raises(SlotError, match="cannot truncate"):
        c.truncate(s, -1)
    c.truncate(s, 200)  # nothing to do
    c.truncate(s, 65)   # position 64 stays: two pages
    assert c.length(s) == 65 and c.page_table(0, s) == kept and c.usage()["pages_held"] == [2]
    c.truncate(s, 64)
    assert c.page_table(0, s) == kept[:1]
    c.reserve([s], [130])  # grows again from there
    c.commit([s], [130])
    assert c.length(s) == 130 and len(c.page_table(0, s)) == 3
    c.truncate(s, 0)
    assert c.usage()["pages_held"] == [0] and c.length(s) == 0
    c.check()
    other = c.acquire()
    c.release(other)
    with pytest.raises(SlotError, match="not held"):
        c.truncate(other, 0)
    # a windowed group: back to where the window still has its pages, not further
    w = make(max_tokens=PAGE_SIZE * 8, requests=[KVRequest(1, 16, 70)])
    s = w.acquire()
    w.reserve([s], [300])
    w.commit([s], [300])  # pages 0..2 were given back
    w.truncate(s, 280)    # position 280 reads keys 211..: page 3 on
    assert w.length(s) == 280 and w.usage()["pages_held"] == [2]
    before = list(w.page_table(0, s))
    with pytest.raises(SlotError, match="given back pages"):
        w.truncate(s, 250)  # would read keys 181..: page 2 is gone
    assert w.length(s) == 280 and w.page_table(0, s) == before
    w.check()
    # fixed-size state has no earlier value
    st = make(requests=[KVRequest(1, 16), StateRequest((4,))])
    s = st.acquire()
    st.reserve([s], [10])
    st.commit([s], [10])
    with pytest.raises(SlotError, match="fixed-size state"):
        st.truncate(s, 5)
    assert st.length(s) == 10


def test_snapshot_and_restore_bring_back_length_pages_and_state():
    """The way back for a model with fixed-size state: truncate is refused, a
    snapshot taken before the tokens that are taken back restores both."""
    c = make(requests=[KVRequest(2, 16), StateRequest((3,))], max_slots=2)
    s = c.acquire()
    state = c.view(1).state
    c.reserve([s], [70])
    c.commit([s], [70])
    state[s] = torch.tensor([1.0, 2.0, 3.0])
    with pytest.raises(SlotError, match="snapshot"):
        c.truncate(s, 10)
    snap = c.snapshot(s)
    c.reserve([s], [200])
    c.commit([s], [200])
    state[s] = torch.tensor([9.0, 9.0, 9.0])
    assert len(c.page_table(0, s)) == 4
    c.restore(snap)
    assert c.length(s) == 70 and len(c.page_table(0, s)) == 2 and state[s].tolist() == [1.0, 2.0, 3.0]
    assert c.usage()["pages_held"] == [2]
    c.check()
    c.restore(snap)  # again: nothing to forget, the state is written once more
    # a snapshot of a longer sequence than the slot holds now, or of an earlier owner, is refused
    later = c.snapshot(s)
    later.length = 500
    with pytest.raises(SlotError, match="only"):
        c.restore(later)
    c.release(s)
    with pytest.raises(SlotError, match="any more"):
        c.restore(snap)
    again = c.acquire()
    assert again == s
    with pytest.raises(SlotError, match="any more"):
        c.restore(snap)
    c.release(again)
    c.check()


def test_a_slots_version_tells_copies_of_its_page_table_when_they_are_stale():
    """Growth at the end keeps a slot's version; being taken, given back or truncated
    changes it (a truncated table may grow back to the same length with other pages)."""
    c = make(max_tokens=64 * 6, max_slots=2)
    a, b = c.acquire(), c.acquire()
    v0 = c.versions[a]
    c.reserve([a], [130])
    c.commit([a], [130])
    assert c.versions[a] == v0
    table, pages = c.page_table(0, a), list(c.page_table(0, a))
    c.truncate(a, 64)
    assert c.versions[a] == v0 + 1
    c.reserve([b], [64])            # b takes the lowest page that a gave back
    c.commit([b], [64])
    c.reserve([a], [130])
    c.commit([a], [130])
    assert c.page_table(0, a) is table and len(table) == len(pages) and table != pages
    c.release(a)
    assert c.versions[a] == v0 + 2
    c.release(b)
    c.check()
