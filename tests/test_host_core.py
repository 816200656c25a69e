"""The native host code on its own (no GPU): a step's requests handled at once by the cache manager,
and the packing of a step's arrays against a restatement in numpy."""
import random

import numpy as np
import pytest

from litellmengine_b200.cache import CacheError, CacheManager, OutOfPages, PagedNeed
from litellmengine_b200.csrc import host


def manager(pages=8, page=4, slots=4, window=None):
    needs = [PagedNeed(2, 16), PagedNeed(2, 16, window=window)] if window else [PagedNeed(2, 16)]
    return CacheManager(needs, page_size=page, max_total_tokens=pages * page, max_slots=slots, max_request_tokens=64 if window else None)


def test_a_step_takes_room_for_all_its_requests_or_for_none():
    m = manager(pages=8)
    a, b, c = m.admit(), m.admit(), m.admit()
    slots = np.asarray([a, b, c], dtype=np.int32)
    assert m.lengths(slots).tolist() == [0, 0, 0]
    m.ensure_all(slots, np.asarray([5, 9, 4], dtype=np.int64))             # 2 + 3 + 1 pages
    assert m.groups[0].pool.free_count == 2
    m.commit_all(slots, np.asarray([5, 9, 4], dtype=np.int64))
    assert m.lengths(slots).tolist() == [5, 9, 4]
    before = [m.groups[0].held_pages(s) for s in (a, b, c)]
    with pytest.raises(OutOfPages, match="do not fit"):                     # 1 + 1 + 1 more pages, two are free
        m.ensure_all(slots, np.asarray([9, 13, 8], dtype=np.int64))
    assert [m.groups[0].held_pages(s) for s in (a, b, c)] == before and m.groups[0].pool.free_count == 2
    with pytest.raises(CacheError, match="never shrinks"):
        m.ensure_all(slots, np.asarray([5, 8, 4], dtype=np.int64))
    with pytest.raises(CacheError, match="not held"):
        m.lengths(np.asarray([a, 3], dtype=np.int32))
    m.ensure_all(slots[:2], np.asarray([8, 13], dtype=np.int64))            # 0 + 1 pages
    idx, val = m.drain_updates()[0]
    assert len(idx) == 7 and sorted(val.tolist()) == list(range(7))
    m.check_invariants()
    for s in (a, b, c):
        m.release(s)
    m.check_invariants()
    assert m.groups[0].pool.free_count == 8 and m.free_slots == 4


def test_committing_a_step_gives_back_what_a_window_has_passed():
    m = manager(pages=12, window=6)
    a, b = m.admit(), m.admit()
    slots = np.asarray([a, b], dtype=np.int32)
    lens = np.asarray([14, 3], dtype=np.int64)
    m.ensure_all(slots, lens)
    assert m.commit_all(slots, lens) == 2                                   # positions 0..7 of `a` lie before its window
    full, win = m.groups
    assert len(full.held_pages(a)) == 4 and len(win.held_pages(a)) == 2 and win.first_held[a] == 2
    m.check_invariants()


def pack(offsets, size, slot, past, q_len, fed, tokens, want, want_count, want_cap):
    base = np.full(size, -7, dtype=np.int32)
    facts = np.empty(4, dtype=np.int64)
    a32 = lambda v: np.ascontiguousarray(v, dtype=np.int32)
    a64 = lambda v: np.ascontiguousarray(v, dtype=np.int64)
    slot, fed, want_count, past, q_len, tokens, want = a32(slot), a32(fed), a32(want_count), a64(past), a64(q_len), a64(tokens), a64(want)
    off = a64(offsets)
    rc = host.lib().hc_pack_step(base.ctypes.data, off.ctypes.data, len(slot), slot.ctypes.data, past.ctypes.data, q_len.ctypes.data,
                                 fed.ctypes.data, tokens.ctypes.data, want.ctypes.data, want_count.ctypes.data, want_cap, facts.ctypes.data)
    return rc, base, facts.tolist()


def test_packing_a_step_against_numpy():
    rng = random.Random(3)
    for _ in range(50):
        B = rng.randint(1, 9)
        q_len = [rng.choice((1, 1, 2, 5, 17)) for _ in range(B)]
        past = [rng.randint(0, 40) for _ in range(B)]
        slot = rng.sample(range(16), B)
        fed = [rng.choice((-1, -1, rng.randint(0, 15))) for _ in range(B)]
        T = sum(q_len)
        tokens = [rng.randrange(1000) for _ in range(T)]
        wants = [sorted(rng.sample(range(n), rng.randint(0, min(n, 3)))) for n in q_len]
        cap, want_cap = 160, 16
        names = ("token_ids", "positions", "token_entry", "entry_slot", "entry_q_start", "entry_q_len", "entry_kv_len",
                 "want_rows", "want_slot", "counts")
        sizes = (cap, cap, cap, 16, 16, 16, 16, cap, cap, 8)
        offsets = np.cumsum((0,) + sizes[:-1])
        rc, base, facts = pack(offsets, sum(sizes), slot, past, q_len, fed, tokens, [j for w in wants for j in w],
                               [len(w) for w in wants], want_cap)
        assert rc == 0
        view = {n: base[o:o + s] for n, o, s in zip(names, offsets, sizes)}
        q_start = np.cumsum(q_len) - np.asarray(q_len)
        expect_tokens = list(tokens)
        for e in range(B):
            if fed[e] >= 0:
                expect_tokens[q_start[e] + q_len[e] - 1] = -1 - fed[e]
        assert view["token_ids"][:T].tolist() == expect_tokens
        assert view["positions"][:T].tolist() == [past[e] + i for e in range(B) for i in range(q_len[e])]
        assert view["token_entry"][:T].tolist() == [e for e in range(B) for _ in range(q_len[e])]
        assert view["entry_slot"][:B].tolist() == slot and view["entry_q_start"][:B].tolist() == q_start.tolist()
        assert view["entry_q_len"][:B].tolist() == q_len
        assert view["entry_kv_len"][:B].tolist() == [p + n for p, n in zip(past, q_len)]
        rows = [q_start[e] + j for e in range(B) for j in wants[e]]
        W = len(rows)
        assert view["want_rows"][:W].tolist() == rows and view["want_slot"][:W].tolist() == [slot[e] for e in range(B) for _ in wants[e]]
        assert all(v == 0 for v in view["want_rows"][W:want_cap]) and all(v == -7 for v in view["want_rows"][max(W, want_cap):])
        assert view["counts"][:3].tolist() == [T, B, W]
        assert facts == [T, W, max(q_len), max(p + n for p, n in zip(past, q_len))]
        assert all(v == -7 for n in ("token_ids", "positions", "token_entry") for v in view[n][T:])     # nothing beyond what it was given


def test_packing_refuses_a_wanted_place_outside_its_entry():
    offsets = np.arange(10) * 8
    rc, _, _ = pack(offsets, 80, [0], [0], [3], [-1], [1, 2, 3], [3], [1], 4)
    assert rc == 2 and "outside the entry's 3 tokens" in host.last_error()
