"""The cache manager: pages of keys and values, block tables, fixed-size state slots.

Host bookkeeping is plain Python and works without a GPU (the tests drive it on the CPU);
device tensors are attached when a device is given.

Vocabulary
  slot    the index a live request holds from admission to release; it picks the request's
          row in every block table and in every state tensor.
  group   the stages (entries of the model's run order) whose caches have the same needs
          (kv heads, head size, window).  A group has its own page pool, its own block
          table and one tensor `[stages, pages, 2, kv_heads, page_size, head_dim]`; a page
          id covers that page in all of the group's stages.
  table   table[slot][i] = physical page holding positions [i*P, (i+1)*P) of that request.
          Resident on the device; the host keeps a mirror and a list of changed entries
          that the next step uploads (`drain_updates`).

The reference keeps one pool and host-side tables that it re-packs and uploads per layer
per step (src/engine/block_table_manager.cpp:17-275, src/ops/attention.cu:959-1020), frees
pages only on an explicit release (src/engine/paged_generate_engine.cpp:386-395) and has no
groups.  Kept from it: LIFO free list that hands out 0,1,2,... first
(block_table_manager.cpp:213-253), all-or-nothing `ensure` (block_table_manager.cpp:60-89),
errors on double free and bad ids (block_table_manager.cpp:226-235,270-274), and the address
rule page*P + pos%P (block_table_manager.cpp:91-122).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


class OutOfPages(RuntimeError):
    """Not enough free pages (or no free slot) for what was asked; nothing was taken."""


class CacheError(RuntimeError):
    """A misuse of the cache manager: double free, unknown slot, shrinking a request."""


class PagePool:
    """Free list of physical page ids, last-in first-out; a fresh pool hands out 0, 1, 2, ..."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._used = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise CacheError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"not enough free pages: want {n}, have {len(self._free)} of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._used[p] = True
        return out

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise CacheError(f"page id {p} is outside the pool")
            if not self._used[p]:
                raise CacheError(f"page {p} freed twice")
        if len(set(pages)) != len(pages):
            raise CacheError("the same page given back twice in one call")
        for p in pages:
            self._used[p] = False
            self._free.append(p)

    def used_pages(self) -> List[int]:
        return [i for i, u in enumerate(self._used) if u]


@dataclass(frozen=True)
class PagedNeed:
    """What a stage asks of the cache when it keeps keys and values by position: per position,
    `num_kv_heads` keys of `head_dim` values and as many values of `value_dim` (None: of
    `head_dim` too, and keys and values then share one tensor with an axis of two)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every earlier position stays; w: only the last w
    value_dim: Optional[int] = None

    @property
    def key_width(self) -> int:
        return self.head_dim

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """What a stage asks when it keeps a state of fixed size per request (zeroed at admission)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class CacheGroup:
    def __init__(self, need: PagedNeed, stages: List[int], page_size: int, num_pages: int,
                 max_slots: int, max_pages_per_request: int):
        self.need = need
        self.stages = list(stages)
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.max_pages_per_request = max_pages_per_request
        self.table = np.full((max_slots, max_pages_per_request), -1, dtype=np.int32)
        self.first_held = [0] * max_slots     # lowest logical page still held
        self.num_logical = [0] * max_slots    # logical pages ever appended
        self.pending: List[Tuple[int, int]] = []    # (flat table index, page id) not yet on the device
        self.kv = None                        # device tensor [stages, pages, 2, kv_heads, P, d] when keys and values are equally wide
        self.keys = None                      # [stages, pages, kv_heads, P, key width] (a view of `kv` when that exists)
        self.values = None                    # [stages, pages, kv_heads, P, value width]
        self.table_dev = None                 # device int32 [max_slots, max_pages_per_request]

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def missing(self, slot: int, new_len: int) -> int:
        return max(0, self.pages_for(new_len) - self.num_logical[slot])

    def append(self, slot: int, new_len: int) -> None:
        want = self.pages_for(new_len)
        if want > self.max_pages_per_request:
            raise CacheError(f"a request of {new_len} tokens needs {want} pages; the table holds "
                             f"{self.max_pages_per_request}")
        have = self.num_logical[slot]
        if want <= have:
            return
        pages = self.pool.take(want - have)
        for i, p in enumerate(pages):
            self.table[slot, have + i] = p
            self.pending.append((slot * self.max_pages_per_request + have + i, p))
        self.num_logical[slot] = want

    def trim_window(self, slot: int, length: int) -> int:
        """Give back pages every position of which lies before the window of the next query
        (position `length`, which sees keys > length - window).  Returns how many."""
        w = self.need.window
        if w is None:
            return 0
        first_needed = max(0, length - w + 1)
        keep_from = min(first_needed // self.page_size, self.num_logical[slot])
        lo = self.first_held[slot]
        if keep_from <= lo:
            return 0
        self.pool.give([int(self.table[slot, i]) for i in range(lo, keep_from)])
        self.first_held[slot] = keep_from
        return keep_from - lo

    def release(self, slot: int) -> None:
        lo, hi = self.first_held[slot], self.num_logical[slot]
        self.pool.give([int(self.table[slot, i]) for i in range(lo, hi)])
        self.first_held[slot] = 0
        self.num_logical[slot] = 0

    def held_pages(self, slot: int) -> List[int]:
        return [int(self.table[slot, i]) for i in range(self.first_held[slot], self.num_logical[slot])]


class CacheManager:
    """Owns every group's pages and tables, the slots, and the per-slot state tensors.

    stage_needs[s] is a `PagedNeed`, a `StateNeed`, None (the stage keeps nothing), or
    ('borrow', t): stage s reads the cache of the earlier stage t.
    """

    def __init__(self, stage_needs: Sequence, page_size: int, max_total_tokens: int, max_slots: int,
                 max_request_tokens: Optional[int] = None, dtype=None, device=None,
                 extra_state: Optional[Dict[str, StateNeed]] = None):
        if page_size <= 0:
            raise CacheError("--page-size must be positive")
        if max_slots <= 0 or max_total_tokens <= 0:
            raise CacheError("max_slots and max_total_tokens must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.num_pages = (max_total_tokens + page_size - 1) // page_size
        # A request can be longer than the pool only if every group forgets old positions.
        keeps_all = any(isinstance(n, PagedNeed) and n.window is None for n in stage_needs)
        self.max_request_tokens = max_request_tokens or max_total_tokens
        if keeps_all:
            self.max_request_tokens = min(self.max_request_tokens, self.num_pages * page_size)
        max_pages_per_request = (self.max_request_tokens + page_size - 1) // page_size
        self.device = device
        self.dtype = dtype

        self.groups: List[CacheGroup] = []
        self.stage_group: Dict[int, Tuple[int, int]] = {}     # stage -> (group index, index inside group)
        self.stage_state: Dict[int, StateNeed] = {}
        by_need: Dict[PagedNeed, int] = {}
        for s, need in enumerate(stage_needs):
            if isinstance(need, PagedNeed):
                gi = by_need.get(need)
                if gi is None:
                    gi = len(self.groups)
                    by_need[need] = gi
                    self.groups.append(CacheGroup(need, [], page_size, self.num_pages, max_slots,
                                                  max_pages_per_request))
                g = self.groups[gi]
                self.stage_group[s] = (gi, len(g.stages))
                g.stages.append(s)
            elif isinstance(need, StateNeed):
                self.stage_state[s] = need
        for s, need in enumerate(stage_needs):
            if isinstance(need, tuple) and need and need[0] == "borrow":
                src = need[1]
                if src not in self.stage_group:
                    raise CacheError(f"stage {s} borrows the cache of stage {src}, which has none")
                self.stage_group[s] = self.stage_group[src]

        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots
        self._length = [0] * max_slots
        self.state: Dict[object, object] = {}     # stage index or name -> device tensor [max_slots, *shape]
        self._extra_state = dict(extra_state or {})
        if device is not None:
            self._allocate_device()

    # ---- device side ---------------------------------------------------------------------
    def _allocate_device(self) -> None:
        import torch
        for g in self.groups:
            n = g.need
            if n.key_width == n.value_width:
                g.kv = torch.zeros((len(g.stages), g.pool.num_pages, 2, n.num_kv_heads, self.page_size, n.head_dim),
                                   dtype=self.dtype, device=self.device)
                g.keys, g.values = g.kv[:, :, 0], g.kv[:, :, 1]
            else:
                g.keys = torch.zeros((len(g.stages), g.pool.num_pages, n.num_kv_heads, self.page_size, n.key_width),
                                     dtype=self.dtype, device=self.device)
                g.values = torch.zeros((len(g.stages), g.pool.num_pages, n.num_kv_heads, self.page_size, n.value_width),
                                       dtype=self.dtype, device=self.device)
            # -1 like the host mirror: a kernel that reads an entry no request was ever given refuses
            # it (status 3 or 4) instead of reading page 0 of someone else
            g.table_dev = torch.full((self.max_slots, g.max_pages_per_request), -1, dtype=torch.int32,
                                     device=self.device)
        for key, need in list(self.stage_state.items()) + list(self._extra_state.items()):
            self.state[key] = torch.zeros((self.max_slots,) + tuple(need.shape),
                                          dtype=getattr(torch, need.dtype), device=self.device)

    def stage_cache(self, stage: int):
        """(kv tensor [pages, 2, kv_heads, P, d] of the stage, or None when its keys and values differ
        in width; its group's device table; the group)."""
        gi, k = self.stage_group[stage]
        g = self.groups[gi]
        return (g.kv[k] if g.kv is not None else None), g.table_dev, g

    def stage_pages(self, stage: int):
        """(keys [pages, kv_heads, P, key width], values [pages, kv_heads, P, value width]) of the stage."""
        gi, k = self.stage_group[stage]
        g = self.groups[gi]
        return (g.keys[k] if g.keys is not None else None), (g.values[k] if g.values is not None else None)

    def bytes_per_token(self) -> int:
        import torch
        esz = torch.empty((), dtype=self.dtype).element_size() if self.dtype is not None else 2
        return sum(g.need.num_kv_heads * (g.need.key_width + g.need.value_width) * esz * len(g.stages)
                   for g in self.groups)

    # ---- slots -----------------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self) -> int:
        """Take a slot for a new request; its state tensors are zeroed."""
        if not self._free_slots:
            raise OutOfPages("no free request slot")
        slot = self._free_slots.pop()
        self._live[slot] = True
        self._length[slot] = 0
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def _check_live(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots) or not self._live[slot]:
            raise CacheError(f"slot {slot} is not held by a request")

    def length(self, slot: int) -> int:
        self._check_live(slot)
        return self._length[slot]

    def release(self, slot: int) -> None:
        """The request is over (finished or preempted): every page and the slot go back."""
        self._check_live(slot)
        for g in self.groups:
            g.release(slot)
        self._live[slot] = False
        self._length[slot] = 0
        self._free_slots.append(slot)

    # ---- pages -----------------------------------------------------------------------------
    def pages_missing(self, slot: int, new_len: int) -> List[int]:
        self._check_live(slot)
        return [g.missing(slot, new_len) for g in self.groups]

    def can_hold(self, wants: Sequence[Tuple[Optional[int], int]]) -> bool:
        """Would `ensure` succeed for all of (slot or None for a request not yet admitted,
        new length) together?"""
        need = [0] * len(self.groups)
        new_slots = 0
        for slot, new_len in wants:
            if new_len > self.max_request_tokens:
                return False
            if slot is None:
                new_slots += 1
                for i, g in enumerate(self.groups):
                    need[i] += g.pages_for(new_len)
            else:
                for i, m in enumerate(self.pages_missing(slot, new_len)):
                    need[i] += m
        return new_slots <= self.free_slots and all(n <= g.pool.free_count for n, g in zip(need, self.groups))

    def reserve(self, need: Sequence[int], slot: Optional[int], new_len: int) -> Optional[List[int]]:
        """`need` (pages per group already promised in this step) plus what (slot or None, new
        length) wants, or None if that does not fit the free pages.  `can_hold` one request at a
        time, for callers that build a step up."""
        if new_len > self.max_request_tokens:
            return None
        if slot is None:
            total = [n + g.pages_for(new_len) for n, g in zip(need, self.groups)]
        else:
            total = [n + m for n, m in zip(need, self.pages_missing(slot, new_len))]
        return total if all(t <= g.pool.free_count for t, g in zip(total, self.groups)) else None

    def ensure(self, slot: int, new_len: int) -> None:
        """Make room for positions [0, new_len) of the request, in every group, or take nothing."""
        self._check_live(slot)
        if new_len < self._length[slot]:
            raise CacheError("a request's cache never shrinks")
        if new_len > self.max_request_tokens:
            raise OutOfPages(f"a request of {new_len} tokens exceeds the limit of {self.max_request_tokens}")
        for g, m in zip(self.groups, self.pages_missing(slot, new_len)):
            if m > g.pool.free_count:
                raise OutOfPages(f"not enough free pages: want {m}, have {g.pool.free_count} of {g.pool.num_pages}")
        for g in self.groups:
            g.append(slot, new_len)

    def commit(self, slot: int, new_len: int) -> int:
        """The step that filled positions up to new_len has been issued: record the length and
        give back pages that a window has passed.  Returns the number of pages given back."""
        self._check_live(slot)
        if new_len < self._length[slot]:
            raise CacheError("a request's cache never shrinks")
        self._length[slot] = new_len
        return sum(g.trim_window(slot, new_len) for g in self.groups)

    def drain_updates(self) -> List[Tuple[np.ndarray, np.ndarray]]:
        """Per group: (flat table indices, page ids) changed since the last call."""
        out = []
        for g in self.groups:
            if g.pending:
                arr = np.asarray(g.pending, dtype=np.int32)
                out.append((arr[:, 0].copy(), arr[:, 1].copy()))
                g.pending.clear()
            else:
                out.append((np.empty(0, np.int32), np.empty(0, np.int32)))
        return out

    # ---- checks ----------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for gi, g in enumerate(self.groups):
            held: List[int] = []
            for slot in range(self.max_slots):
                if self._live[slot]:
                    held += g.held_pages(slot)
                elif g.num_logical[slot] or g.first_held[slot]:
                    raise CacheError(f"group {gi}: released slot {slot} still has pages")
            if len(set(held)) != len(held):
                raise CacheError(f"group {gi}: a page is held twice")
            used = set(g.pool.used_pages())
            if used != set(held):
                raise CacheError(f"group {gi}: pool says {sorted(used)} are out, requests hold {sorted(held)}")
            if g.pool.free_count + len(held) != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.free_count} free + {len(held)} held != {g.pool.num_pages}")
        live = sum(self._live)
        if live + len(self._free_slots) != self.max_slots or len(set(self._free_slots)) != len(self._free_slots):
            raise CacheError("slot accounting is off")
