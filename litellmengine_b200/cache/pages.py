"""The cache manager: pages of keys and values, block tables, fixed-size state slots.

The bookkeeping (pools, tables, slots) is native code (`csrc/host_core.cpp`, no device needed: the
tests drive it on the CPU); the classes here give it its names, raise its errors and own the device
tensors, which are attached when a device is given.

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

import ctypes

import numpy as np

from ..csrc import host


class OutOfPages(RuntimeError):
    """Not enough free pages (or no free slot) for what was asked; nothing was taken."""


class CacheError(RuntimeError):
    """A misuse of the cache manager: double free, unknown slot, shrinking a request."""


def _check(rc: int) -> None:
    if rc == 1:
        raise OutOfPages(host.last_error())
    if rc:
        raise CacheError(host.last_error())


def _int32(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


class PagePool:
    """Free list of physical page ids, last-in first-out; a fresh pool hands out 0, 1, 2, ..."""

    def __init__(self, num_pages: int, _borrowed=None):
        self._lib = host.lib()
        self._own = _borrowed is None
        self._h = self._lib.hc_pool_new(int(num_pages)) if self._own else _borrowed
        if not self._h:
            raise CacheError(host.last_error())
        self.num_pages = self._lib.hc_pool_num_pages(self._h)

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            self._lib.hc_pool_delete(self._h)
            self._h = None

    @property
    def free_count(self) -> int:
        return self._lib.hc_pool_free_count(self._h)

    def take(self, n: int) -> List[int]:
        out = np.empty(max(int(n), 0), dtype=np.int32)
        _check(self._lib.hc_pool_take(self._h, int(n), out.ctypes.data))
        return out.tolist()

    def give(self, pages: Sequence[int]) -> None:
        arr = _int32(list(pages))
        _check(self._lib.hc_pool_give(self._h, arr.ctypes.data, len(arr)))

    def used_pages(self) -> List[int]:
        out = np.empty(self.num_pages, dtype=np.int32)
        return out[:self._lib.hc_pool_used(self._h, out.ctypes.data)].tolist()


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
    """One group's view of the native records: its pool, its table `[slots, pages per request]`
    (-1 where nothing is held), and per slot the lowest logical page still held and the number of
    logical pages ever appended (numpy views of the library's memory), beside the device tensors."""

    def __init__(self, need: PagedNeed, stages: List[int], page_size: int):
        self.need = need
        self.stages = list(stages)
        self.page_size = page_size
        self.pool: Optional[PagePool] = None
        self.max_pages_per_request = 0
        self.table: Optional[np.ndarray] = None
        self.first_held: Optional[np.ndarray] = None
        self.num_logical: Optional[np.ndarray] = None
        self.kv = None                        # device tensor [stages, pages, 2, kv_heads, P, d] when keys and values are equally wide
        self.keys = None                      # [stages, pages, kv_heads, P, key width] (a view of `kv` when that exists)
        self.values = None                    # [stages, pages, kv_heads, P, value width]
        self.table_dev = None                 # device int32 [max_slots, max_pages_per_request]

    def _bind(self, lib, handle, index: int, max_slots: int, max_pages_per_request: int) -> None:
        self.max_pages_per_request = max_pages_per_request
        self.pool = PagePool(0, _borrowed=lib.hc_cache_pool(handle, index))
        view = lambda ptr, shape: np.ctypeslib.as_array(ptr, shape=shape)
        self.table = view(lib.hc_cache_table(handle, index), (max_slots, max_pages_per_request))
        self.first_held = view(lib.hc_cache_first_held(handle, index), (max_slots,))
        self.num_logical = view(lib.hc_cache_num_logical(handle, index), (max_slots,))

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def held_pages(self, slot: int) -> List[int]:
        return [int(p) for p in self.table[slot, self.first_held[slot]:self.num_logical[slot]]]


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
                    self.groups.append(CacheGroup(need, [], page_size))
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

        self._lib = host.lib()
        windows = _int32([-1 if g.need.window is None else g.need.window for g in self.groups])
        self._h = self._lib.hc_cache_new(len(self.groups), windows.ctypes.data, page_size, self.num_pages, max_slots,
                                         max_pages_per_request, self.max_request_tokens)
        if not self._h:
            raise CacheError(host.last_error())
        for i, g in enumerate(self.groups):
            g._bind(self._lib, self._h, i, max_slots, max_pages_per_request)
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
    def __del__(self):
        if getattr(self, "_h", None):
            for g in self.groups:                          # their views point into what is about to go
                g.table = g.first_held = g.num_logical = g.pool = None
            self._lib.hc_cache_delete(self._h)
            self._h = None

    @property
    def free_slots(self) -> int:
        return self._lib.hc_cache_free_slots(self._h)

    def admit(self) -> int:
        """Take a slot for a new request; its state tensors are zeroed."""
        slot = ctypes.c_int()
        _check(self._lib.hc_cache_admit(self._h, ctypes.byref(slot)))
        for t in self.state.values():
            t[slot.value].zero_()
        return slot.value

    def length(self, slot: int) -> int:
        out = ctypes.c_longlong()
        _check(self._lib.hc_cache_length(self._h, int(slot), ctypes.byref(out)))
        return out.value

    def release(self, slot: int) -> None:
        """The request is over (finished or preempted): every page and the slot go back."""
        _check(self._lib.hc_cache_release(self._h, int(slot)))

    # ---- pages -----------------------------------------------------------------------------
    def pages_missing(self, slot: int, new_len: int) -> List[int]:
        out = np.empty(len(self.groups), dtype=np.int32)
        _check(self._lib.hc_cache_pages_missing(self._h, int(slot), int(new_len), out.ctypes.data))
        return out.tolist()

    def can_hold(self, wants: Sequence[Tuple[Optional[int], int]]) -> bool:
        """Would `ensure` succeed for all of (slot or None for a request not yet admitted,
        new length) together?"""
        slots = _int32([-1 if s is None else s for s, _ in wants])
        lens = np.ascontiguousarray([n for _, n in wants], dtype=np.int64)
        yes = ctypes.c_int()
        _check(self._lib.hc_cache_can_hold(self._h, len(slots), slots.ctypes.data, lens.ctypes.data, ctypes.byref(yes)))
        return bool(yes.value)

    def reserve(self, need: Sequence[int], slot: Optional[int], new_len: int) -> Optional[List[int]]:
        """`need` (pages per group already promised in this step) plus what (slot or None, new
        length) wants, or None if that does not fit the free pages.  `can_hold` one request at a
        time, for callers that build a step up."""
        have = _int32(need)
        total = np.empty(len(self.groups), dtype=np.int32)
        fits = ctypes.c_int()
        _check(self._lib.hc_cache_reserve(self._h, have.ctypes.data, -1 if slot is None else int(slot), int(new_len),
                                          total.ctypes.data, ctypes.byref(fits)))
        return total.tolist() if fits.value else None

    def ensure(self, slot: int, new_len: int) -> None:
        """Make room for positions [0, new_len) of the request, in every group, or take nothing."""
        _check(self._lib.hc_cache_ensure(self._h, int(slot), int(new_len)))

    def commit(self, slot: int, new_len: int) -> int:
        """The step that filled positions up to new_len has been issued: record the length and
        give back pages that a window has passed.  Returns the number of pages given back."""
        given = ctypes.c_int()
        _check(self._lib.hc_cache_commit(self._h, int(slot), int(new_len), ctypes.byref(given)))
        return given.value

    # ---- a step's requests at once (what the step function calls) ---------------------------
    def lengths(self, slots: np.ndarray) -> np.ndarray:
        """int64 lengths of the requests in `slots` (int32)."""
        out = np.empty(len(slots), dtype=np.int64)
        _check(self._lib.hc_cache_lengths(self._h, len(slots), slots.ctypes.data, out.ctypes.data))
        return out

    def ensure_all(self, slots: np.ndarray, new_lens: np.ndarray) -> None:
        """`ensure` for every (slot, new length) of a step together, or take nothing."""
        _check(self._lib.hc_cache_ensure_all(self._h, len(slots), slots.ctypes.data, new_lens.ctypes.data))

    def commit_all(self, slots: np.ndarray, new_lens: np.ndarray) -> int:
        given = ctypes.c_int()
        _check(self._lib.hc_cache_commit_all(self._h, len(slots), slots.ctypes.data, new_lens.ctypes.data, ctypes.byref(given)))
        return given.value

    def drain_updates(self) -> List[Tuple[np.ndarray, np.ndarray]]:
        """Per group: (flat table indices, page ids) changed since the last call."""
        out = []
        for i in range(len(self.groups)):
            n = self._lib.hc_cache_pending(self._h, i)
            idx, val = np.empty(n, np.int32), np.empty(n, np.int32)
            if n:
                self._lib.hc_cache_drain(self._h, i, idx.ctypes.data, val.ctypes.data)
            out.append((idx, val))
        return out

    # ---- checks ----------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        _check(self._lib.hc_cache_check(self._h))
