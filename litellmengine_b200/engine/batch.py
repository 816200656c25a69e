"""One step's batch: what the host knows, packed once into a pinned buffer and copied to
fixed device arrays that every kernel of the step reads.

The reference builds fresh host vectors and device tensors for every call and only knows
two shapes of batch: one prompt from position 0, or B single tokens
(src/engine/paged_generate_engine.cpp:221-278,444-473).  Here a batch is any list of
(request, its next tokens): prompt portions at any past length beside single decoded tokens.

The batch itself carries only facts about entries and tokens.  Work lists that one kind of
kernel wants (which rows go to which kernel, tiles, sorted orders) belong to the part that
launches that kernel: it offers a `StepPrelude`, which is given room in the same pinned
buffer, fills it from the entries once per step, and finds its device views in
`batch.preludes[name]` in every layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..csrc import host
from ..parts.context import StepFacts, StepPrelude

# the sections the native packing writes, in the order it takes their offsets
_PACKED = ("token_ids", "positions", "token_entry", "entry_slot", "entry_q_start", "entry_q_len", "entry_kv_len",
           "want_rows", "want_slot", "counts")


@dataclass
class StepEntry:
    """One request's share of a step: its slot, the tokens to run now (they follow what the
    cache already holds for it), and the places among them whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    past: int = 0                     # filled in by the step function: tokens already cached
    feedback: int = -1                # >= 0: the LAST token is not known to the host yet; it is entry
                                      # `feedback` of the tokens the previous step sampled on the device


class _Region:
    """One layout of the step's arrays: a pinned staging buffer and its fixed device twin."""

    def __init__(self, token_cap: int, max_entries: int, num_groups: int, device, preludes: Sequence[StepPrelude]):
        self.token_cap = token_cap
        self.max_updates = token_cap + 2 * max_entries + 8       # new pages a step can append, with slack
        T, B, U = token_cap, max_entries, self.max_updates
        off = 0
        self.off = {}
        sections = [("token_ids", T), ("positions", T), ("token_entry", T), ("entry_slot", B),
                    ("entry_q_start", B), ("entry_q_len", B), ("entry_kv_len", B), ("want_rows", T),
                    ("want_slot", T), ("counts", 8 + num_groups), ("state_index", 8 * B), ("state_value", 8 * B)]
        for p in preludes:
            sections += [(f"{p.name}:{k}", int(n)) for k, n in p.sections(T, B).items()]
        self.prelude_keys = {p.name: list(p.sections(T, B)) for p in preludes}
        for g in range(num_groups):
            sections += [(f"upd_index{g}", U), (f"upd_value{g}", U)]
        for name, n in sections:
            self.off[name] = (off, n)
            off += n
        self.size = off
        self.packed_offsets = np.asarray([self.off[name][0] for name in _PACKED], dtype=np.int64)
        self.pinned = torch.zeros(off, dtype=torch.int32, pin_memory=True)
        self.host = self.pinned.numpy()
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event()
        self._in_flight = False

    def host_view(self, name: str) -> np.ndarray:
        o, n = self.off[name]
        return self.host[o:o + n]

    def dev_view(self, name: str, count: Optional[int] = None) -> torch.Tensor:
        o, n = self.off[name]
        return self.dev[o:o + (n if count is None else count)]

    def wait_reusable(self) -> None:
        if self._in_flight:
            self.copied.synchronize()
            self._in_flight = False

    def upload(self) -> None:
        self.dev.copy_(self.pinned, non_blocking=True)
        self.copied.record()
        self._in_flight = True


class StepBuffers:
    """Pinned staging and device arrays sized once: a large layout for the largest step and a
    small one for steps of at most `max_entries` tokens (decode steps), so that those copy a few
    kilobytes to the device instead of the large layout's hundred and more.  A step lives in one
    of the two; device addresses inside each are fixed, which is what a captured graph needs."""

    def __init__(self, max_tokens: int, max_entries: int, num_groups: int, device,
                 preludes: Sequence[StepPrelude] = ()):
        self.max_tokens, self.max_entries, self.num_groups = max_tokens, max_entries, num_groups
        self.device = torch.device(device)
        self.preludes: List[StepPrelude] = []
        for p in preludes:                                        # one per name, first come
            if all(p.name != q.name for q in self.preludes):
                self.preludes.append(p)
        self.large = _Region(max_tokens, max_entries, num_groups, self.device, self.preludes)
        self.small = _Region(min(max_tokens, max_entries), max_entries, num_groups, self.device, self.preludes)
        self.max_updates = self.large.max_updates
        self.status = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.last = self.large                                    # the region of the step packed last

    def host_view(self, name: str) -> np.ndarray:
        """Of the step packed last."""
        return self.last.host_view(name)

    def dev_view(self, name: str, count: Optional[int] = None) -> torch.Tensor:
        return self.last.dev_view(name, count)

    def region_for(self, num_tokens: int, updates) -> _Region:
        small = self.small
        if num_tokens <= small.token_cap and all(len(idx) <= small.max_updates for idx, _ in updates):
            return small
        return self.large


@dataclass
class StepBatch:
    """Device views of one step (exact lengths) plus the host-side facts kernels are chosen by."""
    token_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T] absolute position of each token in its request
    token_entry: torch.Tensor        # int32 [T] index of the token's entry
    entry_slot: torch.Tensor         # int32 [B]
    entry_q_start: torch.Tensor      # int32 [B] first row of the entry in the batch
    entry_q_len: torch.Tensor        # int32 [B]
    entry_kv_len: torch.Tensor       # int32 [B] cached length after this step
    want_rows: torch.Tensor          # int32 [W] rows whose logits are wanted
    want_slot: torch.Tensor          # int32 [W] slot of each wanted row
    status: torch.Tensor             # int32 [2]
    num_tokens: int
    num_entries: int
    num_want: int
    max_q_len: int
    max_kv_len: int
    entries: List[StepEntry] = field(default_factory=list)
    feedback: Optional[torch.Tensor] = None   # int32 device buffer that negative token ids point into
    layout: str = "large"                     # which of StepBuffers' two layouts holds this step's arrays
    preludes: Dict[str, object] = field(default_factory=dict)   # the parts' `StepPrelude` views by name
    # True while the step is captured as a graph that must serve ANY step of as many tokens: kernels
    # whose work depends on how the tokens are divided among requests launch over their preludes'
    # padded lists, and the wanted rows are `want_rows` padded to `want_cap` entries
    any_division: bool = False
    want_cap: int = 0
    state_ranges: List[tuple] = field(default_factory=list)     # (offset, count) of each state write in the buffer
    # what a part computes on the device in the first layer that needs it and shares with the layers
    # after it (emptied before a step is captured as a graph, so that the graph holds the kernel)
    tables: Dict[object, object] = field(default_factory=dict)
    entry_slots: Optional[np.ndarray] = None                    # host copies for the cache manager: int32 [B] slots,
    entry_new_len: Optional[np.ndarray] = None                  # int64 [B] each request's length after this step


@dataclass
class EntryArrays:
    """A step's entries as arrays, made once: what the checks, the cache manager and the packing read."""
    q_len: np.ndarray                # int64 [B] tokens each entry brings
    slot: np.ndarray                 # int32 [B]
    fed: np.ndarray                  # int32 [B] `StepEntry.feedback`
    tokens: np.ndarray               # int64 [T] all entries' tokens, joined
    want: np.ndarray                 # int64 all entries' wanted places, joined
    want_count: np.ndarray           # int32 [B]
    past: Optional[np.ndarray] = None    # int64 [B], when the cache manager has been asked

    @staticmethod
    def of(entries: Sequence[StepEntry]) -> "EntryArrays":
        B = len(entries)
        q_len = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        if int(q_len.sum()) == B:                                 # single tokens only: no lists to join
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=B)
        elif B:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        else:
            tokens = np.empty(0, np.int64)
        want_count = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=B)
        return EntryArrays(
            q_len=q_len, slot=np.fromiter((e.slot for e in entries), dtype=np.int32, count=B),
            fed=np.fromiter((e.feedback for e in entries), dtype=np.int32, count=B), tokens=tokens,
            want=np.fromiter((j for e in entries for j in e.want), dtype=np.int64, count=int(want_count.sum())),
            want_count=want_count)


def pack_step(buffers: StepBuffers, entries: List[StepEntry], updates,
              feedback: Optional[torch.Tensor] = None, state_writes=(), arrays: Optional[EntryArrays] = None) -> StepBatch:
    """Fill the pinned buffer from `entries` (whose `past` is set) and the cache manager's
    pending table `updates`, let every prelude fill its share, start the copy, and return the
    device views.  `state_writes`: [(flat indices, int32 values)] to be written into per-request
    state tensors by the step function after the copy (they ride in the same buffer; at most
    8 values per entry in all); their places in the buffer come back in `batch.state_ranges`."""
    B = len(entries)
    a = arrays if arrays is not None else EntryArrays.of(entries)
    q_len, slot, fed, tokens, want, want_count = a.q_len, a.slot, a.fed, a.tokens, a.want, a.want_count
    past = a.past if a.past is not None else np.fromiter((e.past for e in entries), dtype=np.int64, count=B)
    T = int(q_len.sum())
    if T > buffers.max_tokens or B > buffers.max_entries:
        raise ValueError(f"a step of {T} tokens in {B} entries exceeds the limits "
                         f"({buffers.max_tokens} tokens, {buffers.max_entries} entries)")
    updates = list(updates)
    region = buffers.region_for(T, updates)
    buffers.last = region
    region.wait_reusable()
    hv = region.host_view
    want_cap = min(buffers.max_entries, region.token_cap)
    if len(want) > region.token_cap:
        raise ValueError(f"{len(want)} wanted rows in a step of {T} tokens")
    facts4 = np.empty(4, dtype=np.int64)
    # token ids, positions, entries, wanted rows (padded to `want_cap` for a graph that reads that many), counts
    if host.lib().hc_pack_step(region.host.ctypes.data, region.packed_offsets.ctypes.data, B, slot.ctypes.data, past.ctypes.data,
                               q_len.ctypes.data, fed.ctypes.data, tokens.ctypes.data, want.ctypes.data,
                               want_count.ctypes.data, want_cap, facts4.ctypes.data):
        raise ValueError(host.last_error())
    w, max_q_len, max_kv_len = int(facts4[1]), int(facts4[2]), int(facts4[3])
    q_start = np.cumsum(q_len) - q_len
    counts = hv("counts")
    facts = StepFacts(q_start=q_start, q_len=q_len, past=past, slot=slot, num_tokens=T)
    filled = [(p, p.fill(facts, {k: hv(f"{p.name}:{k}") for k in region.prelude_keys[p.name]}))
              for p in buffers.preludes]
    for g, (idx, val) in enumerate(updates):
        if len(idx) > buffers.max_updates:
            raise ValueError("more block-table changes than the step buffer holds")
        hv(f"upd_index{g}")[:len(idx)] = idx
        hv(f"upd_value{g}")[:len(val)] = val
        counts[8 + g] = len(idx)
    at, ranges = 0, []
    for idx, val in state_writes:
        n = len(idx)
        if at + n > 8 * buffers.max_entries:
            raise ValueError("more per-request state values than the step buffer holds")
        hv("state_index")[at:at + n] = idx
        hv("state_value")[at:at + n] = val
        ranges.append((at, n))
        at += n
    region.upload()
    dv = region.dev_view
    batch = StepBatch(
        token_ids=dv("token_ids", T), positions=dv("positions", T), token_entry=dv("token_entry", T),
        entry_slot=dv("entry_slot", B), entry_q_start=dv("entry_q_start", B), entry_q_len=dv("entry_q_len", B),
        entry_kv_len=dv("entry_kv_len", B), want_rows=dv("want_rows", w), want_slot=dv("want_slot", w),
        status=buffers.status, num_tokens=T, num_entries=B, num_want=w, max_q_len=max_q_len,
        max_kv_len=max_kv_len, entries=entries, feedback=feedback,
        layout="small" if region is buffers.small else "large", want_cap=want_cap)
    batch.state_ranges = ranges
    batch.entry_slots, batch.entry_new_len = slot, past + q_len
    for p, got in filled:
        batch.preludes[p.name] = p.views({k: dv(f"{p.name}:{k}") for k in region.prelude_keys[p.name]}, got)
    return batch
