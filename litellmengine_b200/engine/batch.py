"""One step's batch: what the host knows, packed once into a pinned buffer and copied to
fixed device arrays that every kernel of the step reads.

The reference builds fresh host vectors and device tensors for every call and only knows
two shapes of batch: one prompt from position 0, or B single tokens
(src/engine/paged_generate_engine.cpp:221-278,444-473).  Here a batch is any list of
(request, its next tokens): prompt portions at any past length beside single decoded tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


PREFILL_TILE_ROWS = 128         # query rows per tile of the tensor-core prefill attention kernel


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

    def __init__(self, token_cap: int, max_entries: int, num_groups: int, device):
        self.token_cap = token_cap
        self.max_updates = token_cap + 2 * max_entries + 8       # new pages a step can append, with slack
        T, B, U = token_cap, max_entries, self.max_updates
        off = 0
        self.off = {}
        for name, n in (("token_ids", T), ("positions", T), ("token_entry", T), ("entry_slot", B),
                        ("entry_q_start", B), ("entry_q_len", B), ("entry_kv_len", B), ("want_rows", T),
                        ("want_slot", T), ("decode_rows", T), ("prefill_tiles", 2 * (T // PREFILL_TILE_ROWS + B + 1)),
                        ("counts", 8 + num_groups)):
            self.off[name] = (off, n)
            off += n
        for g in range(num_groups):
            self.off[f"upd_index{g}"] = (off, U)
            off += U
            self.off[f"upd_value{g}"] = (off, U)
            off += U
        self.size = off
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

    def __init__(self, max_tokens: int, max_entries: int, num_groups: int, device):
        self.max_tokens, self.max_entries, self.num_groups = max_tokens, max_entries, num_groups
        self.device = torch.device(device)
        self.large = _Region(max_tokens, max_entries, num_groups, self.device)
        self.small = _Region(min(max_tokens, max_entries), max_entries, num_groups, self.device)
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
    decode_rows: torch.Tensor        # int32 [n_decode] rows of entries that bring a single token
    prefill_tiles: torch.Tensor      # int32 [n_tiles, 2] (entry, first row inside it) of entries that bring more
    status: torch.Tensor             # int32 [2]
    num_tokens: int
    num_entries: int
    num_want: int
    max_q_len: int
    max_kv_len: int
    num_decode: int = 0
    num_prefill_tiles: int = 0
    entries: List[StepEntry] = field(default_factory=list)
    feedback: Optional[torch.Tensor] = None   # int32 device buffer that negative token ids point into
    layout: str = "large"                     # which of StepBuffers' two layouts holds this step's arrays
    tables: dict = field(default_factory=dict)   # what parts compute once a step and share between layers


def pack_step(buffers: StepBuffers, entries: List[StepEntry], updates,
              feedback: Optional[torch.Tensor] = None) -> StepBatch:
    """Fill the pinned buffer from `entries` (whose `past` is set) and the cache manager's
    pending table `updates`, start the copy, and return the device views."""
    T = sum(len(e.tokens) for e in entries)
    B = len(entries)
    if T > buffers.max_tokens or B > buffers.max_entries:
        raise ValueError(f"a step of {T} tokens in {B} entries exceeds the limits "
                         f"({buffers.max_tokens} tokens, {buffers.max_entries} entries)")
    updates = list(updates)
    region = buffers.region_for(T, updates)
    buffers.last = region
    region.wait_reusable()
    hv = region.host_view
    tok, pos, ent = hv("token_ids"), hv("positions"), hv("token_entry")
    slot, qs, ql, kl = hv("entry_slot"), hv("entry_q_start"), hv("entry_q_len"), hv("entry_kv_len")
    wr, ws = hv("want_rows"), hv("want_slot")
    dec, tiles = hv("decode_rows"), hv("prefill_tiles")
    n_dec = n_tiles = 0
    row = w = 0
    max_q = max_kv = 0
    for i, e in enumerate(entries):
        n = len(e.tokens)
        tok[row:row + n] = np.asarray(e.tokens, dtype=np.int32)
        if e.feedback >= 0:
            tok[row + n - 1] = -1 - e.feedback
        pos[row:row + n] = np.arange(e.past, e.past + n, dtype=np.int32)
        ent[row:row + n] = i
        slot[i], qs[i], ql[i], kl[i] = e.slot, row, n, e.past + n
        for j in e.want:
            if not 0 <= j < n:
                raise ValueError(f"want={j} is outside the entry's {n} tokens")
            wr[w], ws[w] = row + j, e.slot
            w += 1
        if n == 1:
            dec[n_dec] = row
            n_dec += 1
        else:
            for q0 in range(0, n, PREFILL_TILE_ROWS):
                tiles[2 * n_tiles], tiles[2 * n_tiles + 1] = i, q0
                n_tiles += 1
        max_q, max_kv = max(max_q, n), max(max_kv, e.past + n)
        row += n
    counts = hv("counts")
    counts[0], counts[1], counts[2], counts[3], counts[4] = T, B, w, n_dec, n_tiles
    if n_tiles > 1:
        # longest first: a tile late in a long prompt walks the most keys, so it should start early
        tl = tiles[:2 * n_tiles].reshape(n_tiles, 2)
        cost = np.array([entries[int(e)].past + int(q0) for e, q0 in tl])
        tl[:] = tl[np.argsort(-cost, kind="stable")]
    for g, (idx, val) in enumerate(updates):
        if len(idx) > buffers.max_updates:
            raise ValueError("more block-table changes than the step buffer holds")
        hv(f"upd_index{g}")[:len(idx)] = idx
        hv(f"upd_value{g}")[:len(val)] = val
        counts[8 + g] = len(idx)
    region.upload()
    dv = region.dev_view
    return StepBatch(
        token_ids=dv("token_ids", T), positions=dv("positions", T), token_entry=dv("token_entry", T),
        entry_slot=dv("entry_slot", B), entry_q_start=dv("entry_q_start", B), entry_q_len=dv("entry_q_len", B),
        entry_kv_len=dv("entry_kv_len", B), want_rows=dv("want_rows", w), want_slot=dv("want_slot", w),
        decode_rows=dv("decode_rows", n_dec), prefill_tiles=dv("prefill_tiles", 2 * n_tiles).view(n_tiles, 2),
        num_decode=n_dec, num_prefill_tiles=n_tiles, status=buffers.status, num_tokens=T, num_entries=B, num_want=w, max_q_len=max_q, max_kv_len=max_kv,
        entries=entries, feedback=feedback, layout="small" if region is buffers.small else "large")
