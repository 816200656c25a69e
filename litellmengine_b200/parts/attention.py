"""The attention mixer: grouped-query causal attention over the paged cache."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from ..cache import PagedNeed
from ..config.specs import MixerSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .context import StageContext, StepPrelude
from .registry import lookup, register_mixer


class AttentionWork(StepPrelude):
    """How the attention kernels cut a step: rows of entries that bring one token go to the
    split-key decode kernel, longer portions are cut into tiles of `ops.PREFILL_TILE_ROWS` query
    rows (entry, first row inside it) for the tensor-core prompt kernel, longest walk first.
    Both lists are padded with -1 up to what a step of as many tokens could need at most, so that
    a launch over the whole padded list does the same work (a kernel's block that meets -1 returns
    at once): that is how a captured graph of a step of T tokens serves every later step of T
    tokens, however they are divided among requests."""
    name = "attention_work"

    @dataclass
    class Views:
        decode_rows: torch.Tensor        # int32 [num_decode] rows of entries that bring a single token
        prefill_tiles: torch.Tensor      # int32 [num_prefill_tiles, 2]
        num_decode: int
        num_prefill_tiles: int
        padded_rows: torch.Tensor        # the same lists over their padding: [rows_cap], [tiles_cap, 2]
        padded_tiles: torch.Tensor

    def sections(self, max_tokens: int, max_entries: int):
        self.max_entries = max_entries
        return {"decode_rows": max_tokens,
                "prefill_tiles": 2 * (max_tokens // ops.PREFILL_TILE_ROWS + max_entries + 1)}

    def caps(self, num_tokens: int):
        """The most rows and tiles a step of `num_tokens` tokens can have."""
        return (min(num_tokens, self.max_entries),
                num_tokens // ops.PREFILL_TILE_ROWS + min(num_tokens // 2, self.max_entries) + 1)

    def fill(self, facts, out):
        R = ops.PREFILL_TILE_ROWS
        single = facts.q_len == 1
        n_dec = int(single.sum())
        rows_cap, tiles_cap = self.caps(facts.num_tokens)
        tiles_cap = min(tiles_cap, len(out["prefill_tiles"]) // 2)
        out["decode_rows"][:n_dec] = facts.q_start[single]
        out["decode_rows"][n_dec:rows_cap] = -1
        n_tiles = 0
        if n_dec < len(facts.q_len):
            tiles = [(i, q0) for i in np.nonzero(~single)[0] for q0 in range(0, int(facts.q_len[i]), R)]
            # longest first: a tile late in a long prompt walks the most keys, so it should start early
            tiles.sort(key=lambda t: -(int(facts.past[t[0]]) + t[1]))
            n_tiles = len(tiles)
            out["prefill_tiles"][:2 * n_tiles] = np.asarray(tiles, dtype=np.int64).reshape(-1)
        out["prefill_tiles"][2 * n_tiles:2 * tiles_cap] = -1
        return n_dec, n_tiles, rows_cap, tiles_cap

    def views(self, dev, filled):
        n_dec, n_tiles, rows_cap, tiles_cap = filled
        return AttentionWork.Views(dev["decode_rows"][:n_dec], dev["prefill_tiles"][:2 * n_tiles].view(n_tiles, 2),
                                   n_dec, n_tiles, dev["decode_rows"][:rows_cap],
                                   dev["prefill_tiles"][:2 * tiles_cap].view(tiles_cap, 2))


@register_mixer("attention")
class AttentionMixer:
    """q/k/v projections without bias fused into one product, per-head RMSNorm of q and k,
    rotation, cache write, attention over the pages, output projection
    (src/model/qwen3.cpp:357-449,464-481,550-567).  kv head of query head h is h // (heads /
    kv_heads); scores are scaled by 1/sqrt(head_dim) unless the spec gives a scale
    (src/ops/attention.cu:204-207)."""

    graph_safe = True          # forward only launches kernels on the current stream
    any_division_safe = True   # and nothing in it is shaped by the number of entries of the step

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError("attention heads must be a positive multiple of kv heads")
        if spec.head_dim <= 0 or spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim}: the attention kernels take multiples of 16 up to 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec = spec
        self.hidden = hidden_size
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.d))
        self.dtype = compute_dtype
        self.device = torch.device(device)
        self.position = lookup("position", spec.position.kind)(spec.position, self.d, device)
        self.q_norm = self.k_norm = None
        if spec.qk_norm is not None:
            cls = lookup("norm", spec.qk_norm.kind)
            self.q_norm = cls(spec.qk_norm, self.d)
            self.k_norm = cls(spec.qk_norm, self.d) if spec.has_kv else None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        p = {"q_proj.weight": ParamSpec((self.nq * self.d, self.hidden)),
             "o_proj.weight": ParamSpec((self.hidden, self.nq * self.d))}
        if self.spec.has_kv:
            p["k_proj.weight"] = ParamSpec((self.nkv * self.d, self.hidden))
            p["v_proj.weight"] = ParamSpec((self.nkv * self.d, self.hidden))
        if self.q_norm is not None:
            p["q_norm.weight"] = self.q_norm.parameters()["weight"]
        if self.k_norm is not None:
            p["k_norm.weight"] = self.k_norm.parameters()["weight"]
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t["q_proj.weight"]]
        if self.spec.has_kv:
            parts += [t["k_proj.weight"], t["v_proj.weight"]]
        # Row concatenation, so one product yields [q | k | v] per token.  A float32 member
        # keeps the fused matrix in float32.
        dt = torch.float32 if any(x.dtype == torch.float32 for x in parts) else parts[0].dtype
        self.w_qkv = torch.cat([x.to(dt) for x in parts], dim=0).contiguous()
        self.w_o = t["o_proj.weight"].contiguous()
        ops.prepare_streaming(self.w_qkv)           # a tiled copy for decode steps (bfloat16 on a GPU only)
        ops.prepare_streaming(self.w_o)
        if self.q_norm is not None:
            self.q_norm.load({"weight": t["q_norm.weight"]})
        if self.k_norm is not None:
            self.k_norm.load({"weight": t["k_norm.weight"]})

    def cache_need(self):
        if not self.spec.has_kv:
            return None
        return PagedNeed(self.nkv, self.d, self.spec.window)

    def step_prelude(self):
        return AttentionWork()

    @property
    def graph_variant_group(self):
        return ("attention", self.nkv)

    def graph_variant(self, batch, padded: bool) -> int:
        """The decode kernel's key splits: the one launch choice here that depends on lengths."""
        work = batch.preludes.get(AttentionWork.name)
        if work is None:
            return 0
        n_dec = work.padded_rows.shape[0] if padded else work.num_decode
        return decode_key_splits(self.device, n_dec, self.nkv, batch.max_kv_len) if n_dec else 0

    def forward(self, x: torch.Tensor, ctx: StageContext) -> torch.Tensor:
        b = ctx.batch
        qkv = ops.linear(x, self.w_qkv, out_dtype=torch.float32, partials_ok=True)   # normalised, rotated in 32-bit
        has_kv = self.spec.has_kv and ctx.writes_cache
        if self.spec.has_kv and not ctx.writes_cache:
            raise RuntimeError("a mixer with its own keys and values was given a borrowed cache")
        eps = self.spec.qk_norm.eps if self.spec.qk_norm is not None else 0.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        cache, table = (ctx.cache, ctx.block_table) if has_kv else (None, None)
        if hasattr(self.position, "rotation"):
            # a rotation (or nothing): norms, rotation and cache write in one kernel
            rot = self.position.rotation(b)
            q = ops.qk_norm_rope_kv_write(
                qkv, cache, b.positions, b.token_entry, b.entry_slot, table, qw, kw, eps,
                rot.inv_freq if rot is not None else None, rot.rotary_dim if rot is not None else 0,
                self.nq, self.nkv, self.d, ctx.page_size, has_kv, ctx.status, q_dtype=self.dtype,
                angles=rot.angles if rot is not None else None)
        else:
            # an encoding of the part's own: norms, then the part, then the cache write
            q32, k32 = ops.qk_head_norm(qkv, qw, kw, eps, self.nq, self.nkv, self.d, has_kv)
            T = q32.shape[0]
            q32, k32 = self.position.apply(q32.view(T, self.nq, self.d),
                                           k32.view(T, self.nkv, self.d) if k32 is not None else None, b)
            q = ops.qk_store(q32.reshape(T, self.nq * self.d).contiguous(),
                             k32.reshape(T, self.nkv * self.d).contiguous() if k32 is not None else None, qkv, cache,
                             b.positions, b.token_entry, b.entry_slot, table, self.nq, self.nkv, self.d,
                             ctx.page_size, has_kv, ctx.status, self.dtype)
        a = attention_over_pages(q, ctx, self.nq, self.nkv, self.d, self.spec.window, self.scale)
        # joins the float32 residual; may stay a sum of k-splits if the layer's norm adds them itself
        residual = getattr(ctx, "residual", None)
        if residual is not None and ops.linear_into(a, self.w_o, residual):
            return None                                           # added to the residual in the product's epilogue
        return ops.linear(a, self.w_o, out_dtype=torch.float32, partials_ok=getattr(ctx, "partials_ok", False))


_slots = {}


def _cta_slots(device) -> int:
    n = _slots.get(device)
    if n is None:
        n = _slots[device] = 2 * torch.cuda.get_device_properties(device).multi_processor_count
    return n


# Key splits of the decode kernel by the longest cached length, in steps: a captured graph holds its
# number of splits, so steps whose lengths give the same number share a graph.
_SPLIT_STEPS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64)


def decode_key_splits(device, n_dec: int, nkv: int, max_kv_len: int) -> int:
    """Two rules, measured.  (1) A split costs its launch and its share of the merge, a key costs its
    bytes: for a few rows the best number grows as the square root of the length (one row: 8, 12,
    16, 24 splits at 1,024, 2,304, 4,096, 16,384 keys), at least 64 keys a split.  (2) The grid runs in
    waves of two CTAs per SM: below that ceiling take the fewest splits that fill at least 0.85 of the
    waves they start, else the fullest (at 4,096 keys 20 rows: 5 splits, 40 rows: 4, 48 rows: 2,
    where one split took a quarter longer; 8, 16, 32, 64 rows stay at 4, 2, 1, 1; at 384 keys 48 rows
    stay at one split: 1.71 ms a step on the 0.6B shape against 1.79 with two)."""
    by_length = max(1, min(math.ceil(math.sqrt(max_kv_len / 16.0)), -(-max_kv_len // 64)))
    most = max(s for s in _SPLIT_STEPS if s <= by_length)
    if n_dec * nkv > _cta_slots(device):             # more CTAs than slots already: a split only evens out the waves,
        most = max(1, min(most, max_kv_len // 512))  # which pays for its merge kernel from about 512 keys a split
    key = (device, n_dec * nkv, most)
    got = _split_choice.get(key)
    if got is None:
        slots, ctas = _cta_slots(device), max(1, n_dec * nkv)
        fill = lambda s: ctas * s / (-(-ctas * s // slots) * slots)
        enough = [s for s in range(1, most + 1) if fill(s) >= 0.85]
        got = _split_choice[key] = enough[0] if enough else max(range(1, most + 1), key=lambda s: (fill(s), -s))
    return got


_split_choice: Dict[tuple, int] = {}


def attention_over_pages(q: torch.Tensor, ctx: StageContext, nq: int, nkv: int, d: int,
                         window: Optional[int], scale: float) -> torch.Tensor:
    """Pick the attention kernels for this batch.  Every choice reads the same pages and gives
    the same result up to rounding.  bfloat16 with a head size and group the tuned kernels
    take: single tokens go to the split-key decode kernel, longer portions to the tensor-core
    prefill kernel (a mixed batch launches both, each over its own rows).  Everything else,
    float32 included, goes through the generic kernel."""
    b = ctx.batch
    cache = ctx.cache
    work = b.preludes.get(AttentionWork.name)
    if (work is not None and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
            and ops.fast_attention_supported(d, nq // nkv)):
        out = torch.empty_like(q)
        # A step that is being captured as a graph of "any step of this many tokens" launches both
        # kernels over the padded lists; otherwise over what this step has.
        padded = getattr(b, "any_division", False)
        n_dec = work.padded_rows.shape[0] if padded else work.num_decode
        n_tiles = work.padded_tiles.shape[0] if padded else work.num_prefill_tiles
        if n_dec:
            splits = decode_key_splits(q.device, n_dec, nkv, b.max_kv_len)
            rows = work.padded_rows if padded else (None if n_dec == b.num_tokens else work.decode_rows)
            ops.paged_attention_decode(q, out, cache, rows, n_dec, b.positions, b.token_entry, b.entry_slot,
                                       ctx.block_table, nq, nkv, d, ctx.page_size, window, scale, splits, ctx.status)
        if n_tiles:
            kernel = (ops.paged_attention_prefill_tcgen05
                      if ops.prefill_tcgen05_supported(d, ctx.page_size)
                      else ops.paged_attention_prefill)       # tcgen05/TMEM/TMA where it applies, mma.sync otherwise
            kernel(q, out, cache, work.padded_tiles if padded else work.prefill_tiles, n_tiles, b.entry_slot,
                   b.entry_q_start, b.entry_q_len, b.entry_kv_len, ctx.block_table, nq, nkv, d, ctx.page_size, window,
                   scale, ctx.status)
        return out
    return ops.paged_attention_generic(q, cache, b.positions, b.token_entry, b.entry_slot,
                                       ctx.block_table, nq, nkv, d, ctx.page_size, window, scale, ctx.status)
