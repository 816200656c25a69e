"""Python faces of the CUDA kernels: argument checks, then one ctypes call per launch.

Every function takes CUDA tensors, launches on torch's current stream, allocates only its
result (or writes into `out`), and raises if the kernel refuses the sizes.  There is no CPU
or library fallback here: a tensor that is not on a CUDA device is an error, and a missing
compiler or library surfaces as `BuildError`.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_int32, c_longlong, c_uint32, c_uint64, c_void_p
from typing import Dict, Optional

import torch

from . import build

_libs: Dict[str, ctypes.CDLL] = {}

_REFUSALS = {
    -1: "a size this kernel does not take",
    -2: "a dtype combination this kernel is not built for",
    -3: "a pointer or stride that is not 16-byte aligned",
}


class KernelError(RuntimeError):
    pass


def lib(family: str) -> ctypes.CDLL:
    l = _libs.get(family)
    if l is None:
        l = ctypes.CDLL(build.ensure_built(family))
        _libs[family] = l
    return l


def loaded_libraries():
    return {k: v._name for k, v in _libs.items()}


def _fn(family: str, name: str, argtypes, restype=c_int):
    f = getattr(lib(family), name)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = restype
    return f


class PartialSum:
    """A product left as its k-splits: float32 [splits, rows, cols] whose sum over the first axis
    is the result.  The engine's norm and q/k kernels add the splits while they read, which
    saves a kernel per product in decode steps; `as_tensor` adds them for anyone else."""

    def __init__(self, parts: torch.Tensor, rounds_to: Optional[torch.dtype] = None):
        self.parts = parts
        self.rounds_to = rounds_to      # the product's own dtype when it is not float32: the sum is rounded to it

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def dtype(self):
        return self.parts.dtype


def as_tensor(x):
    if not isinstance(x, PartialSum):
        return x
    total = x.parts.sum(dim=0)
    return total.to(x.rounds_to) if x.rounds_to is not None else total


launch_count = 0          # launches of the engine's own kernels since import (library products are not counted)


def _check(code: int, what: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_REFUSALS.get(code, f'code {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not float32 or bfloat16")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("tensor is not on a CUDA device; the engine has no CPU path")
        if not t.is_contiguous():
            raise KernelError("tensor is not contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_bound_stream: Optional[int] = None


def _stream() -> int:
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """Inside this scope every launch goes to the stream that was current at its entry, looked up
    once (asking for the current stream costs as much as three launches).  For code that does not
    switch streams while it runs: a model's forward pass."""

    def __enter__(self):
        global _bound_stream
        self._prev = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._prev
        return False


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")


# ------------------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor,
              out: Optional[torch.Tensor] = None, feedback: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [T, H] = table[ids]; an id -1-j takes its token from feedback[j] (int32, on the device)."""
    _dev(ids, table, status, out, feedback)
    _i32(ids, "ids")
    if feedback is not None:
        _i32(feedback, "feedback")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn("embedding", "llm_embedding_gather",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _dt(table), _ptr(out), T, H, V, _ptr(status), _ptr(feedback),
             feedback.numel() if feedback is not None else 0, _stream()), "embedding")
    return out


def scatter_int32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor, count: torch.Tensor,
                  max_count: int, status: torch.Tensor) -> None:
    """dst.flat[index[i]] = value[i] for i < count[0] (count is a device scalar; None: for i < max_count)."""
    _dev(dst, index, value, count, status)
    for t, n in ((dst, "dst"), (index, "index"), (value, "value"), (count, "count")):
        _i32(t, n)
    f = _fn("embedding", "llm_scatter_int32",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(dst), dst.numel(), _ptr(index), _ptr(value), _ptr(count), max_count, _ptr(status), _stream()),
           "scatter_int32")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            write_sum: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x (+ delta)) * weight over the last dim; with `write_sum`, x += delta in place.
    `rows` (int32) selects which rows are normalised (out has len(rows) rows)."""
    parts, part_stride = 1, 0
    if isinstance(delta, PartialSum):
        parts, part_stride = delta.parts.shape[0], delta.parts.stride(0)
        delta = delta.parts[0]
    _dev(x, weight, delta, rows, out)
    _i32(rows, "rows")
    H = x.shape[-1]
    if weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("norm weight must be float32 of the row length")
    if delta is not None and delta.shape != x.shape:
        raise KernelError("delta must have x's shape")
    n = rows.numel() if rows is not None else x.numel() // H
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    f = _fn("norm", "llm_rmsnorm",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
             c_int, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), _dt(x), _ptr(delta), _dt(delta) if delta is not None else 0, _ptr(weight), _ptr(out),
             _dt(out), _ptr(rows), n, H, float(eps), 1 if write_sum else 0, parts, part_stride, _stream()), "rmsnorm")
    return out


def silu_and_mul(gate_up, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, 2I] -> [T, I]: silu(first half) * second half.  A `PartialSum` is added up on the way."""
    if isinstance(gate_up, PartialSum):
        parts = gate_up.parts
        _dev(parts, out)
        S, T, two_i = parts.shape
        if out is None:
            out = torch.empty((T, two_i // 2), dtype=gate_up.rounds_to or torch.float32, device=parts.device)
        f = _fn("activation", "llm_silu_and_mul_parts", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(f(_ptr(parts), S, _ptr(out), _dt(out), T, two_i // 2, _stream()), "silu_and_mul")
        return out
    _dev(gate_up, out)
    T, two_i = gate_up.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("activation", "llm_silu_and_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _dt(gate_up), T, inter, _stream()), "silu_and_mul")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h (float32) += delta, in place."""
    delta = as_tensor(delta)
    _dev(h, delta)
    if h.dtype != torch.float32 or h.shape != delta.shape:
        raise KernelError("residual_add wants a float32 residual and a delta of its shape")
    f = _fn("activation", "llm_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(h), _ptr(delta), _dt(delta), h.numel(), _stream()), "residual_add")
    return h


def qk_norm_rope_kv_write(qkv: torch.Tensor, cache: Optional[torch.Tensor], positions, token_entry, entry_slot,
                          block_table: Optional[torch.Tensor], q_norm_w, k_norm_w, eps: float, inv_freq,
                          rotary_dim: int, nq: int, nkv: int, d: int, page_size: int, has_kv: bool,
                          status: torch.Tensor, q_out: Optional[torch.Tensor] = None,
                          q_dtype: Optional[torch.dtype] = None, angles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalise and rotate q and k, write k and v into the cache pages, return q [T, nq*d]
    in `q_dtype` (default: qkv's).
    cache: [num_pages, 2, nkv, page_size, d] of one stage (None with has_kv False).
    angles: the step's table from `rope_angles`, which saves every layer the sines and cosines."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(qkv, cache, positions, token_entry, entry_slot, block_table, q_norm_w, k_norm_w, inv_freq, status, q_out)
    for t, n in ((positions, "positions"), (token_entry, "token_entry"), (entry_slot, "entry_slot"),
                 (block_table, "block_table")):
        _i32(t, n)
    T = qkv.shape[0]
    heads_total = nq + (2 * nkv if has_kv else 0)
    if qkv.shape[1] != heads_total * d:
        raise KernelError(f"qkv row is {qkv.shape[1]}, expected {heads_total * d}")
    if has_kv:
        if cache is None or block_table is None or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
            raise KernelError("cache must be [pages, 2, kv_heads, page_size, head_dim]")
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d):
            raise KernelError("q/k norm weight must be float32 [head_dim]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim):
        raise KernelError("inv_freq must be float32 [rotary_dim/2]")
    if angles is not None and (inv_freq is None or angles.dtype != torch.float32 or not angles.is_contiguous()
                               or tuple(angles.shape) != (T, inv_freq.numel(), 2)):
        raise KernelError("angles must be float32 [T, rotary_dim/2, 2] from rope_angles")
    if q_out is None:
        q_out = torch.empty((T, nq * d), dtype=q_dtype or qkv.dtype, device=qkv.device)
    f = _fn("rope_cache", "llm_qk_norm_rope_kv_write",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), _ptr(q_out), _dt(q_out), _ptr(cache),
             _dt(cache) if cache is not None else _dt(q_out),
             _ptr(positions), _ptr(token_entry), _ptr(entry_slot), _ptr(block_table),
             block_table.shape[1] if block_table is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
             _ptr(inv_freq), rotary_dim if inv_freq is not None else 0, T, nq, nkv, d, page_size,
             1 if has_kv else 0, cache.shape[0] if cache is not None else 0, _ptr(status), parts, part_stride,
             _ptr(angles), _stream()),
           "qk_norm_rope_kv_write")
    return q_out


def qk_head_norm(qkv, q_norm_w, k_norm_w, eps: float, nq: int, nkv: int, d: int, has_kv: bool):
    """The first half of `qk_norm_rope_kv_write` alone: the per-head norms of q and k (a null weight:
    no norm), nothing rotated, nothing written to the cache.  Returns float32 q [T, nq*d] and k
    [T, nkv*d] (None without keys), for a position part that encodes them itself."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(qkv, q_norm_w, k_norm_w)
    T = qkv.shape[0]
    if qkv.shape[1] != (nq + (2 * nkv if has_kv else 0)) * d:
        raise KernelError(f"qkv row is {qkv.shape[1]}, expected {(nq + (2 * nkv if has_kv else 0)) * d}")
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d):
            raise KernelError("q/k norm weight must be float32 [head_dim]")
    q = torch.empty((T, nq * d), dtype=torch.float32, device=qkv.device)
    k = torch.empty((T, nkv * d), dtype=torch.float32, device=qkv.device) if has_kv else None
    f = _fn("rope_cache", "llm_qk_head_norm",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
             c_longlong, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), _ptr(q), _ptr(k), _ptr(q_norm_w), _ptr(k_norm_w), float(eps), T, nq, nkv, d,
             1 if has_kv else 0, parts, part_stride, _stream()), "qk_head_norm")
    return q, k


def qk_store(q: torch.Tensor, k: Optional[torch.Tensor], qkv, cache: Optional[torch.Tensor], positions, token_entry,
             entry_slot, block_table: Optional[torch.Tensor], nq: int, nkv: int, d: int, page_size: int, has_kv: bool,
             status: torch.Tensor, q_dtype: torch.dtype) -> torch.Tensor:
    """The second half: q (float32, encoded by the position part) rounded to `q_dtype`; k (float32,
    encoded) and the v columns of `qkv` written into the pages of `cache`."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(q, k, qkv, cache, positions, token_entry, entry_slot, block_table, status)
    T = qkv.shape[0]
    if q.dtype != torch.float32 or tuple(q.shape) != (T, nq * d) or (has_kv and (
            k is None or k.dtype != torch.float32 or tuple(k.shape) != (T, nkv * d))):
        raise KernelError("q and k must be float32 [T, heads * head_dim]")
    if has_kv and (cache is None or block_table is None or tuple(cache.shape[1:]) != (2, nkv, page_size, d)):
        raise KernelError("cache must be [pages, 2, kv_heads, page_size, head_dim]")
    q_out = torch.empty((T, nq * d), dtype=q_dtype, device=q.device)
    f = _fn("rope_cache", "llm_qk_store",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(q), _ptr(k), _ptr(qkv), _dt(qkv), _ptr(q_out), _dt(q_out), _ptr(cache),
             _dt(cache) if cache is not None else _dt(q_out), _ptr(positions), _ptr(token_entry), _ptr(entry_slot),
             _ptr(block_table), block_table.shape[1] if block_table is not None else 0, T, nq, nkv, d, page_size,
             1 if has_kv else 0, cache.shape[0] if cache is not None else 0, _ptr(status), parts, part_stride,
             _stream()), "qk_store")
    return q_out


ROPE_TABLE_MIN_TOKENS = 64     # steps of fewer tokens compute their angles inside the kernel, before it waits


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(sin, cos) of float32(position) * inv_freq for every token of a step: float32 [T, rotary_dim/2, 2],
    computed once for all layers (a prompt portion's rotation kernel is bound by its instructions, and
    most of them are these)."""
    _dev(positions, inv_freq)
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    out = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    f = _fn("rope_cache", "llm_rope_angles", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_angles")
    return out


def paged_attention_generic(q: torch.Tensor, cache: torch.Tensor, positions, token_entry, entry_slot,
                            block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                            window: Optional[int], scale: float, status: torch.Tensor,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token in q [T, nq*d] over its request's pages."""
    _dev(q, cache, positions, token_entry, entry_slot, block_table, status, out)
    for t, n in ((positions, "positions"), (token_entry, "token_entry"), (entry_slot, "entry_slot"),
                 (block_table, "block_table")):
        _i32(t, n)
    T = q.shape[0]
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    if out is None:
        out = torch.empty_like(q)
    f = _fn("attention_generic", "llm_paged_attention_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _dt(q), _ptr(cache), _dt(cache), _ptr(positions), _ptr(token_entry),
             _ptr(entry_slot), _ptr(block_table), block_table.shape[1], T, nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_generic")
    return out


def fast_attention_supported(d: int, group: int) -> bool:
    """Whether the tuned bfloat16 kernels (tensor-core prefill, split-key decode) take this shape."""
    if d % 64 != 0:          # they are written for head sizes 64 and 128: do not compile them just to hear "no"
        return False
    a = _fn("attention_decode", "llm_paged_decode_supported", [c_int, c_int])
    b = _fn("attention_prefill", "llm_paged_prefill_supported", [c_int])
    return bool(a(d, group)) and bool(b(d))


PREFILL_TILE_ROWS = 128
_scratch: Dict[str, torch.Tensor] = {}
_scratch_retired = []          # outgrown buffers stay alive: a captured graph may still point at them


def decode_scratch(device, floats: int) -> Optional[torch.Tensor]:
    """The float32 scratch the split-key decode kernel merges through; grown on demand, never
    freed (launches on one stream are ordered, so one buffer per device serves them all)."""
    if floats <= 0:
        return None
    key = str(device)
    t = _scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _scratch_retired.append(t)
        t = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def paged_attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, rows: Optional[torch.Tensor],
                           n_rows: int, positions, token_entry, entry_slot, block_table: torch.Tensor, nq: int,
                           nkv: int, d: int, page_size: int, window: Optional[int], scale: float, num_splits: int,
                           status: torch.Tensor) -> torch.Tensor:
    """Attention for single decoded tokens (rows of q named by `rows`, or rows 0..n_rows-1), written
    into the same rows of `out`.  bfloat16 only."""
    _dev(q, out, cache, rows, positions, token_entry, entry_slot, block_table, status)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the decode attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    need = _fn("attention_decode", "llm_paged_decode_scratch_floats", [c_int, c_int, c_int, c_int],
               restype=c_longlong)(n_rows, nq, d, num_splits)
    scratch = decode_scratch(q.device, int(need))
    f = _fn("attention_decode", "llm_paged_attention_decode",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), _ptr(rows), n_rows, _ptr(positions), _ptr(token_entry),
             _ptr(entry_slot), _ptr(block_table), block_table.shape[1], nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], num_splits, _ptr(scratch), _ptr(status),
             _stream()), "paged_attention_decode")
    if num_splits > 1:
        global launch_count
        launch_count += 1                         # the merge kernel
    return out


def paged_attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                            n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                            block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                            window: Optional[int], scale: float, status: torch.Tensor) -> torch.Tensor:
    """Attention for prompt portions: `tiles` int32 [n_tiles, 2] = (entry, first row of a
    PREFILL_TILE_ROWS-row tile inside the entry).  bfloat16 only."""
    _dev(q, out, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    f = _fn("attention_prefill", "llm_paged_attention_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d,
             page_size, int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_prefill")
    return out


def prefill_tcgen05_supported(d: int, page_size: int) -> bool:
    f = _fn("attention_prefill_tcgen05", "llm_paged_prefill_tcgen05_supported", [c_int, c_int])
    return bool(f(d, page_size))


def paged_attention_prefill_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                                    n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                                    block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                    window: Optional[int], scale: float, status: torch.Tensor) -> torch.Tensor:
    """The prompt-portion attention on tcgen05/TMEM with TMA loads (head size 128, pages of 8..64);
    same arguments as `paged_attention_prefill`."""
    _dev(q, out, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    f = _fn("attention_prefill_tcgen05", "llm_paged_attention_prefill_tcgen05",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), q.shape[0], _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_prefill_tcgen05")
    return out


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(logits, out)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("logits must be float32 [rows, vocab]")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    scratch = decode_scratch(logits.device, R * 64 * 2)
    f = _fn("sampling", "llm_argmax_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), R, V, _ptr(out), _ptr(scratch), _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, row_slot: torch.Tensor, sampler_state: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row by the row's slot state {seed_lo, seed_hi, counter, temperature bits};
    temperature <= 0 takes the argmax.  Advances the counters of sampled rows."""
    _dev(logits, row_slot, sampler_state, out)
    _i32(row_slot, "row_slot")
    _i32(sampler_state, "sampler_state")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("logits must be float32 [rows, vocab]")
    if sampler_state.dim() != 2 or sampler_state.shape[1] != 4:
        raise KernelError("sampler_state must be int32 [slots, 4]")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "llm_sample_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), R, V, _ptr(row_slot), _ptr(sampler_state), _ptr(out), _stream()), "sample_rows")
    return out


def sampler_uniform(seed: int, counter: int) -> float:
    """The u in [0,1) that the sampling kernel draws for (seed, counter); runs on the host."""
    f = _fn("sampling", "llm_sampler_uniform", [c_uint64, c_uint32], restype=c_float)
    return float(f(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFF))


# ------------------------------------------------------------------------------------------
_skinny_scratch: Dict[str, torch.Tensor] = {}


def skinny_scratch(device, floats: int) -> Optional[torch.Tensor]:
    """Scratch for the streaming product's k-splits; grown on demand, never freed."""
    if floats <= 0:
        return None
    key = str(device)
    t = _skinny_scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _scratch_retired.append(t)
        t = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _skinny_scratch[key] = t
    return t


SKINNY_MAX_ROWS = 16     # rows up to which `linear` takes the engine's own streaming kernel
SKINNY_SMALL_MAX_ROWS = 32    # and for small (latency-bound) products, see `skinny_small`
_skinny_small: Dict[tuple, bool] = {}


def skinny_small(n: int, k: int) -> bool:
    """Whether an [n, k] product has fewer items than would give every CTA slot of the streaming kernel
    four: then latency bounds it, not bytes, and the kernel takes it up to 32 rows."""
    got = _skinny_small.get((n, k))
    if got is None:
        got = _skinny_small[(n, k)] = bool(_fn("gemm_skinny", "llm_linear_skinny_small", [c_int, c_int])(n, k))
    return got



# ---- weights stored tile by tile for the streaming product ----------------------------------
# The streaming product reads the plain [N, K] weights box by box through the copy engine, or, 2.5 %
# (batch 8) to 4.5 % (batch 1) faster per decode step, a second copy of them stored in its
# shared-memory order.  That copy doubles the weights' memory, so it is made only for models whose
# weights are a small share of the device: `begin_model` decides once per model.
_TILED_POLICY = os.environ.get("LLM_TILED", "auto")   # on | auto | off
_TILED_SHARE = 0.125                                   # auto: models whose matrices take up to this share of the device's memory
_tiled: Dict[int, torch.Tensor] = {}                   # weight.data_ptr() -> its tiled copy
_tiled_allowed = _TILED_POLICY != "off"          # until a model says otherwise (`begin_model`)
TILE_ROWS, TILE_K = 64, 256


def begin_model(matrix_bytes: int, device) -> bool:
    """Called before a model's weights are loaded with the bytes of its bfloat16 matrices: decides
    whether `prepare_streaming` makes tiled copies for them (all of them or none).  `LLM_TILED=on` /
    `off` overrides the rule."""
    global _tiled_allowed
    device = torch.device(device)
    if _TILED_POLICY == "off" or device.type != "cuda":
        _tiled_allowed = False
    elif _TILED_POLICY == "on":
        _tiled_allowed = True
    else:
        _, total = torch.cuda.mem_get_info(device)
        _tiled_allowed = matrix_bytes <= _TILED_SHARE * total
    return _tiled_allowed


def tile_weight(weight: torch.Tensor) -> torch.Tensor:
    """bfloat16 [N, K] -> the same values as [N/64 tiles, K/256 steps] blocks of 32 KB, each four
    sub-tiles of [64 rows][64 k-values] with 128-byte rows whose 16-byte chunks are XOR-swizzled by
    the row (chunk c of row r at position c ^ (r % 8)), zero-padded at the edges.  A stage of the
    streaming product is one block for up to 8 tokens and half a block for 9 to 16; a K-major tcgen05 operand of 128 rows x 64
    k-values is two sub-tiles."""
    N, K = weight.shape
    tn, nk = -(-N // TILE_ROWS), -(-K // TILE_K)
    padded = torch.zeros((tn * TILE_ROWS, nk * TILE_K), dtype=weight.dtype, device=weight.device)
    padded[:N, :K] = weight
    v = padded.view(tn, TILE_ROWS, nk, TILE_K // 64, 8, 8)               # [tile, row, step, sub, chunk, 8 values]
    r = torch.arange(TILE_ROWS, device=weight.device)[:, None]
    p = torch.arange(8, device=weight.device)[None, :]
    src = p ^ (r & 7)                                                     # the chunk that lands at position p of row r
    idx = src[None, :, None, None, :, None].expand(tn, TILE_ROWS, nk, TILE_K // 64, 8, 8)
    return torch.gather(v, 4, idx).permute(0, 2, 3, 1, 4, 5).contiguous().view(tn, nk, TILE_ROWS * TILE_K)


def prepare_streaming(weight: Optional[torch.Tensor]) -> None:
    """Keep a tiled copy of a bfloat16 weight for decode steps of up to 16 tokens, if `begin_model`
    allowed copies for the model being loaded.  The copy lives as long as the weight."""
    if (weight is None or not _tiled_allowed or not weight.is_cuda or weight.dtype != torch.bfloat16
            or weight.dim() != 2 or weight.shape[1] % 8 != 0):
        return
    key = weight.data_ptr()
    if key in _tiled:
        return
    _tiled[key] = tile_weight(weight)
    weakref.finalize(weight, _tiled.pop, key, None)


_tiled_generation = 0


def release_streaming() -> int:
    """Drop every tiled copy (the weights themselves stay; products fetch them box by box from their
    plain layout from then on).  Returns how many copies went.  Captured CUDA graphs that read the copies must
    not be replayed afterwards: `streaming_generation` changes, and the runner drops its graphs."""
    global _tiled_generation
    n = len(_tiled)
    if n:
        torch.cuda.synchronize()                 # nothing in flight still reads them
        _tiled.clear()
        _tiled_generation += 1
    return n


def streaming_generation() -> int:
    """Counts the times the tiled copies were dropped."""
    return _tiled_generation


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                  out: Optional[torch.Tensor] = None, partials_ok: bool = False):
    """x [M <= 32, K] @ weight[N, K]^T with the engine's own weight-streaming kernel (bfloat16
    operands, float32 accumulation, float32 or bfloat16 result).  With `partials_ok` a product
    that is cut into k-splits comes back as a `PartialSum` instead of being added up."""
    _dev(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("the skinny product takes bfloat16 operands")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError("x and weight disagree on K")
    global launch_count
    tiled = _tiled.get(weight.data_ptr())
    g = _fn("gemm_skinny", "llm_linear_skinny_tiled" if tiled is not None else "llm_linear_skinny_boxes",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    st, wp = stream_status(x.device), _ptr(tiled if tiled is not None else weight)
    f = lambda xp, _w, yp, dt, sp, sn, m, n, k, keep, stream: g(xp, wp, yp, dt, sp, sn, m, n, k, keep, _ptr(st), stream)
    splits = _fn("gemm_skinny", "llm_linear_skinny_splits", [c_int, c_int, c_int])(M, N, K)
    if partials_ok and splits > 1 and out is None:
        parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        _check(f(_ptr(x), _ptr(weight), None, 0, _ptr(parts), parts.numel(), M, N, K, 1, _stream()), "linear_skinny")
        return PartialSum(parts, None if out_dtype == torch.float32 else out_dtype)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    scratch = skinny_scratch(x.device, splits * M * N if splits > 1 else 0)
    _check(f(_ptr(x), _ptr(weight), _ptr(out), _dt(out), _ptr(scratch), scratch.numel() if scratch is not None else 0,
             M, N, K, 0, _stream()), "linear_skinny")
    launch_count += 1 if splits > 1 else 0        # the kernel that adds the k-splits
    return out


_stream_status: Dict[str, torch.Tensor] = {}


def stream_status(device) -> torch.Tensor:
    """The status word of the engine's matrix products (code 8: a bounded wait of the weight-streaming
    product ran out; 9: of the paired product)."""
    key = str(device)
    t = _stream_status.get(key)
    if t is None:
        t = _stream_status[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return t


def linear_pair(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """x [T, K] @ weight[N, K]^T for prompt portions with the engine's own tcgen05 kernel, in which
    two CTAs of a cluster share a tile of 256 tokens x 256 features (bfloat16 operands, float32
    accumulation in tensor memory, float32 or bfloat16 result).  With `accumulate` the product is
    added to the float32 `out` in place."""
    if accumulate and (out is None or out.dtype != torch.float32):
        raise KernelError("accumulating wants a float32 out")
    _dev(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("the paired product takes bfloat16 operands")
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError("x and weight disagree on K")
    if out is None:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if out.shape != (T, N) or not out.is_contiguous():
        raise KernelError("out must be a contiguous [T, N]")
    f = _fn("gemm_pair_tcgen05", "llm_linear_pair",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(out), _dt(out), 1 if accumulate else 0, T, N, K, _ptr(stream_status(x.device)),
             _stream()), "linear_pair")
    return out


def linear_pair_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x @ gate^T) * (x @ up^T) for w_gate_up = [gate; up] of 2 I rows, as bfloat16 [T, I]: the
    paired tcgen05 product with the activation in its epilogue (gate and up are rounded to bfloat16
    before the activation, as the separate kernel would read them)."""
    _dev(x, w_gate_up, out)
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        raise KernelError("the paired product takes bfloat16 operands")
    T, K = x.shape
    if w_gate_up.shape[1] != K or w_gate_up.shape[0] % 2 != 0:
        raise KernelError("x and the gate/up weight disagree")
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((T, inter), dtype=torch.bfloat16, device=x.device)
    f = _fn("gemm_pair_tcgen05", "llm_linear_pair_silu_mul", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(w_gate_up), _ptr(out), T, inter, K, _ptr(stream_status(x.device)), _stream()), "linear_pair_silu_mul")
    return out


_PAIR_POLICY = os.environ.get("LLM_PAIR", "auto")       # auto | all | off: which prompt-portion products take the paired kernel
PAIR_MIN_ROWS = 129                                      # fewer rows leave the second CTA of a pair idle
# Thousandths of the clusters' time that a product's tiles must fill for the paired kernel to be taken
# under `auto`; None: only under `all`.  With the activation in its epilogue it saves a kernel and wins
# from 0.85 on (prefill of the Qwen3-8B shape, 2,048 / 4,096 / 8,192 tokens: 26.9 / 56.2 / 123.9 ms
# against 27.9 / 58.8 / 124.1 with the library product and the activation kernel).  Alone it is level with
# the library kernel by kernel, but a prefill is power-bound and the clocks settle lower with it: taking
# the other products too gave 57.6 and 127.1 ms at 4,096 and 8,192 tokens, and adding into the residual
# 28.9 ms at 2,048.
_PAIR_NEEDS = {"plain": None, "silu": 850, "into": None}


def _pair_takes(x: torch.Tensor, weight: torch.Tensor, n: int, kind: str) -> bool:
    """Whether the paired tcgen05 product is the faster way for these operands: bfloat16 on the GPU,
    enough rows, and tiles that keep the clusters busy."""
    if (_PAIR_POLICY == "off" or not x.is_cuda or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16
            or x.shape[0] < PAIR_MIN_ROWS or not x.is_contiguous() or not weight.is_contiguous()):
        return False
    eff = _fn("gemm_pair_tcgen05", "llm_linear_pair_efficiency", [c_int, c_int, c_int, c_int])(
        x.shape[0], n, x.shape[1], 1 if kind == "silu" else 0)
    if eff <= 0:
        return False
    need = _PAIR_NEEDS[kind]
    return _PAIR_POLICY == "all" or (need is not None and eff >= need)


def linear_into(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual (float32 [T, N]) += x @ weight^T in the product's epilogue, if the paired kernel takes
    these operands; False, and nothing done, if not."""
    if (residual.dtype != torch.float32 or not residual.is_contiguous() or residual.shape != (x.shape[0], weight.shape[0])
            or not _pair_takes(x, weight, weight.shape[0], "into")):
        return False
    linear_pair(x, weight, torch.float32, out=residual, accumulate=True)
    return True


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out_dtype: torch.dtype):
    """silu(x @ gate^T) * (x @ up^T) for w_gate_up = [gate; up]: one kernel where the paired product
    takes it, else the product (which may stay a sum of k-splits) followed by the activation kernel."""
    if out_dtype == torch.bfloat16 and _pair_takes(x, w_gate_up, w_gate_up.shape[0] // 2, "silu"):
        return linear_pair_silu_mul(x, w_gate_up)
    return silu_and_mul(linear(x, w_gate_up, out_dtype=out_dtype, partials_ok=True))


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           partials_ok: bool = False):
    """x [T, K] @ weight[N, K]^T.  Up to 16 bfloat16 rows (decode steps; up to 32 for the small products
    of small models) go through the engine's
    own weight-streaming kernel: alone it is level with the library for N = 4096..24576 and
    faster for K = 12288 (32 us against 36) and N = 151936 (203 against 218), and in a step it
    starts fetching weights while the kernel before it drains (a whole decode step of the
    Qwen3-8B shape at batch 8: 4.35 ms against 4.77 with the library products).  Everything else
    goes through the library matrix product (under `LLM_PAIR=all`, prompt portions take the paired tcgen05
    product `linear_pair`; by default only the gate/up product does, through `linear_silu_mul`) (the reference uses cuBLAS for all its products,
    src/layers/linear.cu:169-215).  bfloat16 operands accumulate in float32; a float32 weight
    keeps its product in true float32 (no TF32), whatever x is."""
    _dev(x, weight)
    rows = x.shape[0]
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and weight.data_ptr() % 16 == 0
            and rows >= 1 and (rows <= SKINNY_MAX_ROWS
                               or (rows <= SKINNY_SMALL_MAX_ROWS and skinny_small(weight.shape[0], weight.shape[1])))):
        return linear_skinny(x, weight, out_dtype or x.dtype, partials_ok=partials_ok)
    if x.shape[0] >= PAIR_MIN_ROWS and (out_dtype or x.dtype) in (torch.float32, torch.bfloat16) and _pair_takes(
            x, weight, weight.shape[0], "plain"):
        return linear_pair(x, weight, out_dtype or x.dtype)
    if weight.dtype == torch.float32:
        y = torch.mm(x if x.dtype == torch.float32 else x.float(), weight.t())
        want = out_dtype or x.dtype
        return y if want == torch.float32 else y.to(want)
    if x.dtype != weight.dtype:
        x = x.to(weight.dtype)
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())


def configure_library_products() -> None:
    """No reduced-precision modes in the library products: float32 stays IEEE float32 and
    bfloat16 products reduce in float32."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:
        pass
