"""The decode attention entry point that allocates nothing, called the way a host without the
engine's Python side calls it: through its exported C symbol, with the caller's own inputs and
outputs.  Such a host (one that gave all device memory to its own pool, or one that cannot risk
the device-wide stall of cudaMalloc inside its loop) gets the key splits' scratch from a static
array inside the library.  Checked here: two calls in a row give what the allocating entry point
gives, and a call that needs more scratch than the array holds is refused with a readable message
and launches nothing.  This file is collected last, so a
run that stops at the first failure has already run every other test."""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_decode_attention_without_allocation_matches_the_allocating_entry_point():
    from litellmengine_b200.csrc import ops
    lib = ops.lib("attention_decode")
    fn = lib.llm_paged_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    lib.llm_paged_attention_decode_noalloc_needed.argtypes = [c_int, c_int, c_int, c_int]
    lib.llm_paged_attention_decode_noalloc_needed.restype = c_longlong
    lib.llm_noalloc_strerror.argtypes = [c_int]
    lib.llm_noalloc_strerror.restype = ctypes.c_char_p

    torch.manual_seed(0)
    nq, nkv, d, page, B = 8, 2, 128, 16, 5
    lens = [700, 33, 1, 260, 513]
    width = max((n + page - 1) // page for n in lens) + 1
    pages = B * width
    cache = torch.randn(pages, 2, nkv, page, d, device=DEV).to(torch.bfloat16)
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(B, width).contiguous()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    ent = torch.arange(B, dtype=torch.int32, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    stream = torch.cuda.current_stream().cuda_stream

    for call in range(2):                         # two calls in a row share the static scratch
        q = torch.randn(B, nq * d, device=DEV).to(torch.bfloat16)
        for splits in (1, 5):
            want = torch.zeros_like(q)
            ops.paged_attention_decode(q, want, cache, None, B, pos, ent, slot, table, nq, nkv, d, page, None, scale,
                                       splits, status)
            got = torch.zeros_like(q)
            before = torch.cuda.memory_allocated()
            rc = fn(q.data_ptr(), got.data_ptr(), cache.data_ptr(), None, B, pos.data_ptr(), ent.data_ptr(),
                    slot.data_ptr(), table.data_ptr(), table.shape[1], nq, nkv, d, page, 0, scale, pages, splits,
                    status.data_ptr(), stream)
            assert rc == 0, lib.llm_noalloc_strerror(rc).decode()
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            err = float((got.float() - want.float()).abs().max())
            assert err <= 1e-2 * max(1.0, float(want.float().abs().max())), f"call {call}, {splits} splits: {err}"
            assert float(got.float().abs().max()) > 0
    assert status.tolist() == [0, 0]

    # sizes beyond the static array: refused, nothing launched, the output is untouched
    big_rows, big_splits = 4096, 16
    need = lib.llm_paged_attention_decode_noalloc_needed(big_rows, nq, d, big_splits)
    assert need == big_rows * nq * big_splits * (d + 2) > 4 * 1024 * 1024
    out = torch.full((B, nq * d), 7.0, device=DEV).to(torch.bfloat16)
    rc = fn(q.data_ptr(), out.data_ptr(), cache.data_ptr(), None, big_rows, pos.data_ptr(), ent.data_ptr(),
            slot.data_ptr(), table.data_ptr(), table.shape[1], nq, nkv, d, page, 0, scale, pages, big_splits,
            status.data_ptr(), stream)
    torch.cuda.synchronize()
    assert rc == -4 and b"exceeds" in lib.llm_noalloc_strerror(rc) and bool((out == 7.0).all())
