"""The decode attention entry point that allocates nothing, called the way a host without the
engine's Python side calls it: through its exported C symbol, with the caller's own inputs and
outputs.  Such a host (one that gave all device memory to its own pool, or one that cannot risk
the device-wide stall of cudaMalloc inside its loop) gets the key splits' scratch from a static
array inside the library.  Checked here: two calls in a row give what the allocating entry point
gives and what attention computed plainly in double precision gives; the device's free memory (as
the driver reports it, not only the tensor library's own pool) is the same before and after the
calls; and a call that needs more scratch than the array holds is refused with a readable message
and launches nothing.  This file is collected last, so a run that stops at the first failure has
already run every other test."""
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

    def plain(q):
        """softmax(q k^T / sqrt(d)) v per request and head in float64, keys gathered page by page."""
        out = torch.zeros(B, nq, d, dtype=torch.float64)
        c, tb, qd = cache.double().cpu(), table.cpu(), q.double().cpu().view(B, nq, d)
        for b, n in enumerate(lens):
            kv = torch.stack([c[tb[b, t // page], :, :, t % page] for t in range(n)])      # [n, 2, nkv, d]
            for h in range(nq):
                k, v = kv[:, 0, h // (nq // nkv)], kv[:, 1, h // (nq // nkv)]
                out[b, h] = torch.softmax(k @ qd[b, h] / math.sqrt(d), dim=0) @ v
        return out.view(B, nq * d)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    ent = torch.arange(B, dtype=torch.int32, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    stream = torch.cuda.current_stream().cuda_stream

    def call(q, got, splits):
        return fn(q.data_ptr(), got.data_ptr(), cache.data_ptr(), None, B, pos.data_ptr(), ent.data_ptr(),
                  slot.data_ptr(), table.data_ptr(), table.shape[1], nq, nkv, d, page, 0, scale, pages, splits,
                  status.data_ptr(), stream)

    # One warm call first: it loads the module's kernels and looks the array's address up, after which
    # the device's free memory must not move.  Every tensor the loop needs exists before the reading.
    qs = [torch.randn(B, nq * d, device=DEV).to(torch.bfloat16) for _ in range(2)]
    gots = [[torch.zeros_like(qs[0]) for _ in range(2)] for _ in range(2)]
    assert call(qs[0], gots[0][0], 5) == 0
    torch.cuda.synchronize()
    free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for i in range(2):                            # two calls in a row share the static scratch
        for j, splits in enumerate((1, 5)):
            rc = call(qs[i], gots[i][j], splits)
            assert rc == 0, lib.llm_noalloc_strerror(rc).decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory changed across the calls"
    assert torch.cuda.memory_allocated() == torch_before

    for i in range(2):
        ref = plain(qs[i])
        for j, splits in enumerate((1, 5)):
            got = gots[i][j]
            want = torch.zeros_like(got)
            ops.paged_attention_decode(qs[i], want, cache, None, B, pos, ent, slot, table, nq, nkv, d, page, None, scale,
                                       splits, status)
            err = float((got.float() - want.float()).abs().max())
            assert err <= 1e-2 * max(1.0, float(want.float().abs().max())), f"call {i}, {splits} splits: {err}"
            err = float((got.double().cpu() - ref).abs().max())
            assert err <= 1e-2 * max(1.0, float(ref.abs().max())), f"call {i}, {splits} splits against plain: {err}"
            assert float(got.float().abs().max()) > 0
    assert status.tolist() == [0, 0]
    q = qs[1]

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
