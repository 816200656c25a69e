"""Per-kernel micro-benchmarks: time one kernel at a model's sizes with CUDA events and report
achieved bytes/s (or flop/s) beside the peak.

    python -m litellmengine_b200.csrc.microbench decode_attention --batch 64 --context 4096
    python -m litellmengine_b200.csrc.microbench prefill_attention --tokens 2048
    python -m litellmengine_b200.csrc.microbench rmsnorm --tokens 2048
    python -m litellmengine_b200.csrc.microbench linear --tokens 8 --n 6144 --k 4096

Sizes default to the Qwen3-8B shape (32 heads, 8 kv heads, head 128, hidden 4096, page 16).
Between timed launches a buffer larger than L2 is overwritten, so every launch starts cold.
`--iters 1 --warmup 1` keeps a run short enough to put under a profiler.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import ops

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    out = dict(FALLBACK, source="fallback")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            for k in FALLBACK:
                v = d.get(k)
                v = v.get("value") if isinstance(v, dict) else v
                if isinstance(v, (int, float)) and v > 0:
                    out[k] = float(v)
            out["source"] = "measured"
        except Exception:
            pass
    return out


class Flusher:
    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e-3


def paged_setup(args, dev, q_len):
    """`batch` requests of `context` cached tokens in shuffled pages; q_len query rows each."""
    B, S, P, nq, nkv, d = args.batch, args.context, args.page, args.heads, args.kv_heads, args.head_dim
    width = (S + P - 1) // P
    pages = B * width
    cache = torch.randn(pages, 2, nkv, P, d, device=dev, dtype=torch.bfloat16)
    table = torch.randperm(pages, device=dev).to(torch.int32).view(B, width).contiguous()
    T = B * q_len
    q = torch.randn(T, nq * d, device=dev, dtype=torch.bfloat16)
    pos = (torch.arange(S - q_len, S, device=dev, dtype=torch.int32)).repeat(B)
    ent = torch.arange(B, device=dev, dtype=torch.int32).repeat_interleave(q_len)
    slot = torch.arange(B, device=dev, dtype=torch.int32)
    return cache, table, q, pos, ent, slot


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["decode_attention", "prefill_attention", "rmsnorm", "qk_rope_write",
                                       "silu_and_mul", "linear", "argmax"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--out-dtype", default="bfloat16")
    ap.add_argument("--impl", default="auto", choices=["auto", "library", "own", "tcgen05", "pair", "pair_silu", "library_silu"],
                    help="linear: the library product, the engine's own streaming kernel, or what the engine picks")
    ap.add_argument("--tiled", action="store_true", help="linear --impl own: over a tile-by-tile copy of the weights")
    ap.add_argument("--chain", type=int, default=0,
                    help="linear: time CHAIN launches back to back, each over weights of its own (together larger "
                         "than L2), as one CUDA graph; the figure is the time per launch inside a stream of kernels")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    ops.configure_library_products()
    pk = peaks()
    flush = Flusher(dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    nq, nkv, d, P = args.heads, args.kv_heads, args.head_dim, args.page
    scale = 1.0 / math.sqrt(d)
    res = {"kernel": args.kernel}

    if args.kernel == "decode_attention":
        cache, table, q, pos, ent, slot = paged_setup(args, dev, 1)
        out = torch.empty_like(q)
        from ..parts.attention import decode_key_splits
        splits = args.splits or decode_key_splits(dev, args.batch, nkv, args.context)     # what the engine picks
        fn = lambda: ops.paged_attention_decode(q, out, cache, None, args.batch, pos, ent, slot, table, nq, nkv, d, P,
                                                None, scale, splits, status)
        nbytes = args.batch * args.context * 2 * nkv * d * 2
        res.update(batch=args.batch, context=args.context, splits=splits, bytes=nbytes)
    elif args.kernel == "prefill_attention":
        args.batch, args.context = 1, args.tokens
        cache, table, q, pos, ent, slot = paged_setup(args, dev, args.tokens)
        out = torch.empty_like(q)
        R = ops.PREFILL_TILE_ROWS
        n_tiles = (args.tokens + R - 1) // R
        tiles = torch.tensor([[0, R * i] for i in reversed(range(n_tiles))], dtype=torch.int32, device=dev)
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
        kern = ops.paged_attention_prefill_tcgen05 if args.impl == "tcgen05" else ops.paged_attention_prefill
        q_start, q_len, kv_len = i32(0), i32(args.tokens), i32(args.tokens)
        fn = lambda: kern(q, out, cache, tiles, n_tiles, slot, q_start, q_len, kv_len, table, nq, nkv, d, P, None,
                          scale, status)
        res["impl"] = args.impl
        res.update(tokens=args.tokens, flops=4 * nq * d * args.tokens * (args.tokens + 1) // 2)
    elif args.kernel == "rmsnorm":
        x = torch.randn(args.tokens, args.hidden, device=dev)
        delta = torch.randn(args.tokens, args.hidden, device=dev)
        w = torch.ones(args.hidden, device=dev)
        fn = lambda: ops.rmsnorm(x, w, 1e-6, torch.bfloat16, delta=delta, write_sum=True)
        res.update(tokens=args.tokens, bytes=args.tokens * args.hidden * (4 + 4 + 4 + 2))
    elif args.kernel == "qk_rope_write":
        args.batch, args.context = 1, args.tokens
        cache, table, q, pos, ent, slot = paged_setup(args, dev, args.tokens)
        qkv = torch.randn(args.tokens, (nq + 2 * nkv) * d, device=dev)
        w = torch.ones(d, device=dev)
        inv = torch.rand(d // 2, device=dev)
        angles = ops.rope_angles(pos, inv) if args.tokens >= ops.ROPE_TABLE_MIN_TOKENS and args.impl != "own" else None
        fn = lambda: ops.qk_norm_rope_kv_write(qkv, cache, pos, ent, slot, table, w, w, 1e-6, inv, d, nq, nkv, d, P,
                                               True, status, q_dtype=torch.bfloat16, angles=angles)
        res.update(tokens=args.tokens, bytes=args.tokens * (nq + 2 * nkv) * d * (4 + 2))
    elif args.kernel == "silu_and_mul":
        gu = torch.randn(args.tokens, 2 * args.inter, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.silu_and_mul(gu)
        res.update(tokens=args.tokens, bytes=args.tokens * args.inter * 2 * 3)
    elif args.kernel == "argmax":
        lg = torch.randn(args.batch, args.vocab, device=dev)
        fn = lambda: ops.argmax_rows(lg)
        res.update(batch=args.batch, bytes=args.batch * args.vocab * 4)
    else:
        x = torch.randn(args.tokens, args.k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16) * 0.02
        od = torch.float32 if args.out_dtype == "float32" else torch.bfloat16
        if args.tiled:
            ops.prepare_streaming(w)
        if args.impl == "library":
            fn = lambda: torch.mm(x, w.t(), out_dtype=od) if od != x.dtype else torch.mm(x, w.t())
        elif args.impl == "own":
            fn = lambda: ops.linear_skinny(x, w, od)
        elif args.impl == "pair":
            fn = lambda: ops.linear_pair(x, w, od)
        elif args.impl == "pair_silu":                            # w is [gate; up]: N = 2 I
            fn = lambda: ops.linear_pair_silu_mul(x, w)
        elif args.impl == "library_silu":
            fn = lambda: ops.silu_and_mul(torch.mm(x, w.t()))
        else:
            fn = lambda: ops.linear(x, w, out_dtype=od)
        if args.chain:
            ws = [torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(args.chain)]
            if args.tiled:
                for wi in ws:
                    ops.prepare_streaming(wi)
            one = {"library": lambda wi: torch.mm(x, wi.t(), out_dtype=od) if od != x.dtype else torch.mm(x, wi.t()),
                   "own": lambda wi: ops.linear_skinny(x, wi, od)}.get(args.impl, lambda wi: ops.linear(x, wi, out_dtype=od))
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for wi in ws:
                    one(wi)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for wi in ws:
                        one(wi)
            chain_fn = graph.replay
            fn = lambda: chain_fn()
            res["chain"] = args.chain
        res["impl"] = args.impl
        res.update(m=args.tokens, n=args.n, k=args.k, bytes=args.n * args.k * 2 + args.tokens * (args.k * 2 + args.n * od.itemsize),
                   flops=2 * args.tokens * args.n * args.k)

    sec = timed(fn, args.iters, args.warmup, flush)
    if args.kernel == "linear" and args.chain:
        sec /= args.chain
    res["us"] = round(sec * 1e6, 2)
    if "bytes" in res:
        res["GB/s"] = round(res["bytes"] / sec / 1e9, 1)
        res["hbm_frac"] = round(res["GB/s"] / pk["hbm_gbs"], 3)
    if "flops" in res:
        res["TFLOP/s"] = round(res["flops"] / sec / 1e12, 1)
        res["bf16_frac"] = round(res["TFLOP/s"] / pk["bf16_tflops"], 3)
    res["peaks"] = pk["source"]
    assert status.tolist() == [0, 0], "a kernel recorded a refused index"
    print(json.dumps(res))


if __name__ == "__main__":
    main()
