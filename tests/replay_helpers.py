"""Shared by the GPU tests: traces in the replay format, runners on tiny models, comparison
of replayed logits with the plain implementation at the same (request, position)."""
from __future__ import annotations

import random
from typing import Dict, List, Tuple

import numpy as np
import torch

import plain_qwen3 as pq
import tiny_models as tm

# Tolerances are fractions of max(1, max |reference logit|).
FP32_TOL = 1e-5       # float32 run against the plain code in double precision
# A bfloat16 run is compared twice.  Against the plain code rounding to bfloat16 where the
# engine does (same weights, sharpened attention): what is left is summation order and the
# rounding of values that straddle a bfloat16 boundary.  Against the plain float32 code on
# unsharpened weights: bfloat16's own error.
BF16_TOL = 1e-2
BF16_VS_FP32_TOL = 1.5e-2
# One way of cutting against another: both are roundings of the same exact value (the library
# matrix product picks its summation order by the number of rows), so the bound is the same.
FP32_CUT_TOL = FP32_TOL
BF16_CUT_TOL = BF16_TOL


def tol_for(dtype: str) -> float:
    return FP32_TOL if dtype == "float32" else BF16_TOL


def sharpen(w: Dict[str, torch.Tensor], factor: float = 4.0, bf16_exact: bool = False) -> Dict[str, torch.Tensor]:
    """Scale the q-norm weights so that attention scores spread out and single keys matter:
    with N(0, 0.02) weights softmax is nearly uniform and a lost key would hide in the mean."""
    out = dict(w)
    for n in w:
        if n.endswith("q_norm.weight"):
            t = w[n] * factor
            out[n] = t.to(torch.bfloat16).to(torch.float32) if bf16_exact else t
    return out


def make_runner(cfg: dict, weights: Dict[str, torch.Tensor], dtype: str, page: int, max_total_tokens: int,
                max_requests: int = 4, max_tokens_per_step: int = 1024):
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.engine import ModelRunner
    from litellmengine_b200.weights import DictSource
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    src = DictSource({k: (v.to(store) if v.dim() == 2 else v) for k, v in weights.items()})
    return ModelRunner.from_config(config_from_dict(cfg), dtype=dtype, device="cuda:0", source=src,
                                   page_size=page, max_total_tokens=max_total_tokens,
                                   max_requests=max_requests, max_tokens_per_step=max_tokens_per_step)


# ---- traces ------------------------------------------------------------------------------------
def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    return [{"step": i, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]}
            for i, (r, t) in enumerate(reqs.items())]


def trace_tail_decode(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps = []
    for r, t in reqs.items():
        n0 = max(len(t) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": r, "tokens": t[:n0], "want": list(range(n0))}], "end": []})
        for k in range(n0, len(t)):
            steps.append({"step": len(steps), "entries": [{"id": r, "tokens": [t[k]], "want": [0]}],
                          "end": [r] if k == len(t) - 1 else []})
        if n0 == len(t):
            steps[-1]["end"] = [r]
    return steps


def trace_portions(reqs: Dict[str, List[int]], seed: int, sizes=(2, 3, 5, 7, 16, 17, 31, 2, 64)) -> List[dict]:
    rng = random.Random(seed)
    steps = []
    for r, t in reqs.items():
        at = 0
        while at < len(t):
            n = min(rng.choice(sizes), len(t) - at)
            if len(t) - at - n == 1:          # never leave a single token: portions go down to two
                n += 1
            steps.append({"step": len(steps), "entries": [{"id": r, "tokens": t[at:at + n], "want": list(range(n))}],
                          "end": [r] if at + n == len(t) else []})
            at += n
    return steps


def trace_mixed(reqs: Dict[str, List[int]], seed: int, max_live: int = 4, prompt_frac: float = 0.6) -> List[dict]:
    """Up to `max_live` requests at a time.  Each feeds its first part in portions of changing
    size and the rest one token per step; every step batches whatever the live requests have
    next, so portions of some stand beside decoded tokens of others.  A finished request
    ends at once and the next one starts, in pages the ended one gave back."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: List[Tuple[str, List[int], int, int]] = []          # id, tokens, fed so far, length of the prompt part
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            r, t = waiting.pop(0)
            live.append((r, t, 0, min(len(t), max(2, int(len(t) * prompt_frac)))))
        entries, ended, nxt = [], [], []
        for r, t, at, plen in live:
            if rng.random() < 0.15 and len(live) > 1:          # a request may sit a step out
                nxt.append((r, t, at, plen))
                continue
            if at < plen:
                n = min(rng.choice((2, 3, 6, 11, 16, 23)), plen - at)
                if plen - at - n == 1:
                    n += 1
                assert n >= 1
            else:
                n = 1
            entries.append({"id": r, "tokens": t[at:at + n], "want": list(range(n))})
            at += n
            if at == len(t):
                ended.append(r)
            else:
                nxt.append((r, t, at, plen))
        live = nxt
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: List[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `round_to`."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return peak


# ---- comparison --------------------------------------------------------------------------------
def collect(steps: List[dict], logits_by_step: Dict[int, np.ndarray]) -> Dict[Tuple[str, int], np.ndarray]:
    """(request, position) -> logits row."""
    at: Dict[str, int] = {}
    out = {}
    for s in steps:
        rows = logits_by_step.get(s["step"])
        k = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        assert rows is None or k == len(rows)
    return out


def run_trace(runner, steps: List[dict]) -> Dict[Tuple[str, int], np.ndarray]:
    from litellmengine_b200.engine.trace import replay
    got = {}
    replay(runner, steps, lambda step, lg: got.__setitem__(step, lg.float().cpu().numpy()))
    runner.cache.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in runner.cache.groups), "pages left behind"
    return collect(steps, got)


def rounds_attention_weights(cfg: dict) -> bool:
    """The tensor-core attention kernels (head sizes 64 and 128) hand the weights exp(score - max)
    to the second product as bfloat16; the generic kernel, which every other head size runs,
    keeps them in float32."""
    return cfg["head_dim"] in (64, 128)


def plain_rows(cfg: dict, weights, reqs: Dict[str, List[int]], dtype: str = "float32") -> Dict[str, np.ndarray]:
    """Whole-sequence logits from the plain code.  For a float32 run the oracle works in double
    precision, so that the error measured is the engine's own; for a bfloat16 run it works in
    float32 and rounds to bfloat16 where the engine does."""
    if dtype == "bfloat16":
        attn_act = pq.to_bf16 if rounds_attention_weights(cfg) else None
        return {r: pq.forward_logits(t, weights, cfg, act=pq.to_bf16, attn_act=attn_act).numpy() for r, t in reqs.items()}
    return {r: pq.forward_logits(t, weights, cfg, wd=torch.float64).numpy() for r, t in reqs.items()}


def assert_rows_match(got: Dict[Tuple[str, int], np.ndarray], ref: Dict[str, np.ndarray], tol: float, what: str):
    """Reports the FIRST wrong (request, position), which is what tells a page edge from a
    portion start from a reused page."""
    scale = max(1.0, max(float(np.abs(v).max()) for v in ref.values()))
    assert got, "nothing was compared"
    for (r, pos) in sorted(got, key=lambda k: (k[0], k[1])):
        err = float(np.abs(got[(r, pos)] - ref[r][pos]).max())
        assert err <= tol * scale, f"{what}: request {r} position {pos}: max error {err:.3e} > {tol * scale:.3e}"


def requests_for(cfg: dict, lengths: List[int], seed: int) -> Dict[str, List[int]]:
    return {f"r{i}": tm.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lengths)}
