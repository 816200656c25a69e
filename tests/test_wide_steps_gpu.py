"""The steps a benchmark times, checked: two layers at the widths of a real 8B model (hidden 4,096,
32/8 heads of 128, feed-forward 12,288; a small vocabulary keeps it quick), stepped with 8 to 64
live requests, decode-only and beside a prompt portion, as captured graphs and as plain launches,
against the plain implementation; and the same model at a context of 4,096 tokens in every way of
cutting, in float32 and in bfloat16.  Then the tiny head-size-128 model with 64 requests decoding
together in a cache too small for them.

The plain implementation runs on the GPU here (same formulas, the tensor library's float32 and
float64 products): at these widths the CPU would take minutes."""
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import replay_helpers as rh
import tiny_models as tm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDE2 = dict(tm.WIDE_G, num_hidden_layers=2)
PAGE = 16


@pytest.fixture(scope="module")
def wide():
    """Weights that a bfloat16 engine holds exactly, attention sharpened as for the other models of
    head size 128, and a copy on the GPU for the plain code."""
    w = rh.sharpen(tm.make_weights(WIDE2, tm.WIDE_G_SEED, bf16_exact=True), 2.0, bf16_exact=True)
    return w, {k: v.to(DEV) for k, v in w.items()}


def plain_on_gpu(wg, reqs, dtype):
    torch.backends.cuda.matmul.allow_tf32 = False
    out = {}
    for r, t in reqs.items():
        if dtype == "bfloat16":
            lg = pq.forward_logits(t, wg, WIDE2, act=pq.to_bf16, attn_act=pq.to_bf16)
        else:
            lg = pq.forward_logits(t, wg, WIDE2, wd=torch.float64)
        out[r] = lg.cpu().numpy()
    return out


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("n", [8, 9, 16, 17, 40, 64])
def test_decode_steps_of_many_requests(wide, n, graphs):
    """n live requests of different lengths: prompts several to a step, then decode steps of all n (the
    second is captured as a graph, the third replays it), a step of n decoded tokens beside a 200-token
    portion of one more request, and a decode step after it.  Every logit row against the plain code."""
    from litellmengine_b200.engine import StepEntry
    w, wg = wide
    rng = random.Random(n)
    reqs = {f"r{i}": tm.random_tokens(WIDE2, rng.randint(20, 260) + 5, 1000 * n + i) for i in range(n)}
    reqs["late"] = tm.random_tokens(WIDE2, 230, 77 + n)
    ref = plain_on_gpu(wg, reqs, "bfloat16")
    runner = rh.make_runner(WIDE2, w, "bfloat16", PAGE, max_total_tokens=(n + 1) * 288, max_requests=n + 1,
                            max_tokens_per_step=1536)
    runner.use_graphs = runner.use_graphs and graphs
    steps, names = [], list(reqs)[:n]
    for i in range(0, n, 4):                                   # prompts, four requests to a step
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": r, "tokens": reqs[r][:-5], "want": [len(reqs[r]) - 6]} for r in names[i:i + 4]]})
    for d in range(5):
        entries = [{"id": r, "tokens": [reqs[r][len(reqs[r]) - 5 + d]], "want": [0]} for r in names]
        if d == 3:                                             # a prompt portion beside the decoded tokens
            entries.insert(n // 2, {"id": "late", "tokens": reqs["late"][:200], "want": [0, 127, 128, 199]})
        steps.append({"step": len(steps), "entries": entries, "end": names if d == 4 else []})
    steps.append({"step": len(steps), "entries": [{"id": "late", "tokens": reqs["late"][200:], "want": [0, 29]}], "end": ["late"]})
    got = rh.run_trace(runner, steps)
    assert len(got) == n * 6 + 6
    assert (runner.graph_replays > 0) == graphs
    rh.assert_rows_match(got, ref, rh.BF16_TOL, f"{n} requests, graphs {graphs}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_at_a_context_of_4096(wide, dtype):
    """Requests of 4,096, 1,500, 700 and 300 tokens: whole, the last 32 tokens one by one, in portions
    of changing size (2 to 1,000 tokens), and mixed with up to four live requests in a pool sized to
    the peak, so that pages are used again.  Every position against the plain code."""
    w, wg = wide
    reqs = {f"r{i}": tm.random_tokens(WIDE2, n, 4096 + i) for i, n in enumerate((4096, 1500, 700, 300))}
    ref = plain_on_gpu(wg, reqs, dtype)
    tol = rh.tol_for(dtype)
    for what, steps in (("whole", rh.trace_whole(reqs)), ("tail", rh.trace_tail_decode(reqs, 32)),
                        ("portions", rh.trace_portions(reqs, 7, sizes=(2, 3, 1000, 17, 129, 640, 31, 2, 64, 257))),
                        ("mixed", rh.trace_mixed(reqs, 8, 4))):
        runner = rh.make_runner(WIDE2, w, dtype, PAGE, max_total_tokens=rh.peak_tokens(steps, 64), max_requests=4,
                                max_tokens_per_step=4096)
        got = rh.run_trace(runner, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        rh.assert_rows_match(got, ref, tol, f"context 4096 {dtype} {what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sixty_four_requests_decode_together_under_page_pressure(dtype):
    """The tiny model of head size 128 with 64 request slots: 64 greedy requests in a cache that holds
    seven eighths of what they need at their longest, so that some are preempted and recomputed
    while 50 and more decode together.  Float32: the tokens are the plain implementation's.  bfloat16: a
    token may differ only where the two best logits are closer than bfloat16 resolves."""
    from litellmengine_b200.engine import PagedGenerateEngine
    cfg, page = tm.TINY_E, tm.TINY_E_PAGE
    bf = dtype == "bfloat16"
    w = tm.make_weights(cfg, tm.TINY_E_SEED, bf16_exact=bf)
    rng = random.Random(5)
    prompts = [tm.random_tokens(cfg, rng.randint(6, 40), 500 + i) for i in range(64)]
    new = 14
    peak = sum(-(-(len(p) + new) // page) * page for p in prompts)
    runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=peak * 7 // 8 // page * page, max_requests=64, max_tokens_per_step=256)
    eng = PagedGenerateEngine(runner, chunk=32)
    most = 0
    ids = [eng.add_request(p, new) for p in prompts]
    while eng.has_work():
        eng.step()
        most = max(most, sum(1 for r in eng.scheduler.running if r.extend_len == 1))
    runner.check_status()
    runner.cache.check_invariants()
    assert eng.scheduler.num_preemptions > 0 and most >= 50, (eng.scheduler.num_preemptions, most)
    assert all(g.pool.free_count == g.pool.num_pages for g in runner.cache.groups)
    act = pq.to_bf16 if bf else pq.identity
    for p, i in zip(prompts, ids):
        got = eng.request(i).generated_ids
        assert len(got) == new
        if not bf:
            assert got == pq.greedy_generate(p, w, cfg, new)
            continue
        seq = list(p)
        for t in got:
            lg = pq.forward_logits(seq, w, cfg, act=act, attn_act=act)[-1]
            best = pq.argmax_token(lg)
            if t != best:
                assert float(lg[best] - lg[t]) < 2e-2, f"token {t} instead of {best}"
            seq.append(t)
