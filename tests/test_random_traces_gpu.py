"""Random traces and random generation jobs, a few seeds of each in every tiny configuration.

A trace here is anything the replay format allows: requests admitted in any order, portions of any
size anywhere (single tokens inside a prompt too), entries in any order within a step, requests that
sit a step out, wanted places that are all, some, the last or none of a portion, a pool of exactly
the peak, graphs on or off.  Each is compared with the plain implementation and with the same
requests run whole.  A generation job is prompts of 1 to 90 tokens with budgets of 1 to 24 new
tokens, some sampled, some ending at a stop token, run twice under different slot counts, step
budgets, portion sizes and pools (down to three tenths of what the requests need together, so that
requests are preempted): float32 greedy tokens are the plain implementation's, and a sampled
request's tokens do not depend on the scheduling."""
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import replay_helpers as rh
import tiny_models as tm

pytestmark = pytest.mark.gpu

CONFIGS = {"A": (tm.TINY_A, tm.TINY_A_PAGE, tm.TINY_A_SEED), "B": (tm.TINY_B, tm.TINY_B_PAGE, tm.TINY_B_SEED),
           "C": (tm.TINY_C, tm.TINY_C_PAGE, tm.TINY_C_SEED), "D": (tm.TINY_D, tm.TINY_D_PAGE, tm.TINY_D_SEED),
           "E": (tm.TINY_E, tm.TINY_E_PAGE, tm.TINY_E_SEED), "F": (tm.TINY_F, tm.TINY_F_PAGE, tm.TINY_F_SEED)}


def random_trace(reqs, rng, max_live):
    waiting = list(reqs.items())
    rng.shuffle(waiting)
    live, steps = [], []
    big = rng.choice((8, 40, 200, 700))
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            r, t = waiting.pop(0)
            live.append([r, t, 0, rng.choice((0, len(t) // 2, len(t) - 1, len(t)))])     # [3]: tokens after it go one by one
        entries, ended, nxt = [], [], []
        order = list(live)
        rng.shuffle(order)
        for item in order:
            r, t, at, plen = item
            if rng.random() < 0.2 and len(live) > 1:                                      # sits this step out
                nxt.append(item)
                continue
            n = min(rng.choice((1, 2, 3, 5, 15, 16, 17, 31, 33, 64, 127, 128, 129, big)), plen - at) if at < plen else 1
            mode = rng.random()
            want = (list(range(n)) if mode < 0.5 else [n - 1] if mode < 0.7 else
                    sorted(rng.sample(range(n), min(n, rng.randint(1, 4)))) if mode < 0.85 else [])
            entries.append({"id": r, "tokens": t[at:at + n], "want": want})
            item[2] = at + n
            if item[2] == len(t):
                ended.append(r)
            else:
                nxt.append(item)
        live = nxt
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_random_traces(name, dtype):
    cfg, page, wseed = CONFIGS[name]
    bf = dtype == "bfloat16"
    # the q-norm factor that keeps the plain code's own bfloat16 emulation within the bound at these
    # lengths (requests here are longer than in the fixed traces: 3 instead of 4 below head size 128)
    factor = 2.0 if cfg["head_dim"] == 128 else 3.0 if bf else 4.0
    w = rh.sharpen(tm.make_weights(cfg, wseed, bf16_exact=bf), factor, bf16_exact=bf)
    maxpos = cfg["max_position_embeddings"]
    for seed in range(3):
        rng = random.Random(seed * 7919 + ord(name) + (1 if bf else 0))
        lens = [rng.choice((2, 3, rng.randint(4, 40), rng.randint(40, min(maxpos, 400)), min(maxpos, rng.randint(100, 900))))
                for _ in range(rng.randint(2, 8))]
        reqs = {f"r{i}": tm.random_tokens(cfg, n, seed * 1000 + i) for i, n in enumerate(lens)}
        max_live = rng.randint(1, 4)
        steps = random_trace(reqs, rng, max_live)
        most = max(sum(len(e["tokens"]) for e in s["entries"]) for s in steps)
        runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=rh.peak_tokens(steps, max(64, page)),
                                max_requests=max_live, max_tokens_per_step=max(most, 16))
        runner.use_graphs = runner.use_graphs and rng.random() < 0.7
        got = rh.run_trace(runner, steps)
        ref = rh.plain_rows(cfg, w, reqs, dtype)
        rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"{name} {dtype} seed {seed} against the plain code")
        whole_runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=max(lens) + 2 * max(64, page), max_requests=1)
        whole = rh.run_trace(whole_runner, rh.trace_whole(reqs))
        scale = max(1.0, max(float(np.abs(v).max()) for v in ref.values()))
        tol = (rh.BF16_CUT_TOL if bf else rh.FP32_CUT_TOL) * scale
        for k in sorted(got):
            err = float(np.abs(got[k] - whole[k]).max())
            assert err <= tol, f"{name} {dtype} seed {seed}: {k} differs from the whole run by {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_random_generation_jobs(name):
    from litellmengine_b200.engine import PagedGenerateEngine
    cfg, page, wseed = CONFIGS[name]
    w = tm.make_weights(cfg, wseed)
    maxpos = cfg["max_position_embeddings"]
    for seed in range(4):
        rng = random.Random(seed * 31 + ord(name))
        n = rng.randint(1, 14)
        prompts = [tm.random_tokens(cfg, rng.choice((1, 2, rng.randint(3, 20), rng.randint(20, min(90, maxpos - 30)))), seed * 100 + i)
                   for i in range(n)]
        news = [rng.choice((1, 2, rng.randint(3, 24))) for _ in range(n)]
        temps = [rng.choice((0.0, 0.0, 0.7, 1.3)) for _ in range(n)]
        eos = rng.choice((-1, -1, rng.randrange(cfg["vocab_size"])))
        need = [-(-(len(p) + m) // page) * page for p, m in zip(prompts, news)]
        outs = []
        for _ in range(2):
            pool = max(max(need), int(sum(need) * rng.choice((0.3, 0.5, 0.8, 1.0)))) // page * page
            slots = rng.randint(1, 8)
            runner = rh.make_runner(cfg, w, "float32", page, max_total_tokens=pool, max_requests=slots,
                                    max_tokens_per_step=max(rng.choice((16, 64, 256, 1024)), slots))
            runner.use_graphs = runner.use_graphs and rng.random() < 0.7
            eng = PagedGenerateEngine(runner, chunk=rng.choice((None, 2, 3, 8, 32, 100)), pipelined=rng.random() < 0.7)
            ids = [eng.add_request(p, m, eos, t, 1000 + i) for i, (p, m, t) in enumerate(zip(prompts, news, temps))]
            for _ in range(20000):
                if not eng.has_work():
                    break
                eng.step()
            assert not eng.has_work(), "the job did not end"
            runner.check_status()
            runner.cache.check_invariants()
            assert all(g.pool.free_count == g.pool.num_pages for g in runner.cache.groups), "pages left behind"
            outs.append([list(eng.request(i).generated_ids) for i in ids])
        for i, (p, m, t) in enumerate(zip(prompts, news, temps)):
            a, b = outs[0][i], outs[1][i]
            assert len(a) == m or (eos >= 0 and a[-1] == eos), f"seed {seed} request {i}: {len(a)} tokens of {m}"
            if t > 0.0:
                assert a == b, f"seed {seed} request {i}: sampled tokens depend on the scheduling"
                continue
            ref = pq.greedy_generate(p, w, cfg, m, eos)
            for got in (a, b):
                if got == ref:
                    continue
                j = next(x for x in range(min(len(got), len(ref))) if got[x] != ref[x])
                lg = pq.forward_logits(list(p) + ref[:j], w, cfg, wd=torch.float64)[-1]
                gap = float(lg[ref[j]] - lg[got[j]])                       # a tie within float32 rounding is no fault
                assert gap < 1e-5, f"seed {seed} request {i} token {j}: {got[j]} for {ref[j]}, margin {gap:.2e}"
