"""Generation through the Python entry point and the command line: greedy tokens equal the
plain implementation's, sampling is reproducible and follows its streams, page pressure
changes nothing but the schedule."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import replay_helpers as rh
import tiny_models as tm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine_for(cfg, w, dtype, page, pool, **kw):
    from litellmengine_b200.engine import PagedGenerateEngine
    runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=pool, max_requests=kw.pop("max_requests", 4),
                            max_tokens_per_step=kw.pop("max_tokens_per_step", 64))
    return PagedGenerateEngine(runner, **kw)


def test_greedy_generation_config_a_float32():
    """Tiny configuration A: prompts of 5, 9 and 13 tokens, 8 greedy steps each, page size 4."""
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, tm.TINY_A_SEED)
    prompts = [tm.random_tokens(cfg, n, 40 + n) for n in (5, 9, 13)]
    eng = engine_for(cfg, w, "float32", tm.TINY_A_PAGE, pool=96)
    got = eng.generate(prompts, max_new_tokens=8)
    assert got == [pq.greedy_generate(p, w, cfg, 8) for p in prompts]
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.free_slots == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_chunked_and_mixed(dtype):
    """Tiny configuration B: prompts of 1, 7, 16 and 33 tokens, prefilled in
    portions of 6 beside decoding requests.  A bfloat16 run may differ from the plain code only
    where the two best logits are closer than bfloat16 resolves."""
    cfg = tm.TINY_B
    bf = dtype == "bfloat16"
    w = tm.make_weights(cfg, tm.TINY_B_SEED, bf16_exact=bf)
    prompts = [tm.random_tokens(cfg, n, 60 + n) for n in (1, 7, 16, 33)]
    eng = engine_for(cfg, w, dtype, tm.TINY_B_PAGE, pool=256, chunk=6, max_tokens_per_step=16)
    got = eng.generate(prompts, max_new_tokens=12)
    act = pq.to_bf16 if bf else pq.identity
    for p, new in zip(prompts, got):
        assert len(new) == 12
        ids = list(p)
        for t in new:
            lg = pq.forward_logits(ids, w, cfg, act=act)[-1]
            best = pq.argmax_token(lg)
            if t != best:
                assert bf and float(lg[best] - lg[t]) < 2e-2, f"token {t} instead of {best}"
            ids.append(t)


def test_eos_and_release_and_reference_surface():
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, tm.TINY_A_SEED)
    prompt = tm.random_tokens(cfg, 7, 1)
    free = pq.greedy_generate(prompt, w, cfg, 8)
    eng = engine_for(cfg, w, "float32", 4, pool=64)
    rid = eng.add_request(prompt, 8, eos_token_id=free[3])
    out = eng.generate_until_finished(rid)
    stop = free.index(free[3])
    assert out == prompt + free[:stop + 1] and eng.finished(rid)
    assert eng.request(rid).finish_reason == "eos"
    eng.release_request(rid)
    with pytest.raises(KeyError):
        eng.request(rid)
    z = eng.add_request(prompt, 0)
    assert eng.finished(z) and eng.generate_until_finished(z) == prompt
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.runner.cache.groups)


def test_page_pressure_preempts_and_results_do_not_change():
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, tm.TINY_A_SEED)
    prompts = [tm.random_tokens(cfg, 10, 200 + i) for i in range(4)]
    want = [pq.greedy_generate(p, w, cfg, 14) for p in prompts]
    roomy = engine_for(cfg, w, "float32", 4, pool=256)
    assert roomy.generate(prompts, 14) == want and roomy.scheduler.num_preemptions == 0
    tight = engine_for(cfg, w, "float32", 4, pool=48)          # 12 pages for 4 requests of up to 23 tokens
    assert tight.generate(prompts, 14) == want
    assert tight.scheduler.num_preemptions > 0
    tight.runner.cache.check_invariants()


def test_pipelined_and_unpipelined_stepping_give_the_same_tokens():
    """Launching a step before the tokens of the one before are read changes nothing but the
    timing: greedy and sampling requests, an end-of-sequence token found one step late, so few
    pages that requests are preempted with a token still on the device."""
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, tm.TINY_A_SEED)
    prompts = [tm.random_tokens(cfg, n, 300 + n) for n in (10, 3, 12, 7, 9)]
    free = [pq.greedy_generate(p, w, cfg, 14) for p in prompts]
    eos = free[1][4]

    def run(pipelined, pool):
        eng = engine_for(cfg, w, "float32", 4, pool=pool, pipelined=pipelined, chunk=5, max_tokens_per_step=12)
        ids = [eng.add_request(p, 14, eos_token_id=eos if i == 1 else -1, temperature=0.7 if i == 3 else 0.0,
                               seed=50 + i) for i, p in enumerate(prompts)]
        steps = 0
        while eng.has_work():
            eng.step()
            steps += 1
            assert steps < 2000
        eng.runner.check_status()
        eng.runner.cache.check_invariants()
        assert all(g.pool.free_count == g.pool.num_pages for g in eng.runner.cache.groups)
        return [eng.request(i).generated_ids for i in ids], [eng.request(i).finish_reason for i in ids], eng

    want, why, _ = run(False, 256)
    assert why[1] == "eos" and want[1] == free[1][:free[1].index(eos) + 1] and want[0] == free[0]
    for pool in (256, 48):
        got, why2, eng = run(True, pool)
        assert got == want and why2 == why
        assert (eng.scheduler.num_preemptions > 0) == (pool == 48)


@pytest.mark.parametrize("seed", [0, 1])
def test_many_requests_arriving_over_time_under_page_pressure(seed):
    """Forty greedy requests of random lengths, added a few at a time while others run, some ending
    at an end-of-sequence token, in a cache too small for all of them (preemptions) and with
    pipelined steps: every request's tokens are those of the plain implementation run alone."""
    import random
    rng = random.Random(seed)
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, tm.TINY_A_SEED)
    jobs = []
    for i in range(40):
        prompt = tm.random_tokens(cfg, rng.randint(1, 30), 500 + 40 * seed + i)
        n_new = rng.randint(1, 20)
        free = pq.greedy_generate(prompt, w, cfg, n_new)
        eos = free[rng.randrange(len(free))] if rng.random() < 0.3 else -1
        want = free[:free.index(eos) + 1] if eos >= 0 else free
        jobs.append((prompt, n_new, eos, want))
    eng = engine_for(cfg, w, "float32", 4, pool=96, max_requests=6, chunk=rng.choice([3, 7, 16]), max_tokens_per_step=24)
    ids, pending, steps = [], list(range(len(jobs))), 0
    while pending or eng.has_work():
        for _ in range(rng.randint(0, 3)):
            if pending:
                j = pending.pop(0)
                ids.append((j, eng.add_request(jobs[j][0], jobs[j][1], eos_token_id=jobs[j][2])))
        if eng.has_work():
            eng.step()
        steps += 1
        assert steps < 5000
    eng.runner.check_status()
    for j, rid in ids:
        assert eng.request(rid).generated_ids == jobs[j][3], f"request {j}"
    assert eng.scheduler.num_preemptions > 0
    eng.runner.cache.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.runner.cache.groups)


def test_temperature_sampling_is_reproducible_and_batch_independent():
    """Tiny configuration B: 12 sampling steps at temperature 0.8 with a fixed seed."""
    from litellmengine_b200.csrc import ops
    cfg, w = tm.TINY_B, tm.make_weights(tm.TINY_B, tm.TINY_B_SEED)
    prompts = [tm.random_tokens(cfg, n, 80 + n) for n in (1, 7, 16, 33)]

    def run(batch, **kw):
        eng = engine_for(cfg, w, "float32", 8, pool=256, **kw)
        ids = [eng.add_request(p, 12, temperature=0.8, seed=1000 + i) for i, p in batch]
        eng.run()
        return {i: eng.request(r).generated_ids for (i, _), r in zip(batch, ids)}
    together = run(list(enumerate(prompts)), chunk=6, max_tokens_per_step=16)
    again = run(list(enumerate(prompts)), chunk=6, max_tokens_per_step=16)
    assert together == again
    alone = {}
    for i, p in enumerate(prompts):
        alone.update(run([(i, p)]))
    assert alone == together                                # a request's stream is its own
    greedy = run(list(enumerate(prompts)))
    assert any(together[i] != pq.greedy_generate(p, w, cfg, 12) for i, p in enumerate(prompts))
    for i, p in enumerate(prompts):                         # every token sits where u falls in the plain CDF
        ids = list(p)
        for n, t in enumerate(together[i]):
            prob = pq.temperature_probs(pq.forward_logits(ids, w, cfg)[-1], 0.8).double()
            cdf = torch.cumsum(prob, 0)
            u = ops.sampler_uniform(1000 + i, n)
            lo = float(cdf[t - 1]) if t > 0 else 0.0
            assert lo - 1e-5 <= u <= float(cdf[t]) + 1e-5
            ids.append(t)


def test_command_line_and_run_prompt(tmp_path):
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.weights import write_random_model
    cfg = config_from_dict(tm.TINY_B)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=9, dtype=torch.float32)
    from litellmengine_b200.weights import SafetensorsSource
    src = SafetensorsSource(d)
    w = {n: src.get(n).clone() for n in src.names()}
    prompt = tm.random_tokens(tm.TINY_B, 6, 4)
    want = pq.greedy_generate(prompt, w, tm.TINY_B, 5)
    ids = ",".join(map(str, prompt))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "litellmengine"), "--model", d, "--input-ids", ids,
                        "--max-tokens=5", "--temperature", "0", "--dtype", "float32", "--page-size", "8"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    gen = lines[lines.index("Generated token ids:") + 1].strip()
    new = lines[lines.index("New token ids:") + 1].strip()
    assert new == ",".join(map(str, want)) and gen == ids + "," + new
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_prompt"), "--model", d, "--input-ids", ids,
                        "--max-tokens", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().splitlines()[-1] == ",".join(map(str, want)), r.stdout + r.stderr
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "litellmengine"), "--model", d, "--input-ids", "1,x"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "Invalid token id: x" in r.stderr and "Usage:" in r.stderr


def test_dropping_the_tiled_weight_copies_keeps_generation_right():
    """The second, tiled copies of the decode weights go when the cache needs their room: captured
    graphs that point at them are dropped with them, and the same tokens come out through the
    plain weight layout."""
    from litellmengine_b200.csrc import ops
    cfg, seed, page = tm.TINY_E, tm.TINY_E_SEED, tm.TINY_E_PAGE
    w = tm.make_weights(cfg, seed, bf16_exact=True)
    engine = engine_for(cfg, w, "bfloat16", page, 1024, max_tokens_per_step=256)
    runner = engine.runner
    prompts = [tm.random_tokens(cfg, n, 40 + n) for n in (5, 31, 64)]
    first = engine.generate(prompts, max_new_tokens=24)
    assert runner.graph_replays > 0 and len(ops._tiled) > 0
    replays = runner.graph_replays
    assert ops.release_streaming() > 0 and len(ops._tiled) == 0
    again = engine.generate(prompts, max_new_tokens=24)
    assert again == first
    assert runner.graph_replays > replays                   # captured anew, without the copies
    runner.check_status()
