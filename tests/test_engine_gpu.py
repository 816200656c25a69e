"""The engine against the plain implementation, in float32 and in bfloat16, for every way of
cutting the work: whole, a tail decoded token by token, portions of changing size, and mixed
batches of up to four live requests over so few pages that they are used again."""
import numpy as np
import pytest
import torch

import replay_helpers as rh
import tiny_models as tm

pytestmark = pytest.mark.gpu

MODELS = {
    "A": (tm.TINY_A, tm.TINY_A_SEED, tm.TINY_A_PAGE),
    "B": (tm.TINY_B, tm.TINY_B_SEED, tm.TINY_B_PAGE),
    "C": (tm.TINY_C, tm.TINY_C_SEED, tm.TINY_C_PAGE),
    "D": (tm.TINY_D, tm.TINY_D_SEED, tm.TINY_D_PAGE),
    "E": (tm.TINY_E, tm.TINY_E_SEED, tm.TINY_E_PAGE),
    "F": (tm.TINY_F, tm.TINY_F_SEED, tm.TINY_F_PAGE),
}
LENGTHS = {"A": [5, 9, 13, 40, 77], "B": [1, 7, 16, 33, 70, 121], "C": [64, 97, 150, 333],
           "D": [2, 63, 64, 65, 129, 200, 333, 700], "E": [2, 64, 127, 128, 129, 200, 333, 700],
           "F": [3, 65, 130, 257, 500]}


# Factor on the q-norm weights.  Head size 128 gets a smaller one: with 4 the plain code's own
# bfloat16 emulation is 3e-2 (E) and 5e-2 (F) of the largest logit away from exact arithmetic, against
# 1.6e-2 for D, and a comparison at 1e-2 would only measure on which side single roundings fall (the
# worst positions are then scattered decoded tokens, a different one for each way of cutting).  With 2
# the emulation's own error is 9e-3 and 7e-3.
SHARPEN = {"A": 4.0, "B": 4.0, "C": 4.0, "D": 4.0, "E": 2.0, "F": 2.0}


def setup(name, dtype, sharp=True):
    cfg, seed, page = MODELS[name]
    bf = dtype == "bfloat16"
    w = tm.make_weights(cfg, seed, bf16_exact=bf)
    if sharp:
        w = rh.sharpen(w, SHARPEN[name], bf16_exact=bf)
    reqs = rh.requests_for(cfg, LENGTHS[name], seed)
    return cfg, page, w, reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_every_way_of_cutting_matches_the_plain_implementation(name, dtype):
    cfg, page, w, reqs = setup(name, dtype)
    ref = rh.plain_rows(cfg, w, reqs, dtype)
    longest = max(len(t) for t in reqs.values())
    traces = {
        "whole": rh.trace_whole(reqs),
        "tail": rh.trace_tail_decode(reqs, 32),
        "portions": rh.trace_portions(reqs, seed=3),
        "mixed": rh.trace_mixed(reqs, seed=5, max_live=4),
        "mixed2": rh.trace_mixed(reqs, seed=6, max_live=3, prompt_frac=0.3),
    }
    results = {}
    for what, steps in traces.items():
        pool = rh.peak_tokens(steps, round_to=page)               # exactly enough: pages must be reused
        runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=pool, max_requests=4,
                                max_tokens_per_step=max(longest, 64))
        got = rh.run_trace(runner, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"{name} {dtype} {what}")
        results[what] = got
    cut_tol = rh.FP32_CUT_TOL if dtype == "float32" else rh.BF16_CUT_TOL
    whole = {r: np.stack([results["whole"][(r, p)] for p in range(len(t))]) for r, t in reqs.items()}
    for what in ("tail", "portions", "mixed", "mixed2"):
        rh.assert_rows_match(results[what], whole, cut_tol, f"{name} {dtype} {what} against whole")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_bfloat16_against_the_plain_float32_code(name):
    """Unsharpened N(0, 0.02) weights, bfloat16 run, plain code in float32 without any rounding."""
    cfg, page, w, reqs = setup(name, "bfloat16", sharp=False)
    ref = rh.plain_rows(cfg, w, reqs, "float32")
    for steps in (rh.trace_whole(reqs), rh.trace_mixed(reqs, seed=8, max_live=4)):
        runner = rh.make_runner(cfg, w, "bfloat16", page, max_total_tokens=rh.peak_tokens(steps, page),
                                max_tokens_per_step=1024)
        rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.BF16_VS_FP32_TOL, f"{name} bf16 vs fp32 plain")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [4, 8, 16, 64])
def test_other_page_sizes(page, dtype):
    cfg, _, w, reqs = setup("B", dtype)
    ref = rh.plain_rows(cfg, w, reqs, dtype)
    steps = rh.trace_mixed(reqs, seed=11, max_live=4)
    runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=rh.peak_tokens(steps, page), max_tokens_per_step=256)
    rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.tol_for(dtype), f"page {page}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """Three tokens of prompt, then 400 tokens one by one: every page edge is crossed by a
    single-token step, and the first tokens of the sequence are decoded too."""
    cfg, page, w, _ = setup("D" if dtype == "bfloat16" else "C", dtype)
    toks = tm.random_tokens(cfg, 403, 77)
    ref = rh.plain_rows(cfg, w, {"x": toks}, dtype)
    steps = rh.trace_tail_decode({"x": toks}, tail=400)
    runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=rh.peak_tokens(steps, page))
    rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.tol_for(dtype), "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype):
    """Lengths 1, 2, 3 and a request fed entirely one token at a time from position 0."""
    cfg, page, w, _ = setup("A", dtype)
    reqs = {f"s{n}": tm.random_tokens(cfg, n, 900 + n) for n in (1, 2, 3, 6)}
    ref = rh.plain_rows(cfg, w, reqs, dtype)
    for steps in (rh.trace_whole(reqs), rh.trace_tail_decode(reqs, tail=64)):
        runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=64)
        rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.tol_for(dtype), "first tokens")


def test_logits_only_where_wanted_and_a_step_may_want_nothing():
    cfg, page, w, _ = setup("B", "float32")
    toks = tm.random_tokens(cfg, 30, 5)
    ref = rh.plain_rows(cfg, w, {"x": toks})["x"]
    runner = rh.make_runner(cfg, w, "float32", page, max_total_tokens=64)
    from litellmengine_b200.engine import StepEntry
    s = runner.admit()
    out = runner.step([StepEntry(s, toks[:20], [])])
    assert out.shape == (0, cfg["vocab_size"])
    out = runner.step([StepEntry(s, toks[20:], [9, 0, 3])]).cpu().numpy()
    assert out.shape == (3, cfg["vocab_size"])
    for row, pos in zip(out, (29, 20, 23)):
        assert np.abs(row - ref[pos]).max() <= rh.FP32_TOL
    runner.release(s)


def test_step_refuses_bad_input_without_launching():
    from litellmengine_b200.cache import OutOfPages
    from litellmengine_b200.engine import StepEntry
    cfg, page, w, _ = setup("A", "float32")
    runner = rh.make_runner(cfg, w, "float32", page, max_total_tokens=16, max_requests=2)
    s = runner.admit()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        runner.step([StepEntry(s, [1, cfg["vocab_size"]], [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry(s, list(range(17)), [])])
    with pytest.raises(ValueError, match="twice"):
        runner.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    assert runner.cache.length(s) == 0
    runner.step([StepEntry(s, list(range(16)), [15])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry(s, [3], [0])])
    runner.release(s)
    runner.check_status()
    runner.cache.check_invariants()


def test_a_status_code_in_either_word_is_raised_and_cleared():
    """Kernels record a refused index or a wait that ran out in the step's status word; the engine's
    matrix products record theirs in a word of their own.  `check_status` reads both.  The codes are
    written from the host here: nothing on the device is made to fail."""
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.engine.runner import STATUS_TEXT
    cfg, page, w, _ = setup("A", "float32")
    runner = rh.make_runner(cfg, w, "float32", page, max_total_tokens=16, max_requests=2)
    assert set(STATUS_TEXT) == {1, 2, 3, 4, 5, 6, 8, 9}
    for word, code in ((runner.buffers.status, 4), (ops.stream_status(runner.device), 8),
                       (ops.stream_status(runner.device), 9), (runner.buffers.status, 6)):
        word.copy_(torch.tensor([code, 123], dtype=torch.int32))
        with pytest.raises(RuntimeError, match=f"device status {code}: .*index 123"):
            runner.check_status()
        runner.check_status()                                   # cleared by the raise


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_as_graphs_match_kernel_by_kernel_launches(dtype):
    """Steps made only of single decoded tokens are replayed as CUDA graphs from the third step of
    a batch size on.  Same trace with graphs off: same logits up to rounding (the graph of a mixed
    step chooses its key splits for the most single tokens such a step could hold, the plain
    launches for those it has)."""
    cfg, page, w, _ = setup("D", dtype)
    reqs = rh.requests_for(cfg, [90, 41, 140], 5)
    ref = rh.plain_rows(cfg, w, reqs, dtype)
    steps = rh.trace_mixed(reqs, seed=4, max_live=3, prompt_frac=0.2)
    got = {}
    for graphs in (True, False):
        from litellmengine_b200.config import config_from_dict
        from litellmengine_b200.engine import ModelRunner
        from litellmengine_b200.weights import DictSource
        store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        runner = ModelRunner.from_config(
            config_from_dict(cfg), dtype=dtype, device="cuda:0", page_size=page, max_total_tokens=512,
            max_requests=4, max_tokens_per_step=256, use_graphs=graphs,
            source=DictSource({k: (v.to(store) if v.dim() == 2 else v) for k, v in w.items()}))
        got[graphs] = rh.run_trace(runner, steps)
        rh.assert_rows_match(got[graphs], ref, rh.tol_for(dtype), f"graphs={graphs}")
        assert (runner.graph_replays > 20) == graphs
    worst = max(float(np.abs(got[True][k] - got[False][k]).max()) for k in got[True])
    assert worst <= rh.tol_for(dtype)


def test_graphs_follow_the_key_splits_as_a_context_grows():
    """One request decoding from 200 to 1,300 tokens with head size 128 in bfloat16: the decode
    kernel's key splits grow with the context (4, 6, 8 by 1,300 keys), a captured graph holds its
    number of splits, so the graph's key carries it and a step whose length asks for another number
    is captured anew.  Every decoded position against the plain code, and bit for bit against the same
    trace launched kernel by kernel: graph or not, a step makes the same choices."""
    cfg, page, w, _ = setup("E", "bfloat16")
    reqs = {"r0": tm.random_tokens(cfg, 1300, 91)}
    ref = rh.plain_rows(cfg, w, reqs, "bfloat16")
    steps = rh.trace_tail_decode(reqs, 1100)
    got = {}
    for graphs in (True, False):
        runner = rh.make_runner(cfg, w, "bfloat16", page, max_total_tokens=1344, max_requests=1, max_tokens_per_step=256)
        runner.use_graphs = runner.use_graphs and graphs
        got[graphs] = rh.run_trace(runner, steps)
        rh.assert_rows_match(got[graphs], ref, rh.BF16_TOL, f"growing context, graphs={graphs}")
        if graphs:
            splits = sorted({k[-1][0] for k in runner._graphs if k[1] == "decode"})
            assert splits == [4, 6, 8], splits
            assert runner.graph_replays >= 1100 - 2 * len(splits)
    decoded = [k for k in got[True] if k[1] >= 200]
    assert len(decoded) == 1100 and all(np.array_equal(got[True][k], got[False][k]) for k in decoded)


def test_one_layer_at_real_widths():
    """Hidden 4096, 32/8 heads of 128, intermediate 12288, one layer, bfloat16: the engine's products
    (k-splits, partial sums, tiled weight copies), the TMA decode attention and the tcgen05 prompt
    attention at the sizes they are tuned for, whole and mixed, against the plain code."""
    cfg, seed, page = tm.WIDE_G, tm.WIDE_G_SEED, tm.WIDE_G_PAGE
    w = tm.make_weights(cfg, seed, bf16_exact=True, matrix_std=0.02)
    reqs = rh.requests_for(cfg, [3, 70, 150], seed)
    ref = rh.plain_rows(cfg, w, reqs, "bfloat16")
    for what, steps in (("whole", rh.trace_whole(reqs)), ("mixed", rh.trace_mixed(reqs, seed=2, max_live=3, prompt_frac=0.4))):
        runner = rh.make_runner(cfg, w, "bfloat16", page, max_total_tokens=rh.peak_tokens(steps, page), max_requests=4,
                                max_tokens_per_step=256)
        rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.BF16_TOL, f"wide {what}")


@pytest.mark.parametrize("policy", ["all", "off"])
def test_prompt_portions_through_the_paired_product(policy, monkeypatch):
    """Portions of 129 tokens and more in bfloat16 with every product they allow forced through the
    paired tcgen05 kernel (the activation in the gate/up product's epilogue, the attention's and the
    feed-forward's last products added to the residual where it lies), and with that kernel off:
    both against the plain code, whole and cut into portions that are no multiple of its tiles."""
    from litellmengine_b200.csrc import ops
    monkeypatch.setattr(ops, "_PAIR_POLICY", policy)
    before = ops.launch_count
    for cfg, seed, page, lens in ((tm.TINY_E, tm.TINY_E_SEED, tm.TINY_E_PAGE, [300, 140]),
                                  (tm.WIDE_G, tm.WIDE_G_SEED, tm.WIDE_G_PAGE, [260, 131])):
        w = tm.make_weights(cfg, seed, bf16_exact=True, matrix_std=0.02)
        reqs = rh.requests_for(cfg, lens, seed)
        ref = rh.plain_rows(cfg, w, reqs, "bfloat16")
        for what, steps in (("whole", rh.trace_whole(reqs)), ("portions", rh.trace_portions(reqs, seed=5, sizes=(129, 133, 170)))):
            runner = rh.make_runner(cfg, w, "bfloat16", page, max_total_tokens=rh.peak_tokens(steps, page), max_requests=4,
                                    max_tokens_per_step=512)
            rh.assert_rows_match(rh.run_trace(runner, steps), ref, rh.BF16_TOL, f"paired product {policy} {what}")
    assert ops.launch_count > before
    if policy == "all":
        assert any("gemm_pair_tcgen05" in name for name in ops.loaded_libraries())



@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_one_size_divided_differently_replay_one_graph(dtype):
    """A step that is not all single decoded tokens is captured, the second time its number of tokens is
    seen, as a graph for ANY step of that many tokens: the attention kernels run over work lists padded
    with entries that mean "nothing".  Steps of 24 tokens divided among one to four requests in seven
    different ways (a whole portion; portions beside decoded tokens; decoded tokens that want nothing),
    each wanting at most one row per request: same logits as the plain code, and as with graphs off."""
    from litellmengine_b200.engine import StepEntry
    cfg, page, w, _ = setup("E", dtype)
    reqs = rh.requests_for(cfg, [200, 170, 150, 90], 77)
    ref = rh.plain_rows(cfg, w, reqs, dtype)
    names = list(reqs)
    cuts = [[24], [20, 4], [1, 23], [12, 1, 11], [1, 1, 22], [6, 6, 6, 6], [1, 1, 1, 21], [24], [2, 22], [13, 11]]
    results = {}
    for graphs in (True, False):
        runner = rh.make_runner(cfg, w, dtype, page, max_total_tokens=1024, max_requests=4, max_tokens_per_step=64)
        runner.use_graphs = runner.use_graphs and graphs
        slots = {r: runner.admit() for r in names}
        at = {r: 0 for r in names}
        got = {}
        for step, cut in enumerate(cuts):
            order = names[step % 4:] + names[:step % 4]               # who gets which share changes too
            entries, wanted = [], []
            for r, n in zip(order, cut):
                want = [n - 1] if (step + n) % 3 else []                # some entries want nothing
                entries.append(StepEntry(slots[r], reqs[r][at[r]:at[r] + n], want))
                if want:
                    wanted.append((r, at[r] + n - 1))
                at[r] += n
            logits = runner.step(entries).float().cpu().numpy()
            assert logits.shape[0] == len(wanted)
            for (r, pos), row in zip(wanted, logits):
                got[(r, pos)] = row
        runner.check_status()
        kinds = {k[1] for k in runner._graphs}
        assert all(k[3] == 0 for k in runner._graphs if k[1] != "decode")   # one graph whatever the number of entries
        assert (("any" in kinds) and runner.graph_replays >= 6) if graphs else runner.graph_replays == 0
        rh.assert_rows_match(got, ref, rh.tol_for(dtype), f"24-token steps, graphs {graphs}")
        results[graphs] = got
    assert results[True].keys() == results[False].keys()
