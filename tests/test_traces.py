"""The trace generators the GPU tests replay: every token of every request is fed exactly once,
in order; the mixed traces really mix and really keep several requests live (no GPU)."""
import replay_helpers as rh
import tiny_models as tm


def feeds(steps):
    fed, live, peak_live, mixed = {}, set(), 0, 0
    for s in steps:
        kinds = set()
        for e in s["entries"]:
            assert len(e["tokens"]) >= 1 and all(0 <= w < len(e["tokens"]) for w in e["want"])
            fed.setdefault(e["id"], []).extend(e["tokens"])
            live.add(e["id"])
            kinds.add(len(e["tokens"]) > 1)
        mixed += kinds == {True, False}
        peak_live = max(peak_live, len(live))
        for r in s["end"]:
            live.discard(r)
    assert not live
    return fed, peak_live, mixed


def test_generators_feed_every_token_once():
    reqs = rh.requests_for(tm.TINY_B, [1, 2, 3, 7, 16, 33, 70, 121], 1)
    for steps in (rh.trace_whole(reqs), rh.trace_tail_decode(reqs, 32), rh.trace_portions(reqs, 3),
                  rh.trace_mixed(reqs, 5, 4), rh.trace_mixed(reqs, 6, 3, 0.3)):
        fed, _, _ = feeds(steps)
        assert fed == reqs
        assert [s["step"] for s in steps] == list(range(len(steps)))
    _, peak_live, mixed = feeds(rh.trace_mixed(reqs, 5, 4))
    assert peak_live == 4 and mixed >= 5
    portions = rh.trace_portions({"x": list(range(100))}, 3)
    assert min(len(s["entries"][0]["tokens"]) for s in portions) == 2
    assert rh.peak_tokens(rh.trace_whole({"a": [1] * 65, "b": [1] * 3})) == 128


def test_replay_drives_only_the_step_function():
    """`engine.trace.replay` against a stand-in runner: a request is admitted when its id first
    appears, a step's entries go to `step` as one batch in their order, logits are handed on only
    when something was wanted, requests named in `end` are released after the step, a request may
    sit a step out, and a slot given back is used again."""
    import torch
    from litellmengine_b200.engine.trace import replay

    class Runner:
        def __init__(self):
            self.free, self.log = [2, 1, 0], []

        def admit(self):
            s = self.free.pop()
            self.log.append(("admit", s))
            return s

        def step(self, entries):
            self.log.append(("step", [(e.slot, list(e.tokens), list(e.want)) for e in entries]))
            return torch.zeros(sum(len(e.want) for e in entries), 5)

        def release(self, s):
            self.log.append(("release", s))
            self.free.append(s)

        def check_status(self):
            self.log.append(("check",))

    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": [1, 2], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": [9], "want": [0]}, {"id": "b", "tokens": [4], "want": [0]}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "c", "tokens": [7, 7], "want": [1]}], "end": ["b", "c", "nobody"]},
        {"step": 4, "entries": [], "end": []},
    ]
    r, wrote, done = Runner(), [], []
    replay(r, steps, lambda step, lg: wrote.append((step, tuple(lg.shape))), done.append)
    assert done == [0, 1, 2, 3, 4]
    assert wrote == [(0, (2, 5)), (2, (2, 5)), (3, (1, 5))]          # step 1 wanted nothing, step 4 ran nothing
    assert r.log == [
        ("admit", 0), ("step", [(0, [5, 17, 3], [0, 2])]), ("check",),
        ("admit", 1), ("step", [(1, [1, 2], [])]), ("check",),
        ("step", [(0, [9], [0]), (1, [4], [0])]), ("check",), ("release", 0),
        ("admit", 0), ("step", [(0, [7, 7], [1])]), ("check",), ("release", 1), ("release", 0),
    ]
