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
