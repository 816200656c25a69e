"""The plain implementation against the reference's own CPU code (golden logits made by
tests/golden/make_golden.py), and its parts against closed forms."""
import hashlib
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as pq
import tiny_models as tm

GOLD = os.path.join(os.path.dirname(__file__), "golden")
META = json.load(open(os.path.join(GOLD, "golden.json")))


def _digest(w):
    h = hashlib.sha256()
    for n in sorted(w):
        h.update(n.encode())
        h.update(w[n].numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name,cfg,seed", [("tiny_a", tm.TINY_A, tm.TINY_A_SEED), ("tiny_b", tm.TINY_B, tm.TINY_B_SEED)])
def test_plain_matches_reference_cpu_code(name, cfg, seed):
    w = tm.make_weights(cfg, seed)
    assert _digest(w) == META[name]["weights_sha256"], "tiny weights changed: remake the golden files"
    gold = np.fromfile(os.path.join(GOLD, f"{name}_logits.f32"), dtype="<f4").reshape(META[name]["shape"])
    ours = pq.forward_logits(META[name]["tokens"], w, cfg).numpy()
    assert np.abs(ours - gold).max() <= 2e-6 * max(1.0, np.abs(gold).max())


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, 4.0]])
    out = pq.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3.0 / r * 2.0, 4.0 / r * 0.5]]), atol=1e-6)


def test_rope_rotates_pairs_half_split():
    d = 4
    x = torch.zeros(1, 1, d)
    x[0, 0, 0] = 1.0                         # pair (0, 2)
    y = pq.rope(x, torch.tensor([3]), 10000.0)
    assert torch.allclose(y[0, 0], torch.tensor([math.cos(3.0), 0.0, math.sin(3.0), 0.0]), atol=1e-6)
    assert torch.allclose(pq.rope(x, torch.tensor([0]), 10000.0), x)


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = pq.causal_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0], atol=1e-6) and torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    k2, v2 = k.clone(), v.clone()
    k2[4], v2[4] = 7.0, -3.0                 # a later key must not change earlier outputs
    assert torch.allclose(pq.causal_attention(q, k2, v2)[:4], out[:4])
    w = pq.causal_attention(q, k, v, window=1)
    assert torch.allclose(w[:, 0], v[:, 0], atol=1e-6)


def test_argmax_ties_go_low():
    assert pq.argmax_token(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1


def test_greedy_stops_at_eos_and_keeps_it():
    cfg, w = tm.TINY_A, tm.make_weights(tm.TINY_A, 0)
    free = pq.greedy_generate([1, 2, 3], w, cfg, 6)
    assert len(free) == 6
    cut = pq.greedy_generate([1, 2, 3], w, cfg, 6, eos_token_id=free[2])
    assert cut == free[:free.index(free[2]) + 1]
