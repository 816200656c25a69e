"""bin/trace_run as a user runs it: a model folder written by the random-weights mode, steps on
standard input, `done <step>` lines and <step>.f32 files out, compared with the plain code."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_helpers as rh
import tiny_models as tm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_replays_a_mixed_trace(tmp_path, dtype):
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.weights import SafetensorsSource, write_random_model
    cfg = tm.TINY_C
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    model_dir = write_random_model(config_from_dict(cfg), str(tmp_path / "model"), seed=21, dtype=store)
    src = SafetensorsSource(model_dir)
    w = {n: src.get(n).float() for n in src.names()}
    reqs = rh.requests_for(cfg, [70, 33, 129, 64, 200], 3)
    steps = rh.trace_mixed(reqs, seed=2, max_live=4) 
    out_dir = str(tmp_path / "out")
    proc = subprocess.run(
        [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(rh.peak_tokens(steps, 64))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    got = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            got[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, cfg["vocab_size"])
        else:
            assert not os.path.exists(path)
    rows = rh.collect(steps, got)
    assert len(rows) == sum(len(t) for t in reqs.values())
    rh.assert_rows_match(rows, rh.plain_rows(cfg, w, reqs, dtype), rh.tol_for(dtype), f"trace_run {dtype}")


def test_trace_run_draws_random_weights_from_a_seed(tmp_path):
    """--random-weights --seed S over a folder that holds only config.json replays the same model as
    the folder the random-weights mode writes from seed S: the same logits, bit for bit."""
    import shutil
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.weights import write_random_model
    cfg = tm.TINY_A
    full = write_random_model(config_from_dict(cfg), str(tmp_path / "full"), seed=5, dtype=torch.float32)
    bare = tmp_path / "bare"
    bare.mkdir()
    shutil.copy(os.path.join(full, "config.json"), bare / "config.json")
    reqs = rh.requests_for(cfg, [9, 30], 8)
    steps = rh.trace_portions(reqs, 4)
    outs = []
    for folder, extra in ((full, []), (str(bare), ["--random-weights", "--seed", "5"])):
        out_dir = str(tmp_path / ("out" + str(len(outs))))
        proc = subprocess.run(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
             "--max-tokens", "128", "--page-size", "4"] + extra,
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        outs.append({f: np.fromfile(os.path.join(out_dir, f), dtype="<f4") for f in sorted(os.listdir(out_dir))})
    assert outs[0].keys() == outs[1].keys() and len(outs[0]) == len(steps)
    assert all(np.array_equal(outs[0][f], outs[1][f]) for f in outs[0])
