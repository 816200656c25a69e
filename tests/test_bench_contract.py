"""What `bench.py` promises: one line and exit code 2 for more than one GPU; a reference arm that
prints either the contract's keys or one `unavailable` line with the reason; peaks from
MEASURED_PEAKS.json when that file exists and the stated fallback when it does not."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(*argv):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], capture_output=True, text=True)


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["n_gpus"] == 2


def test_the_reference_arm_without_a_gpu_is_one_line_with_the_reason():
    """Here the reference's engine cannot run (it needs a CUDA device, or its sources are not at
    hand): the arm still exits 0 with one JSON line."""
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3", "--layers", "1", "--no-points")
    assert r.returncode == 0
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    d = json.loads(lines[-1])
    assert len(lines) == 1 and d["impl"] == "reference"
    if "unavailable" in d:
        assert isinstance(d["unavailable"], str) and d["unavailable"] and "\n" not in d["unavailable"]
    else:
        assert d["value"] > 0


@pytest.mark.gpu
def test_the_reference_arm_times_the_reference_engine():
    """One layer of the benchmark's shape through the unmodified reference: the line has the
    contract's keys, float32 as its dtype, and an end-to-end figure of its own."""
    r = run("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "3", "--layers", "1", "--no-points")
    assert r.returncode == 0, r.stderr[-400:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference"
    if "unavailable" in d and "no checkout of the reference" in d["unavailable"]:
        pytest.skip("the reference's sources are not on this machine")
    assert "unavailable" not in d, d
    assert d["dtype"] == "fp32" and d["n_gpus"] == 1 and d["steps"] == 3 and d["unit"] == "tokens/s"
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["e2e"]["value"] > 0
    assert d["e2e"]["value"] <= d["value"] * 1.05                 # the wall clock holds the device time
    assert d["config"]["layers"] == 1 and d["config"]["layers_full"] == 36 and d["config"]["global_batch"] == 8
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] >= 32


def test_peaks_come_from_the_measured_file_or_the_fallback(tmp_path, monkeypatch):
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    p = bench.peaks()
    assert p["source"] == "fallback" and p["hbm_gbs"] == 6650.0 and p["bf16_tflops"] == 1590.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 7012.5, "bf16_tflops": {"value": 1622.0, "clock_mhz": 1900}, "bf16_tflops_sustained": 0}))
    p = bench.peaks()
    assert p["source"] == "measured" and p["hbm_gbs"] == 7012.5 and p["bf16_tflops"] == 1622.0
    assert p["bf16_tflops_sustained"] == 1400.0              # a figure that is no positive number keeps the fallback
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.peaks()["source"] == "fallback"


def test_the_default_shape_is_the_one_the_baseline_names():
    import bench
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        base = json.load(f)
    text = json.dumps(base)
    q = bench.QWEN3_8B
    assert (q["num_hidden_layers"], q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"]) == (36, 4096, 32, 8)
    assert (q["head_dim"], q["intermediate_size"], q["vocab_size"]) == (128, 12288, 151936)
    assert "8B" in text and bench.CONTEXT == 4096 and bench.PREFILL_TOKENS == 2048
