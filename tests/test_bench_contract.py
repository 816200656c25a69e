"""What `bench.py` promises before it touches a GPU: one line and exit code 2 for more than one
GPU, the `unavailable` line for the reference arm, peaks from MEASURED_PEAKS.json when that file
exists and the stated fallback when it does not."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(*argv):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], capture_output=True, text=True)


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["n_gpus"] == 2


def test_the_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


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
