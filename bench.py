#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens/s (the headline), prefill tokens/s at
2,048 tokens, the same decode measured end to end through the Python entry point, and the
fraction of the memory roofline the decode step reaches.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

The model has the layer sizes of Qwen3-8B (36 layers unless --layers says fewer; the JSON names
both numbers), random bfloat16 weights drawn on the device, synthetic uniform-random token ids,
page size 16.  A "step" is one decode step of `batch` requests whose context ends at 4,096
tokens.  Prints ONE JSON line.  For --gpus > 1 it prints one line saying so and exits 2: the
engine runs on one GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
    tie_word_embeddings=False, torch_dtype="bfloat16")
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                v = d.get(k)
                if isinstance(v, dict):
                    v = v.get("value")
                if isinstance(v, (int, float)) and v > 0:
                    out[k] = float(v)
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc, self.lines, self.index = None, [], index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 decode points")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++ project that pip cannot install (no setup.py or "
                          "pyproject.toml); its binary also needs converted real weights and an absent submodule"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not built", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.engine import ModelRunner, PagedGenerateEngine, StepEntry

    pk = peaks()
    cfg_d = dict(QWEN3_8B, num_hidden_layers=args.layers)
    config = config_from_dict(cfg_d)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    gen = torch.Generator().manual_seed(2)

    def tokens(n):
        return torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()

    torch.cuda.set_device(0)
    runner = ModelRunner.from_config(config, seed=2, dtype="bfloat16", device="cuda:0", page_size=PAGE,
                                     max_total_tokens=max_batch * CONTEXT + 64, max_requests=max_batch,
                                     max_tokens_per_step=max(CONTEXT, PREFILL_TOKENS))
    weight_bytes = runner.model.weight_bytes()
    kv_bytes_per_token = runner.cache.bytes_per_token()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill: one 2,048-token prompt, logits at its last token --------------------------------
    def prefill_once():
        s = runner.admit()
        runner.step([StepEntry(s, tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
        runner.release(s)
    for _ in range(3):
        prefill_once()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(reps):
        prefill_once()
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1) / reps
    p = config
    T = PREFILL_TOKENS
    per_layer = 2 * T * p.hidden_size * ((p.num_attention_heads + 2 * p.num_key_value_heads) * p.head_dim
                                          + p.num_attention_heads * p.head_dim + 3 * p.intermediate_size)
    attn = 2 * 2 * p.num_attention_heads * p.head_dim * (T * (T + 1) // 2)
    prefill_flops = args.layers * (per_layer + attn) + 2 * p.hidden_size * p.vocab_size
    prefill = {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode: B requests whose context ends at CONTEXT ------------------------------------------
    def fill(batch, n_steps):
        """Admit `batch` requests and prefill each so that n_steps decode steps end at CONTEXT."""
        slots = []
        for _ in range(batch):
            s = runner.admit()
            runner.step([StepEntry(s, tokens(CONTEXT - n_steps), [])])
            slots.append(s)
        return slots

    def decode_device_timed(batch, steps, warmup, sample_clocks=False):
        slots = fill(batch, steps + warmup)
        feed = [tokens(batch) for _ in range(steps + warmup)]
        for i in range(warmup):
            lg = runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
        launches0 = ops.launch_count
        a, b = ev(), ev()
        a.record()
        for i in range(warmup, warmup + steps):
            lg = runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        launches = ops.launch_count - launches0
        ck = clocks.stop() if clocks else None
        ctx_mid = CONTEXT - steps // 2
        for s in slots:
            runner.release(s)
        return ms, launches, ck, ctx_mid

    ms, launches, clocks, ctx_mid = decode_device_timed(args.batch, args.steps, args.warmup, sample_clocks=True)
    value = args.batch / (ms * 1e-3)
    step_bytes = weight_bytes + kv_bytes_per_token * ctx_mid * args.batch
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]}

    # ---- the same through the Python entry point: host token ids in, host token ids out ------------
    engine = PagedGenerateEngine(runner)
    # Prompts are prefilled one per step, so the first request decodes a few tokens before the
    # last one starts: leave room for that, so that all of them still decode in the timed steps.
    n_new = args.steps + args.warmup + args.batch
    ids = [engine.add_request(tokens(CONTEXT - n_new), n_new + 8) for _ in range(args.batch)]
    while any(engine.request(i).cached_len < engine.request(i).prompt_len for i in ids):
        engine.step()                                    # prompts (and the first sampled tokens)
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(args.steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    assert produced == args.steps * args.batch, "a request left the batch inside the timed steps"
    for i in ids:
        engine.release_request(i)
    e2e = {"value": round(produced / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.buffers.last.size * 4, "d2h_bytes_per_step": args.batch * 4}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            st = max(8, min(args.steps, 32))
            pms, _, _, _ = decode_device_timed(b, st, 3)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)

    out = {
        "metric": "decode tokens/s (Qwen3-8B shape, batch %d, context %d)" % (args.batch, CONTEXT),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform-random token ids)",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden": p.hidden_size, "heads": p.num_attention_heads, "kv_heads": p.num_key_value_heads,
                   "head_dim": p.head_dim, "intermediate": p.intermediate_size, "vocab": p.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (the step reads every weight)"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "gpu_launches": launches,
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
