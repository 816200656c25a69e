#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
                    [--impl ours|reference] [--points LIST | --no-points]

Headline (`value`): decode tokens/s of `batch` requests whose context ends at 4,096 tokens, on a
model with the layer sizes of Qwen3-8B (36 layers unless --layers says fewer; the JSON names both
numbers), random bfloat16 weights drawn on the device, uniform-random token ids, page size 16.  A
"step" is one decode step.  Before the line is printed, the logits of the last timed step are
compared with the same positions recomputed as whole prompts (`checked`); a mismatch exits 1, and a
mismatch of the float32 path exits 1 as well.

Beside it, on the same line: the prefill of 2,048 tokens, the decode step's share of the memory
roofline, the same decode through the Python entry point (`e2e`: host ids in, host ids out), and
`points`: decode at batch 1 and 64 with their roofline fractions, generation of 256 tokens after
2,048-token prompts, the float32 path at batch 8, the Qwen3-0.6B shape with 32 mixed requests, and
the Qwen3-32B shape at batch 16 (each sub-record names its sizes).

`--impl reference` times the unmodified reference engine (float32, its only precision) on the same
shape, batch, context and steps through baseline/reference_arm.py and prints the same keys with
`"impl": "reference"`.  For --gpus > 1 one line says that the engine runs on one GPU; exit code 2.
"""
from __future__ import annotations

import argparse
import gc
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
QWEN3_0P6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                  intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600)
CONTEXT = 4096
LONG_CONTEXT = 32768                 # the further context length of the "long" points (Qwen3-8B allows 40,960)
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
ALL_POINTS = ("decode", "generate", "long", "fp32", "0p6b", "32b")
# The check before the line is printed: decode steps against whole prompts, same model, same positions.
# Two bfloat16 ways of computing one position are two roundings of the same exact value; their
# difference grows with depth like a random walk.  Measured on this shape against the float32 path
# (same weights, context 4,096, batch 8): root-mean-square difference of the logits, as a fraction of
# the largest |logit|, 0.0018 / 0.0030 / 0.0075 at 2 / 8 / 36 layers = 0.00125 * sqrt(layers), for
# decode-vs-float32, whole-vs-float32 and decode-vs-whole alike.  A wrong page, row or split moves
# logits by their own size (0.2 of the largest).  Allowed: 0.002 * sqrt(layers).  The float32 path
# differs between the two ways by 2e-5 of the largest logit at 36 layers (summation order in the
# library products); allowed there: 1e-5 * sqrt(layers).
CHECK_RMS_PER_SQRT_LAYER = 2e-3
CHECK_FP32_MAX_PER_SQRT_LAYER = 1e-5


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


def shape_config(shape: dict, layers: int, batch: int, context: int, **more) -> dict:
    """The flat `config` record of a measurement (every size by name, at most 20 keys)."""
    c = {"layers": layers, "layers_full": shape["num_hidden_layers"], "hidden": shape["hidden_size"],
         "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
         "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
         "tied_head": bool(shape["tie_word_embeddings"]), "global_batch": batch, "seq_len": context,
         "page_size": PAGE, "parallelism": "single GPU"}
    c.update(more)
    return c


# ---- the reference arm -----------------------------------------------------------------------------
def reference_arm(args) -> int:
    """The unmodified reference through its own PagedGenerateEngine: prefill each request, then
    `decode_batch` (src/engine/paged_generate_engine.cpp:99-149,182-341), on random float32 weights
    of the same shape.  Its API takes host token ids and returns host token ids, so its wall-clock
    figure is the end-to-end one."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as ra
        shape = dict(QWEN3_8B, num_hidden_layers=args.layers)
        clocks = ClockSampler()
        clocks.start()
        try:
            r = ra.run(shape, batch=args.batch, context=CONTEXT, steps=args.steps, warmup=args.warmup,
                       page_size=PAGE, seed=2)
        finally:
            ck = clocks.stop()
    except Exception as e:                      # ReferenceUnavailable, a missing compiler, a time-out
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())[:400]}))
        return 0
    points = {}
    if not args.no_points and "0p6b" in args.points.split(","):
        # the workload the reference publishes a figure for (readme.md:66: 32 requests, 64 new tokens each,
        # paged batch decode), with the prompts of the 0.6B benchmark configuration: the whole job timed,
        # prefill and engine construction included, as its own benchmark does
        try:
            j = ra.run(QWEN3_0P6B, batch=32, context=512 + 64, steps=0, warmup=1, page_size=PAGE, seed=3,
                       job={"prompt_min": 64, "prompt_max": 512, "new_tokens": 64})
            points["qwen3_0p6b_mixed"] = {"tok_s": round(j["tokens"] / j["wall_s"], 2), "new_tokens": j["tokens"],
                                          "seconds": round(j["wall_s"], 3), "dtype": "fp32",
                                          "config": shape_config(QWEN3_0P6B, QWEN3_0P6B["num_hidden_layers"], 32, 576,
                                                                 prompt_min=64, prompt_max=512, new_tokens=64)}
        except Exception as e:
            points["qwen3_0p6b_mixed"] = {"unavailable": " ".join(str(e).split())[:300]}
    ms = r["device_ms"] / r["steps"]
    out = {
        "impl": "reference",
        "metric": "decode tokens/s (Qwen3-8B shape, batch %d, context %d)" % (args.batch, CONTEXT),
        "value": round(r["tokens"] / (r["device_ms"] * 1e-3), 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic (random weights, uniform-random token ids)",
        "config": shape_config(QWEN3_8B, args.layers, args.batch, CONTEXT, model="Qwen3-8B shape",
                               note="the reference computes in float32 only"),
        "e2e": {"value": round(r["tokens"] / r["wall_s"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
        "prefill": {"value": round(args.batch * r["longest_prompt"] / r["prefill_s"], 1),
                    "tokens": r["longest_prompt"], "ms": round(r["prefill_s"] * 1e3 / args.batch, 1)},
        "points": points, "clocks": ck,
    }
    print(json.dumps(out))
    return 0


# ---- our arm -------------------------------------------------------------------------------------
class Bench:
    """The measurements of this engine.  Each model lives inside one method, so that its memory
    is free again when the next one is built."""

    def __init__(self, args, pk):
        import torch
        from litellmengine_b200.csrc import ops
        from litellmengine_b200.engine import ModelRunner, PagedGenerateEngine, StepEntry
        self.torch, self.ops = torch, ops
        self.ModelRunner, self.Engine, self.Entry = ModelRunner, PagedGenerateEngine, StepEntry
        self.args, self.pk = args, pk
        self.gen = torch.Generator().manual_seed(2)
        torch.cuda.set_device(0)

    # ---- helpers -----------------------------------------------------------------------------------
    def ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    def tokens(self, n, vocab=QWEN3_8B["vocab_size"]):
        return self.torch.randint(0, vocab, (n,), generator=self.gen).tolist()

    def build(self, shape, layers, dtype, max_batch, context, seed, step_tokens=None):
        from litellmengine_b200.config import config_from_dict
        config = config_from_dict(dict(shape, num_hidden_layers=layers))
        return self.ModelRunner.from_config(config, seed=seed, dtype=dtype, device="cuda:0", page_size=PAGE,
                                            max_total_tokens=max_batch * context + 64, max_requests=max_batch,
                                            max_tokens_per_step=step_tokens or context)

    def free_memory(self):
        gc.collect()
        self.torch.cuda.synchronize()
        self.torch.cuda.empty_cache()

    @staticmethod
    def prefill_flops(p, layers, T, prompts=1):
        per_layer = 2 * T * p.hidden_size * ((p.num_attention_heads + 2 * p.num_key_value_heads) * p.head_dim
                                              + p.num_attention_heads * p.head_dim + 3 * p.intermediate_size)
        attn = 2 * 2 * p.num_attention_heads * p.head_dim * (T * (T + 1) // 2)
        return prompts * (layers * (per_layer + attn) + 2 * p.hidden_size * p.vocab_size)

    def settle(self):
        """Between the prompts (seconds at the power cap) and the decode steps that are timed: wait until
        the device is idle, and a moment longer.  Right after a burst at the cap the SM clock is still
        low, and the first dozen decode steps run 10 % slower (4.0 ms falling to 3.6 over 16 steps when
        measured without this pause); whether a measurement saw that depended on whether the host
        happened to stall first (a graph capture does), not on the engine."""
        self.torch.cuda.synchronize()
        time.sleep(0.3)

    def fill(self, runner, batch, prompt_len):
        slots, prompts = [], []
        for _ in range(batch):
            s = runner.admit()
            prompts.append(self.tokens(prompt_len))
            runner.step([self.Entry(s, prompts[-1], [])])
            slots.append(s)
        return slots, prompts

    def decode_device_timed(self, runner, batch, steps, warmup, context=CONTEXT, sample_clocks=False, keep=False):
        """`batch` requests prefilled so that warmup + steps decode steps end at `context`; the steps
        are timed with CUDA events around the launches.  Returns a record; with `keep` also what a
        check needs (prompts, fed tokens, the last step's logits)."""
        torch, ops, Entry = self.torch, self.ops, self.Entry
        slots, prompts = self.fill(runner, batch, context - (steps + warmup))
        feed = [self.tokens(batch) for _ in range(steps + warmup)]
        self.settle()
        for i in range(warmup):
            lg = runner.step([Entry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
        launches0 = ops.launch_count
        a, b = self.ev(), self.ev()
        a.record()
        for i in range(warmup, warmup + steps):
            lg = runner.step([Entry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        ctx_mid = context - steps // 2
        step_bytes = runner.model.weight_bytes() + runner.cache.bytes_per_token() * ctx_mid * batch
        gbs = step_bytes / (ms * 1e-3) / 1e9
        rec = {"ms": ms, "tok_s": batch / (ms * 1e-3), "gbs": gbs, "frac": gbs / self.pk["hbm_gbs"],
               "launches": ops.launch_count - launches0, "clocks": clocks.stop() if clocks else None}
        if keep:
            rec.update(prompts=prompts, feed=feed, logits=lg.clone())
        for s in slots:
            runner.release(s)
        return rec

    def check_last_step(self, runner, rec):
        """The logits of the last timed decode step (a replayed graph over the pages) against the same
        positions as the last token of whole prompts, each run alone in one step without a graph.
        Returns the largest and the root-mean-square difference and the largest |logit|."""
        worst, scale, sq, n = 0.0, 1.0, 0.0, 0
        for j, prompt in enumerate(rec["prompts"]):
            seq = prompt + [f[j] for f in rec["feed"]]
            s = runner.admit()
            whole = runner.step([self.Entry(s, seq, [len(seq) - 1])])
            runner.release(s)
            diff = (whole[0] - rec["logits"][j]).double()
            worst = max(worst, float(diff.abs().max()))
            sq, n = sq + float((diff * diff).sum()), n + diff.numel()
            scale = max(scale, float(whole.abs().max()))
        runner.check_status()
        return {"max": worst, "rms": (sq / n) ** 0.5, "scale": scale}

    def e2e_decode(self, runner, batch, prompt_len, new_tokens, steps, warmup):
        """Through `PagedGenerateEngine`: host token ids in, host token ids out, every step."""
        engine = self.Engine(runner)
        ids = [engine.add_request(self.tokens(prompt_len), new_tokens) for _ in range(batch)]
        while any(engine.request(i).cached_len < engine.request(i).prompt_len for i in ids):
            engine.step()                                    # prompts (and the first sampled tokens)
        self.settle()
        for _ in range(warmup):
            engine.step()
        self.torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        self.torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        assert produced == steps * batch, "a request left the batch inside the timed steps"
        for i in ids:
            engine.release_request(i)
        while engine.has_work():
            engine.step()
        return produced / e2e_s

    # ---- Qwen3-8B shape, bfloat16: the headline ------------------------------------------------------
    def qwen3_8b(self, want_points, points):
        args, pk, torch = self.args, self.pk, self.torch
        many = bool({"decode", "generate"} & want_points)
        runner = self.build(QWEN3_8B, args.layers, "bfloat16", max(args.batch, 64) if many else args.batch, CONTEXT,
                            seed=2, step_tokens=max(CONTEXT, PREFILL_TOKENS))
        T = PREFILL_TOKENS

        def prefill_once():
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(T), [T - 1])])
            runner.release(s)
        for _ in range(3):
            prefill_once()
        torch.cuda.synchronize()
        reps = 5
        e0, e1 = self.ev(), self.ev()
        e0.record()
        for _ in range(reps):
            prefill_once()
        e1.record()
        torch.cuda.synchronize()
        prefill_ms = e0.elapsed_time(e1) / reps
        flops = self.prefill_flops(runner.config, args.layers, T)
        prefill = {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3),
                   "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

        head = self.decode_device_timed(runner, args.batch, args.steps, args.warmup, sample_clocks=True, keep=True)
        check = self.check_last_step(runner, head)
        check["allowed_rms"] = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * check["scale"]
        check["ok"] = check["rms"] <= check["allowed_rms"]
        out = {"prefill": prefill, "head": head, "check": check}
        if not check["ok"]:
            return out
        # Prompts are prefilled one per step, so the first request decodes a few tokens before the last
        # one starts: leave room for that, so that all of them still decode in the timed steps.
        n_new = args.steps + args.warmup + args.batch
        value = self.e2e_decode(runner, args.batch, CONTEXT - n_new, n_new + 8, args.steps, args.warmup)
        out["e2e"] = {"value": round(value, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": runner.buffers.last.size * 4, "d2h_bytes_per_step": args.batch * 4}
        if "decode" in want_points:
            for b in (1, 64):
                r = self.decode_device_timed(runner, b, max(8, min(args.steps, 32)), 3, keep=True)
                c = self.check_last_step(runner, r)
                allowed = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * c["scale"]
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
                points[f"decode_b{b}_ms"] = round(r["ms"], 3)
                points[f"decode_b{b}_frac"] = round(r["frac"], 4)
                points[f"decode_b{b}_check"] = {"ok": c["rms"] <= allowed, "rms_err": float("%.3g" % c["rms"]),
                                                "allowed_rms": float("%.3g" % allowed)}
            # end to end at batch 64 too (beside `decode_b64`: the host's share of a step grows with the batch)
            n64 = max(8, min(args.steps, 32)) + 3 + 64
            points["e2e_b64"] = round(self.e2e_decode(runner, 64, CONTEXT - n64, n64 + 8, max(8, min(args.steps, 32)), 3), 1)
        if "generate" in want_points:
            # the workload the baseline states: 2,048-token prompts, then 256 new tokens, end to end
            for b in (1, 8, 64):
                points[f"generate_p2048_n256_b{b}"] = round(self.e2e_decode(runner, b, 2048, 256 + b, 200, 8), 1)
        return out

    # ---- the same shape at a context of 32,768 ----------------------------------------------------------
    def qwen3_8b_long(self, points):
        """One 32,768-token prompt in one step (the attention's share of the work grows with the length),
        then decode steps at batch 8 and batch 1 that end at that context: a step reads 39 GB of keys
        and values beside the weights, so the attention kernel is most of it."""
        args, pk, torch = self.args, self.pk, self.torch
        C = LONG_CONTEXT
        try:
            runner = self.build(QWEN3_8B, args.layers, "bfloat16", 8, C, seed=2)
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(C), [C - 1])])
            runner.release(s)
            torch.cuda.synchronize()
            a, b = self.ev(), self.ev()
            a.record()
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(C), [C - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.release(s)
            pms = a.elapsed_time(b)
            flops = self.prefill_flops(runner.config, args.layers, C)
            rec = {"context": C, "prefill_tok_s": round(C / (pms * 1e-3), 1), "prefill_ms": round(pms, 1),
                   "prefill_frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                   "prefill_peak": "sustained"}
            for bsz in (8, 1):
                r = self.decode_device_timed(runner, bsz, 16, 4, context=C, keep=True)
                c = self.check_last_step(runner, r)
                allowed = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * c["scale"]
                rec[f"decode_b{bsz}"] = round(r["tok_s"], 1)
                rec[f"decode_b{bsz}_ms"] = round(r["ms"], 3)
                rec[f"decode_b{bsz}_frac"] = round(r["frac"], 4)
                rec[f"decode_b{bsz}_check"] = {"ok": c["rms"] <= allowed, "rms_err": float("%.3g" % c["rms"]),
                                               "allowed_rms": float("%.3g" % allowed)}
            rec["ok"] = all(rec[f"decode_b{bsz}_check"]["ok"] for bsz in (8, 1))
            points["context_32768"] = rec
        except torch.cuda.OutOfMemoryError as e:
            points["context_32768"] = {"skipped": "out of device memory: " + str(e)[:80]}

    # ---- the same shape in true float32 -------------------------------------------------------------
    def qwen3_8b_fp32(self, points):
        args = self.args
        key = "decode_b%d_fp32" % args.batch
        try:
            runner = self.build(QWEN3_8B, args.layers, "float32", args.batch, CONTEXT, seed=2)
            r = self.decode_device_timed(runner, args.batch, max(4, min(args.steps, 16)), 3, keep=True)
            check = self.check_last_step(runner, r)
            allowed = CHECK_FP32_MAX_PER_SQRT_LAYER * args.layers ** 0.5 * check["scale"]
            points[key] = round(r["tok_s"], 1)
            points[key + "_ms"] = round(r["ms"], 3)
            points[key + "_frac"] = round(r["frac"], 4)
            points[key + "_check"] = {"ok": check["max"] <= allowed, "max_err": float("%.3g" % check["max"]),
                                      "allowed": float("%.3g" % allowed)}
        except self.torch.cuda.OutOfMemoryError as e:
            points[key] = {"skipped": "out of device memory: " + str(e)[:80]}

    # ---- Qwen3-0.6B shape: 32 requests, prompts of 64..512 tokens, 64 new tokens each, mixed steps ----
    def qwen3_0p6b(self, points):
        torch = self.torch
        L = QWEN3_0P6B["num_hidden_layers"]
        runner = self.build(QWEN3_0P6B, L, "bfloat16", 32, 512 + 64 + 16, seed=3, step_tokens=512)
        lens = torch.randint(64, 513, (32,), generator=self.gen).tolist()
        prompts = [self.tokens(n) for n in lens]

        def job():
            engine = self.Engine(runner, chunk=256)
            steps0 = runner.steps_run
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = engine.generate(prompts, max_new_tokens=64)
            torch.cuda.synchronize()
            return sum(len(o) for o in out), time.perf_counter() - t0, runner.steps_run - steps0
        # Warm-up, twice: a decode step of a batch size is captured as a graph the second time that size is
        # seen, and the sizes of the tail (requests finishing one by one) occur once a job.
        job()
        job()
        made, secs, nsteps = job()
        d32 = self.decode_device_timed(runner, 32, 32, 8, context=384)
        points["qwen3_0p6b_mixed"] = {
            "tok_s": round(made / secs, 1), "new_tokens": made, "seconds": round(secs, 4), "steps": nsteps,
            "ms_per_step": round(secs * 1e3 / nsteps, 3), "decode_b32_tok_s": round(d32["tok_s"], 1),
            "decode_b32_ms": round(d32["ms"], 4), "decode_b32_frac": round(d32["frac"], 4), "dtype": "bf16",
            "config": shape_config(QWEN3_0P6B, L, 32, 384, prompt_min=64, prompt_max=512, new_tokens=64, chunk=256,
                                   step_tokens=512)}

    # ---- Qwen3-32B shape: 16 prompts of 4,096 tokens, then 128 decode steps -----------------------------
    def qwen3_32b(self, points):
        torch, pk = self.torch, self.pk
        free, _ = torch.cuda.mem_get_info()
        free += torch.cuda.memory_reserved() - torch.cuda.memory_allocated()
        need = 100e9
        if free < need:
            points["qwen3_32b"] = {"skipped": f"{free / 1e9:.0f} GB of device memory free, {need / 1e9:.0f} needed"}
            return
        try:
            L = QWEN3_32B["num_hidden_layers"]
            runner = self.build(QWEN3_32B, L, "bfloat16", 16, 4096 + 128, seed=4, step_tokens=4096)
            warm = runner.admit()
            runner.step([self.Entry(warm, self.tokens(4096), [4095])])
            runner.release(warm)
            torch.cuda.synchronize()
            slots = []
            a, b = self.ev(), self.ev()
            a.record()
            for _ in range(16):
                s = runner.admit()
                runner.step([self.Entry(s, self.tokens(4096), [4095])])
                slots.append(s)
            b.record()
            torch.cuda.synchronize()
            pms = a.elapsed_time(b)
            for s in slots:
                runner.release(s)
            d = self.decode_device_timed(runner, 16, 120, 8, context=4096 + 128)
            flops = self.prefill_flops(runner.config, L, 4096, 16)
            points["qwen3_32b"] = {
                "decode_tok_s": round(d["tok_s"], 1), "decode_ms": round(d["ms"], 3), "decode_frac": round(d["frac"], 4),
                "prefill_tok_s": round(16 * 4096 / (pms * 1e-3), 1), "prefill_ms": round(pms, 1),
                "prefill_frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                "prefill_peak": "sustained", "weight_gb": round(runner.model.weight_bytes() / 1e9, 2), "dtype": "bf16",
                "config": shape_config(QWEN3_32B, L, 16, 4096 + 128, prompt=4096, decode_steps=128)}
        except torch.cuda.OutOfMemoryError as e:
            points["qwen3_32b"] = {"skipped": "out of device memory: " + str(e)[:80]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", default=",".join(ALL_POINTS),
                    help="which extra measurements to take: " + ",".join(ALL_POINTS))
    ap.add_argument("--no-points", action="store_true", help="the headline, prefill and e2e only")
    args = ap.parse_args()

    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not built", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)
    want_points = set() if args.no_points else {p for p in args.points.split(",") if p}
    unknown = want_points - set(ALL_POINTS)
    if unknown:
        ap.error(f"unknown points {sorted(unknown)}; choose from {ALL_POINTS}")

    pk = peaks()
    bench = Bench(args, pk)
    points = {}
    main_rec = bench.qwen3_8b(want_points, points)
    head, check = main_rec["head"], main_rec["check"]
    if not check["ok"]:
        print(json.dumps({"error": "the last timed decode step's logits differ from the same positions run as "
                                   "whole prompts", "rms_error": check["rms"], "allowed_rms": check["allowed_rms"],
                          "max_error": check["max"], "largest_logit": check["scale"]}))
        return 1
    bench.free_memory()
    for name, fn in (("long", bench.qwen3_8b_long), ("fp32", bench.qwen3_8b_fp32), ("0p6b", bench.qwen3_0p6b), ("32b", bench.qwen3_32b)):
        if name in want_points:
            fn(points)
            bench.free_memory()

    bad = [k for k, v in points.items() if isinstance(v, dict) and v.get("ok") is False]
    if bad:
        print(json.dumps({"error": "decode steps differ from the same positions run as whole prompts",
                          **{k: points[k] for k in bad}}))
        return 1

    out = {
        "metric": "decode tokens/s (Qwen3-8B shape, batch %d, context %d)" % (args.batch, CONTEXT),
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform-random token ids)",
        "config": shape_config(QWEN3_8B, args.layers, args.batch, CONTEXT, model="Qwen3-8B shape",
                               l2="inputs larger than L2 (the step reads every weight)"),
        "prefill": main_rec["prefill"],
        "roofline": {"bound": "hbm", "achieved": round(head["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(head["frac"], 4), "peak_source": pk["source"]},
        "points": points, "e2e": main_rec["e2e"], "gpu_launches": head["launches"],
        "checked": True, "check": {"rms_err": round(check["rms"], 5), "allowed_rms": round(check["allowed_rms"], 5),
                                   "max_err": round(check["max"], 5), "largest_logit": round(check["scale"], 3)},
        "clocks": head["clocks"],
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
