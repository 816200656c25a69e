#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ from the reference's own C++ code.

It compiles the reference's CPU sources (core, layers, ops, model, engine; the
`.cu` files hold the CPU loops beside their kernels, so nvcc builds them, but
only `Device::CPU` code runs) together with anchor_driver.cpp, feeds it the tiny
models of tests/tiny_models.py, and stores the logits of every position as raw
little-endian float32 `[T, vocab]`.  The tests compare the plain implementation
(tests/plain_qwen3.py) with these files; they do not need the reference.

    python tests/golden/make_golden.py --reference-root <checkout of LiteLLMEngine>

The tied model (tiny A) is given a copy of the embedding table as `lm_head.weight`,
because the reference refuses a tied head without one (src/model/qwen3.cpp:1417-1420).
"""
import argparse
import glob
import hashlib
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import tiny_models as tm  # noqa: E402

CASES = {
    "tiny_a": (tm.TINY_A, tm.TINY_A_SEED, 13),
    "tiny_b": (tm.TINY_B, tm.TINY_B_SEED, 33),
}


def weights_digest(w):
    h = hashlib.sha256()
    for n in sorted(w):
        h.update(n.encode())
        h.update(w[n].numpy().tobytes())
    return h.hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", required=True)
    args = ap.parse_args()
    ref = args.reference_root
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "anchor")
        srcs = ([os.path.join(ref, "src/core", f) for f in ("tensor.cpp", "device.cpp", "tensor_memory_tracker.cpp")]
                + sorted(glob.glob(os.path.join(ref, "src/layers/*.cu")))
                + sorted(glob.glob(os.path.join(ref, "src/ops/*.cu")))
                + [os.path.join(ref, "src/ops/paged_attention.cpp"), os.path.join(ref, "src/model/qwen3.cpp")]
                + sorted(glob.glob(os.path.join(ref, "src/engine/*.cpp")))
                + [os.path.join(HERE, "anchor_driver.cpp")])
        subprocess.run(["nvcc", "-std=c++17", "-O1", "-arch=sm_89", "-I", os.path.join(ref, "include"),
                        "-o", exe] + srcs + ["-lcublas", "-lcudart"], check=True)
        meta = {}
        for name, (cfg, seed, T) in CASES.items():
            w = tm.make_weights(cfg, seed)
            digest = weights_digest(w)
            if "lm_head.weight" not in w:
                w = dict(w)
                w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
            bundle = os.path.join(tmp, name + ".bin")
            with open(bundle, "wb") as f:
                f.write(struct.pack("<i", len(w)))
                for n in sorted(w):
                    t = w[n].numpy()
                    f.write(struct.pack("<i", len(n))); f.write(n.encode())
                    f.write(struct.pack("<i", t.ndim)); f.write(struct.pack(f"<{t.ndim}q", *t.shape))
                    f.write(t.astype("<f4").tobytes())
            toks = tm.random_tokens(cfg, T, seed)
            tok_path = os.path.join(tmp, name + ".i32")
            np.asarray(toks, dtype="<i4").tofile(tok_path)
            out = os.path.join(HERE, name + "_logits.f32")
            env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
            subprocess.run([exe, bundle, tok_path, out, str(cfg["vocab_size"]), str(cfg["hidden_size"]),
                            str(cfg["intermediate_size"]), str(cfg["num_hidden_layers"]),
                            str(cfg["num_attention_heads"]), str(cfg["num_key_value_heads"]),
                            str(cfg["head_dim"]), repr(cfg["rms_norm_eps"]), repr(cfg["rope_theta"])],
                           check=True, env=env)
            meta[name] = {"tokens": toks, "weights_sha256": digest, "shape": [T, cfg["vocab_size"]]}
        with open(os.path.join(HERE, "golden.json"), "w") as f:
            json.dump(meta, f, indent=1)
    print("wrote", ", ".join(sorted(CASES)))


if __name__ == "__main__":
    main()
