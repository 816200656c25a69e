"""Builds and runs the reference arm of bench.py: the unmodified LiteLLMEngine sources, compiled
for sm_100a with nvcc, driven by reference_arm.cu.

The reference is a CMake project whose top-level target needs an empty tokenizer submodule, so
this compiles the files its engine is made of directly (the same list its own tests link:
core, layers, ops, model, engine) and leaves out what needs absent third-party code
(model_config.cpp and weight_loader.cpp want nlohmann/json, hf_tokenizer.cpp wants
tokenizers-cpp; main.cpp and model_downloader.cpp are the command line).  The sources are
copied, byte for byte, into baseline/_ref/src-tree first, because the GPU machine has no
checkout of the reference; baseline/_ref is not tracked.

Nothing of this repository's package is imported here.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import shutil
import subprocess
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
TREE = os.path.join(REF_DIR, "src-tree")
BINARY = os.path.join(REF_DIR, "reference_arm")
STAMP = os.path.join(REF_DIR, "reference_arm.json")
DRIVER = os.path.join(HERE, "reference_arm.cu")
DEFAULT_CHECKOUT = os.environ.get("LITELLM_REFERENCE_ROOT", "/root/reference")


class ReferenceUnavailable(RuntimeError):
    pass


def _sources(tree: str) -> List[str]:
    src = os.path.join(tree, "src")
    files = [os.path.join(src, "core", f) for f in ("tensor.cpp", "device.cpp", "tensor_memory_tracker.cpp")]
    files += sorted(glob.glob(os.path.join(src, "layers", "*.cu")))
    files += sorted(glob.glob(os.path.join(src, "ops", "*.cu")))
    files += [os.path.join(src, "ops", "paged_attention.cpp"), os.path.join(src, "model", "qwen3.cpp")]
    files += sorted(glob.glob(os.path.join(src, "engine", "*.cpp")))
    return files


def _digest(paths: List[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.relpath(p, REF_DIR).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def copy_sources(checkout: str = DEFAULT_CHECKOUT) -> None:
    """Copy the reference's src/ and include/ unmodified into baseline/_ref/src-tree."""
    if not os.path.isdir(os.path.join(checkout, "src")):
        raise ReferenceUnavailable(f"no checkout of the reference at {checkout}")
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.isdir(TREE):
        shutil.rmtree(TREE)
    os.makedirs(TREE)
    for sub in ("src", "include"):
        shutil.copytree(os.path.join(checkout, sub), os.path.join(TREE, sub))


def ensure_built(verbose: bool = False) -> str:
    """Path of the reference arm's binary, compiling it if its sources changed or it is absent."""
    if not os.path.isdir(os.path.join(TREE, "src")):
        copy_sources()
    srcs = _sources(TREE)
    missing = [s for s in srcs if not os.path.isfile(s)]
    if missing:
        raise ReferenceUnavailable(f"the reference's source tree lacks {os.path.relpath(missing[0], TREE)}")
    headers = glob.glob(os.path.join(TREE, "include", "**", "*.hpp"), recursive=True)
    digest = _digest(srcs + headers + [DRIVER])
    if os.path.isfile(BINARY) and os.path.isfile(STAMP):
        try:
            with open(STAMP) as f:
                if json.load(f).get("sha256") == digest:
                    return BINARY
        except (OSError, ValueError):
            pass
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise ReferenceUnavailable("nvcc not found: cannot compile the reference")
    cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", os.path.join(TREE, "include"), "-o", BINARY] + srcs + [DRIVER, "-lcublas", "-lcudart"]
    if verbose:
        print("compiling the reference:", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise ReferenceUnavailable("the reference does not compile here: " + r.stdout.strip().splitlines()[-1][:300])
    with open(STAMP, "w") as f:
        json.dump({"sha256": digest, "command": cmd}, f)
    return BINARY


def run(shape: dict, batch: int, context: int, steps: int, warmup: int, page_size: int = 16, seed: int = 2,
        job: Optional[dict] = None, timeout: float = 3000.0) -> dict:
    """Run the binary; returns its JSON.  `shape` has config.json's keys.  `job` = {"prompt_min",
    "prompt_max", "new_tokens"} times a whole generation job instead of decode steps."""
    exe = ensure_built()
    args = [exe, "--layers", shape["num_hidden_layers"], "--hidden", shape["hidden_size"],
            "--heads", shape["num_attention_heads"], "--kv-heads", shape["num_key_value_heads"],
            "--head-dim", shape["head_dim"], "--intermediate", shape["intermediate_size"],
            "--vocab", shape["vocab_size"], "--theta", repr(float(shape["rope_theta"])),
            "--eps", repr(float(shape["rms_norm_eps"])), "--batch", batch, "--context", context,
            "--steps", steps, "--warmup", warmup, "--page-size", page_size, "--seed", seed]
    if job:
        args += ["--prompt-min", job["prompt_min"], "--prompt-max", job["prompt_max"], "--new-tokens", job["new_tokens"]]
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([str(a) for a in args], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                       env=env, timeout=timeout)
    if r.returncode != 0:
        tail = (r.stderr.strip().splitlines() or ["no message"])[-1]
        raise ReferenceUnavailable(f"the reference's engine stopped with code {r.returncode}: {tail[:300]}")
    return json.loads(r.stdout.strip().splitlines()[-1])
