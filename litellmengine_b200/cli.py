"""The command line, with the reference's option names and meanings
(include/runtime/args.hpp:8-37, src/runtime/args.cpp:56-159, src/main.cpp:26-335).

Kept: --model, --prompt, --input-ids, --max-tokens (default 128, > 0), --eos-token-id,
--temperature (default 0.7, >= 0), --top-k (50), --top-p (0.9, in (0,1]), --device,
--verbose, --benchmark, --benchmark-requests (32), --benchmark-warmup (1), --page-size (16),
both `--k v` and `--k=v`, an error plus the usage text for an unknown option, and the two
output lines a caller parses: `Generated token ids:` and `New token ids:` followed by a
comma-separated list or `<none>` (src/main.cpp:313-327, scripts/run_prompt.py:9-27).
Differences: a positive temperature really samples (the reference warns and takes the
argmax, src/main.cpp:175-178); top-k and top-p are parsed, validated and, as in the reference,
not applied; --use-kv-cache, --use-paged-kv-cache, --benchmark-interleaved and
--benchmark-batch-decode are accepted and ignored, because there is one cache (paged) and
one scheduler; --device takes only CUDA devices.  Added: --dtype, --seed, --random-weights,
--max-total-tokens, --chunk, --max-tokens-per-step, --benchmark-prompt-len.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass
from typing import List, Optional

USAGE = """Usage:
  {prog} --model <model_dir> [options]

Options:
  --model <str>            Local model folder (config.json + *.safetensors)
  --prompt <str>           Input prompt (needs tokenizer.json in the model folder)
  --input-ids <str>        Comma-separated token ids, e.g. "1,2,3"
  --max-tokens <int>       Maximum generated tokens, default: 128
  --temperature <float>    Sampling temperature, default: 0.7 (0 = greedy)
  --top-k <int>            Parsed and validated, not applied, default: 50
  --top-p <float>          Parsed and validated, not applied, default: 0.9
  --seed <int>             Seed of the sampling stream and of --random-weights, default: 0
  --device <str>           cuda, cuda:N, gpu or auto (there is no CPU path)
  --dtype <str>            bfloat16 (default) or float32
  --eos-token-id <int>     Stop generation when this token id is generated
  --page-size <N>          Paged KV cache page size, default 16
  --max-total-tokens <N>   Tokens the cache pool holds, default: prompt + max tokens + 16
  --chunk <N>              Longest prompt portion per step, default: --max-tokens-per-step
  --max-tokens-per-step <N>  Token budget of one step, default 8192
  --random-weights         Ignore the folder's weights; draw random ones from --seed
  --benchmark              Time generation instead of printing ids
  --benchmark-requests <N> Requests in the benchmark, default 32
  --benchmark-warmup <N>   Warm-up requests, default 1
  --benchmark-prompt-len <N>  Use N random prompt tokens in the benchmark
  --verbose                Print every step
  -h, --help               Show this help message
"""


@dataclass
class Args:
    model: str = ""
    prompt: str = "What is the capital of France?"
    input_ids: Optional[str] = None
    eos_token_id: Optional[int] = None
    max_tokens: int = 128
    temperature: float = 0.7
    top_k: int = 50
    top_p: float = 0.9
    verbose: bool = False
    device: Optional[str] = None
    benchmark: bool = False
    benchmark_requests: int = 32
    benchmark_warmup: int = 1
    use_kv_cache: bool = False
    use_paged_kv_cache: bool = False
    page_size: int = 16
    benchmark_interleaved: bool = False
    benchmark_batch_decode: bool = False
    # additions
    seed: int = 0
    dtype: str = "bfloat16"
    random_weights: bool = False
    max_total_tokens: Optional[int] = None
    chunk: Optional[int] = None
    max_tokens_per_step: int = 8192
    benchmark_prompt_len: Optional[int] = None


class ArgError(ValueError):
    pass


_VALUE = {"--model": ("model", str), "--prompt": ("prompt", str), "--input-ids": ("input_ids", str),
          "--max-tokens": ("max_tokens", int), "--eos-token-id": ("eos_token_id", int),
          "--temperature": ("temperature", float), "--top-k": ("top_k", int), "--top-p": ("top_p", float),
          "--device": ("device", str), "--benchmark-requests": ("benchmark_requests", int),
          "--benchmark-warmup": ("benchmark_warmup", int), "--page-size": ("page_size", int),
          "--seed": ("seed", int), "--dtype": ("dtype", str), "--max-total-tokens": ("max_total_tokens", int),
          "--chunk": ("chunk", int), "--max-tokens-per-step": ("max_tokens_per_step", int),
          "--benchmark-prompt-len": ("benchmark_prompt_len", int)}
_FLAG = {"--verbose": "verbose", "--benchmark": "benchmark", "--use-kv-cache": "use_kv_cache",
         "--use-paged-kv-cache": "use_paged_kv_cache", "--benchmark-interleaved": "benchmark_interleaved",
         "--benchmark-batch-decode": "benchmark_batch_decode", "--random-weights": "random_weights"}


def parse_args(argv: List[str]) -> Args:
    """src/runtime/args.cpp:82-159: `--k v` or `--k=v`; unknown option is an error."""
    a = Args()
    i = 0
    while i < len(argv):
        arg = argv[i]
        if arg in ("-h", "--help"):
            print(USAGE.format(prog="litellmengine"))
            raise SystemExit(0)
        key, eq, inline = arg.partition("=")
        if key in _VALUE:
            if eq:
                raw = inline
            else:
                if i + 1 >= len(argv):
                    raise ArgError(f"Missing value for argument: {arg}")
                i += 1
                raw = argv[i]
            name, kind = _VALUE[key]
            try:
                setattr(a, name, kind(raw))
            except ValueError:
                raise ArgError(f"Invalid value for {key}: {raw}") from None
        elif arg in _FLAG:
            setattr(a, _FLAG[arg], True)
        else:
            raise ArgError(f"Unknown argument: {arg}")
        i += 1
    if not a.model:
        raise ArgError("Missing required argument: --model")
    if a.max_tokens <= 0:
        raise ArgError("--max-tokens must be greater than 0")
    if a.temperature < 0.0:
        raise ArgError("--temperature must be >= 0")
    if a.top_k < 0:
        raise ArgError("--top-k must be >= 0")
    if a.top_p <= 0.0 or a.top_p > 1.0:
        raise ArgError("--top-p must be in range (0, 1]")
    if a.eos_token_id is not None and a.eos_token_id < 0:
        raise ArgError("--eos-token-id must be >= 0")
    if a.page_size <= 0:
        raise ArgError("--page-size must be positive")
    if a.dtype not in ("bfloat16", "bf16", "float32", "fp32"):
        raise ArgError("--dtype must be bfloat16 or float32")
    return a


def parse_token_ids(text: str) -> List[int]:
    """"1,2,3" -> [1,2,3] with the reference's strictness (src/runtime/token_ids.cpp:64-109)."""
    trimmed = text.strip()
    if not trimmed:
        raise ArgError("Token ids string must not be empty")
    out = []
    for part in trimmed.split(","):
        v = part.strip()
        if not v:
            raise ArgError("Empty token id")
        try:
            n = int(v, 10)
        except ValueError:
            raise ArgError(f"Invalid token id: {v}") from None
        if v[0] == "+" or "_" in v:
            raise ArgError(f"Invalid token id: {v}")
        if n < 0:
            raise ArgError(f"Token id must be non-negative: {v}")
        if n > 2**31 - 1:
            raise ArgError(f"Token id too large: {v}")
        out.append(n)
    return out


def format_token_ids(ids) -> str:
    return ",".join(str(int(t)) for t in ids)


def chat_template(prompt: str, enable_thinking: bool = False) -> str:
    """The reference's fixed Qwen3 template (src/tokenizer/qwen3_chat_template.cpp:7-25)."""
    text = "<|im_start|>user\n" + prompt + "<|im_end|>\n<|im_start|>assistant\n"
    return text + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")


def resolve_device(name: str) -> str:
    """src/core/device.cpp:20-41 without the CPU branch."""
    n = (name or "auto").lower()
    if n in ("auto", "cuda", "gpu"):
        return "cuda:0"
    if n.startswith("cuda:") and n[5:].isdigit():
        return n
    if n == "cpu":
        raise ArgError("--device cpu: this engine has no CPU path")
    raise ArgError(f"Unknown device: {name}")


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        args = parse_args(argv)
        return _run(args)
    except SystemExit as e:
        return int(e.code or 0)
    except Exception as e:                                   # like src/main.cpp:330-334
        print(f"Error: {e}\n", file=sys.stderr)
        print(USAGE.format(prog="litellmengine"), file=sys.stderr)
        return 1


def _run(args: Args) -> int:
    device = resolve_device(args.device or "auto")
    print("LiteLLMEngine (B200)")
    print(f"Device: {device}")
    print("Config:")
    for k, v in (("Model", args.model), ("Prompt", args.prompt), ("Max tokens", args.max_tokens),
                 ("Temperature", args.temperature), ("Top-k", args.top_k), ("Top-p", args.top_p),
                 ("Seed", args.seed), ("Dtype", args.dtype), ("Eos Token Id", args.eos_token_id if
                                                               args.eos_token_id is not None else -1),
                 ("page_size", args.page_size), ("benchmark", args.benchmark)):
        print(f"  {k + ':':<14}{v}")
    if args.use_kv_cache or args.use_paged_kv_cache or args.benchmark_interleaved or args.benchmark_batch_decode:
        print("Note: the cache is always paged and one scheduler batches every step; "
              "--use-kv-cache, --use-paged-kv-cache, --benchmark-interleaved and "
              "--benchmark-batch-decode change nothing.")

    print("\nLoading model metadata...")
    from .config import load_config
    config = load_config(args.model)
    print("Model config:")
    for k, v in config.to_dict().items():
        print(f"  {k}: {v}")

    tokenizer = None
    if args.input_ids is not None:
        input_ids = parse_token_ids(args.input_ids)
        print("\nInput token ids:\n  " + format_token_ids(input_ids))
    elif args.benchmark and args.benchmark_prompt_len:
        import random
        rng = random.Random(args.seed)
        input_ids = [rng.randrange(config.vocab_size) for _ in range(args.benchmark_prompt_len)]
    else:
        path = os.path.join(args.model, "tokenizer.json")
        print(f"\nLoading tokenizer from:\n  {path}")
        if not os.path.isfile(path):
            raise ArgError(f"no tokenizer at {path}; pass --input-ids")
        from tokenizers import Tokenizer            # optional dependency, only on this branch
        tokenizer = Tokenizer.from_file(path)
        input_ids = tokenizer.encode(chat_template(args.prompt, False), add_special_tokens=False).ids
        print(f"\nInput prompt:\n{args.prompt}\n\nEncoded input token ids:\n  " + format_token_ids(input_ids))
    print(f"Input length: {len(input_ids)}")

    if args.temperature != 0.0 and (args.top_k != 50 or args.top_p != 0.9):
        print("\nNote: --top-k and --top-p are not applied; sampling uses the temperature only.")

    from .engine import PagedGenerateEngine
    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)
    n_req = args.benchmark_requests if args.benchmark else 1
    per_request = len(input_ids) + args.max_tokens + 16          # as src/main.cpp:265-268
    total = args.max_total_tokens or per_request * n_req
    print("\nBuilding the model..." if not args.random_weights else "\nBuilding the model with random weights...")
    engine = PagedGenerateEngine(
        config if args.random_weights else args.model, dtype=dtype, device=device, page_size=args.page_size,
        max_total_tokens=total, max_requests=max(n_req, 1), max_tokens_per_step=args.max_tokens_per_step,
        chunk=args.chunk, verbose=args.verbose, seed=args.seed)
    print("Model initialized.")
    eos = args.eos_token_id if args.eos_token_id is not None else -1

    if args.benchmark:
        return _benchmark(engine, input_ids, args, eos)

    print("\nGenerating...")
    rid = engine.add_request(input_ids, args.max_tokens, eos, args.temperature, args.seed)
    generated = engine.generate_until_finished(rid)
    engine.runner.check_status()
    new_ids = generated[len(input_ids):]
    engine.release_request(rid)
    print("\nGenerated token ids:\n  " + format_token_ids(generated))
    print("\nNew token ids:\n  " + (format_token_ids(new_ids) if new_ids else "<none>"))
    if tokenizer is not None:
        print("\nDecoded new text:\n" + tokenizer.decode(new_ids))
    return 0


def _benchmark(engine, input_ids, args: Args, eos: int) -> int:
    """Wall-clock tokens per second over N equal requests run together, after warm-up
    requests (src/benchmark/generation_benchmark.cpp:359-529; unlike it, building the engine
    and its cache pool is outside the timed region)."""
    import torch
    print("\nRunning generation benchmark...")
    for _ in range(max(args.benchmark_warmup, 0)):
        engine.generate([input_ids], min(args.max_tokens, 8), eos, args.temperature, args.seed)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate([input_ids] * args.benchmark_requests, args.max_tokens, eos, args.temperature, args.seed)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    total_new = sum(len(o) for o in outs)
    print("\nGeneration benchmark result")
    print("  Mode:             Paged KV cache, scheduled mixed batches")
    print(f"  Page size:        {args.page_size}")
    print(f"  Requests:         {args.benchmark_requests}")
    print(f"  Prompt tokens:    {len(input_ids)}")
    print(f"  Max new tokens:   {args.max_tokens}")
    print(f"  Total new tokens: {total_new}")
    print(f"  Total time:       {dt * 1e3:.3f} ms")
    print(f"  Throughput:       {total_new / dt:.2f} tok/s")
    print(f"  Latency/token:    {dt * 1e3 / max(total_new, 1):.4f} ms/token")
    return 0
