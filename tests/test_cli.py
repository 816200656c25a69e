"""The command line's options, read as the reference reads its own (src/runtime/args.cpp:82-159,
src/runtime/token_ids.cpp:64-109, src/core/device.cpp:20-41): names, defaults, both spellings of a
value, refusals.  No GPU: nothing here builds an engine."""
import pytest

from litellmengine_b200 import cli


def test_defaults_are_the_references():
    a = cli.parse_args(["--model", "m"])
    assert (a.max_tokens, a.temperature, a.top_k, a.top_p) == (128, 0.7, 50, 0.9)
    assert (a.page_size, a.benchmark_requests, a.benchmark_warmup) == (16, 32, 1)
    assert a.eos_token_id is None and a.input_ids is None and not a.benchmark and not a.verbose
    assert a.prompt == "What is the capital of France?"


def test_a_value_may_follow_its_option_or_an_equals_sign():
    a = cli.parse_args(["--model=folder", "--max-tokens", "7", "--temperature=0", "--input-ids=1,2,3",
                        "--eos-token-id", "5", "--page-size=8", "--seed", "11", "--dtype=float32"])
    assert (a.model, a.max_tokens, a.temperature, a.input_ids, a.eos_token_id) == ("folder", 7, 0.0, "1,2,3", 5)
    assert (a.page_size, a.seed, a.dtype) == (8, 11, "float32")


def test_flags_of_the_reference_that_choose_a_cache_or_a_loop_are_taken_and_change_nothing():
    a = cli.parse_args(["--model", "m", "--use-kv-cache", "--use-paged-kv-cache", "--benchmark",
                        "--benchmark-interleaved", "--benchmark-batch-decode", "--verbose"])
    assert a.use_kv_cache and a.use_paged_kv_cache and a.benchmark_interleaved and a.benchmark_batch_decode
    assert a.benchmark and a.verbose


@pytest.mark.parametrize("argv,msg", [
    ([], "Missing required argument: --model"),
    (["--model", "m", "--frobnicate"], "Unknown argument: --frobnicate"),
    (["--model", "m", "--max-tokens"], "Missing value for argument: --max-tokens"),
    (["--model", "m", "--max-tokens", "many"], "Invalid value for --max-tokens: many"),
    (["--model", "m", "--max-tokens", "0"], "--max-tokens must be greater than 0"),
    (["--model", "m", "--temperature", "-1"], "--temperature must be >= 0"),
    (["--model", "m", "--top-k", "-3"], "--top-k must be >= 0"),
    (["--model", "m", "--top-p", "0"], r"--top-p must be in range \(0, 1\]"),
    (["--model", "m", "--top-p", "1.5"], r"--top-p must be in range \(0, 1\]"),
    (["--model", "m", "--eos-token-id", "-2"], "--eos-token-id must be >= 0"),
    (["--model", "m", "--page-size", "0"], "--page-size must be positive"),
    (["--model", "m", "--dtype", "float16"], "--dtype must be bfloat16 or float32"),
])
def test_refusals(argv, msg):
    with pytest.raises(cli.ArgError, match=msg):
        cli.parse_args(argv)


def test_help_prints_the_usage_and_ends(capsys):
    with pytest.raises(SystemExit) as e:
        cli.parse_args(["--help"])
    assert e.value.code == 0
    out = capsys.readouterr().out
    for opt in ("--model", "--input-ids", "--max-tokens", "--eos-token-id", "--temperature", "--page-size",
                "--benchmark-requests", "--benchmark-warmup", "--verbose"):
        assert opt in out


def test_main_turns_a_refusal_into_the_usage_text_and_a_failure(capsys):
    rc = cli.main(["--model", "m", "--no-such-option"])
    captured = capsys.readouterr()
    assert rc != 0
    assert "Unknown argument: --no-such-option" in captured.out + captured.err
    assert "Usage:" in captured.out + captured.err


def test_token_id_lists_are_read_strictly():
    assert cli.parse_token_ids(" 1, 22 ,333 ") == [1, 22, 333]
    assert cli.format_token_ids([4, 5, 6]) == "4,5,6"
    for bad, msg in (("", "must not be empty"), ("1,,2", "Empty token id"), ("1,x", "Invalid token id: x"),
                     ("+3", "Invalid token id"), ("1_0", "Invalid token id"), ("-4", "non-negative"),
                     (str(2**31), "too large")):
        with pytest.raises(cli.ArgError, match=msg):
            cli.parse_token_ids(bad)


def test_devices():
    assert cli.resolve_device("auto") == cli.resolve_device("cuda") == cli.resolve_device("GPU") == "cuda:0"
    assert cli.resolve_device("cuda:3") == "cuda:3"
    with pytest.raises(cli.ArgError, match="no CPU path"):
        cli.resolve_device("cpu")
    with pytest.raises(cli.ArgError, match="Unknown device"):
        cli.resolve_device("tpu")


def test_the_chat_template_is_the_references():
    assert cli.chat_template("hi") == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n"
    assert cli.chat_template("hi", enable_thinking=True).endswith("<|im_start|>assistant\n<think>\n")


def test_run_prompt_hands_ids_to_the_engine_and_reads_its_new_ids_line(tmp_path):
    """The script's contract with the engine's command line (scripts/run_prompt.py:9-27,96-162): it
    passes --input-ids, --max-tokens and --temperature 0, and picks the line after `New token ids:`.
    A stand-in engine that prints its arguments and the two lines is enough to see both."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    fake = tmp_path / "engine.py"
    fake.write_text("import sys\nprint('argv', ' '.join(sys.argv[1:]))\n"
                    "print('Generated token ids:')\nprint('5,6,7,41,42')\nprint('New token ids:')\nprint('41,42')\n")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(tmp_path), "--engine",
                        str(fake), "--input-ids", "5,6,7", "--max-tokens", "2"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "--input-ids 5,6,7" in r.stdout and "--max-tokens 2" in r.stdout and "--temperature 0" in r.stdout
    assert "[new token ids]\n41,42" in r.stdout
    none = tmp_path / "none.py"
    none.write_text("print('Generated token ids:')\nprint('5')\nprint('New token ids:')\nprint('<none>')\n")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(tmp_path), "--engine",
                        str(none), "--input-ids", "5"], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.rstrip().endswith("[new token ids]")
    both = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(tmp_path),
                           "--input-ids", "5", "--prompt", "x"], capture_output=True, text=True)
    assert both.returncode != 0 and "exactly one" in both.stderr
