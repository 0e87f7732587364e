"""The command line's flag rules, which follow the reference's (apps/hf_infer.cpp:179-285): no GPU needed."""
import pytest

from microllm_rocm_b200 import cli

BASE = ["--model", "folder", "--tokens", "1,2,3"]


def check(argv):
    options = cli.parse(argv)
    cli.validate(options)
    return options


def test_pairs_names_and_types():
    o = check(BASE + ["--new-tokens", "4", "--top-k", "3", "--dtype", "bf16"])
    assert o["new-tokens"] == 4 and o["top-k"] == 3 and cli.compute_dtype(o) == "bfloat16"
    with pytest.raises(cli.UsageError, match="missing CLI value"):
        cli.parse(BASE + ["--new-tokens"])
    with pytest.raises(cli.UsageError, match="unknown CLI option"):
        cli.parse(["--no-such-flag", "1"])
    with pytest.raises(cli.UsageError, match="cannot read"):
        cli.parse(BASE + ["--new-tokens", "four"])


@pytest.mark.parametrize("argv,message", [
    (["--tokens", "1"], "--config and --weights are required"),
    (BASE + ["--device", "cpu"], "no CPU path"),
    (BASE + ["--workload", "train"], "--workload must be"),
    (BASE + ["--top-k", "0"], "--top-k must be positive"),
    (BASE + ["--batch", "0"], "--batch must be positive"),
    (BASE + ["--cache-prefill-mode", "half"], "full or token"),
    (BASE + ["--new-tokens", "-1"], "cannot be negative"),
    (BASE + ["--steps", "0"], "--steps positive"),
    (BASE + ["--workload", "decode"], "decode workload requires positive --new-tokens"),
    (BASE + ["--workload", "prefill", "--new-tokens", "2"], "prefill workload requires --new-tokens 0"),
    (BASE + ["--bf16-attention", "true"], "requires --bf16-ffn true"),
    (BASE + ["--cache-logits-output", "x.bin", "--new-tokens", "1"], "at least two new tokens"),
    (["--model", "folder", "--workload", "continuous"], "continuous workload requires"),
    (["--model", "folder"], "--tokens is required"),
    (BASE + ["--stop-on-eos", "maybe"], "--stop-on-eos must be true or false"),
    (BASE + ["--trace-output", "t.jsonl"], "--trace-output requires prefill workload"),
    (BASE + ["--trace-output", "t.jsonl", "--workload", "prefill", "--prefill-steps", "2"], "--trace-output requires prefill workload"),
    (BASE + ["--trace-max-elements", "0"], "--trace-max-elements must be positive"),
])
def test_rules_of_the_reference(argv, message):
    with pytest.raises(cli.UsageError, match=message):
        check(argv)


def test_switches_between_paths_this_engine_does_not_have():
    check(BASE + ["--prefill-logits", "full"])
    with pytest.raises(cli.UsageError, match="--prefill-logits must be last or full"):
        check(BASE + ["--prefill-logits", "all"])
    check(BASE + ["--use-cache", "true", "--prefill-logits", "last", "--batch-argmax-mode", "device",
                  "--decode-mode", "generation", "--continuous-prefill-batch", "true", "--continuous-diagnostics", "false"])
    for flag, value in (("--use-cache", "false"), ("--batch-argmax-mode", "host"),
                        ("--decode-mode", "steady"), ("--continuous-prefill-batch", "false"), ("--continuous-diagnostics", "true")):
        with pytest.raises(cli.UsageError, match="not available in this engine"):
            check(BASE + [flag, value])
    with pytest.raises(cli.UsageError, match="--decode-mode must be generation or steady"):
        check(BASE + ["--decode-mode", "fast"])
    for flag in ("--text", "--vocab", "--merges", "--continuous-cache-buckets", "--kv-cache-fp32-layers"):
        with pytest.raises(cli.UsageError, match="does not have"):
            cli.parse(["--model", "folder", flag, "x"])


def test_help_lists_every_option(capsys):
    from microllm_rocm_b200 import cli
    assert cli.main(["--help"]) == 0
    text = capsys.readouterr().out
    for name in cli.DEFAULTS:
        assert f"--{name} " in text
