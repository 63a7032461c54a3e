"""The command line: what it refuses (on the CPU), and -- on a GPU -- that its tokens, traces, hashes, perplexity,
files and phase times are what the engine and the plain implementation give (the reference's counterparts:
tests/validation.test.ts:37-170 for refusals, tests/runtime.test.ts:63-89,169-181,210-226 for the rest)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_model
from tiny import TINY, random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "bin", "smolmoe_b200")


def _main(argv, capsys):
    from smolmoe_c99_b200.engine.cli import main
    code = main(argv)
    captured = capsys.readouterr()
    stats = json.loads(captured.err.strip().splitlines()[-1])
    return code, captured.out, stats


# ---- refusals: no GPU is touched before the arguments have been checked ---------------------------------------------
@pytest.mark.parametrize("argv,message", [
    ([], "a model folder"),
    (["m"], "--prompt or --prompt-file"),
    (["m", "--prompt", "1 2 x"], "list of token ids"),
    (["m", "--prompt", "1 2", "--seed", "0"], "seed and batch"),
    (["m", "--prompt", "1 2", "--batch", "0"], "seed and batch"),
    (["m", "--prompt", "1 2", "--tokens", "-1"], "tokens must not be negative"),
    (["m", "--prompt", "1 2", "--step-tokens", "0"], "step-tokens must be positive"),
    (["m", "--prompt", "1 2", "--context", "0"], "context must be positive"),
    (["m", "--prompt", "1 2", "--temperature", "1e-9"], "temperature"),
    (["m", "--prompt", "1 2", "--temperature", "101"], "temperature"),
    (["m", "--prompt", "1 2", "--top-p", "0"], "top-p"),
    (["m", "--prompt", "1 2", "--top-p", "1.5"], "top-p"),
    (["m", "--prompt", "1 2", "--top-k", "-3"], "top-k"),
])
def test_arguments_that_are_refused(argv, message):
    from smolmoe_c99_b200.engine.cli import main
    with pytest.raises(SystemExit) as e:
        main(argv)
    assert message in str(e.value)


def test_options_that_argparse_refuses():
    from smolmoe_c99_b200.engine.cli import main
    for argv in (["m", "--dtype", "float16"], ["m", "--kernels", "quick"], ["m", "--tokens", "many"], ["m", "--no-such-option"]):
        with pytest.raises(SystemExit) as e:
            main(argv + ["--prompt", "1"])
        assert e.value.code == 2


def test_random_weights_are_written_without_a_gpu(tmp_path):
    from smolmoe_c99_b200.engine.cli import main
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY["A"]))
    assert main(["--random", str(cfg), "--seed", "5", "--save", str(tmp_path / "m")]) == 0
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    again = tmp_path / "m2"
    main(["--random", str(cfg), "--seed", "5", "--save", str(again)])
    assert (tmp_path / "m" / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()


# ---- on the GPU -------------------------------------------------------------------------------------------------------
def _prompts(name, lengths, seed):
    return [random_tokens(n, TINY[name]["vocab_size"], seed + i) for i, n in enumerate(lengths)]


def _flags(prompts):
    out = []
    for p in prompts:
        out += ["--prompt", " ".join(map(str, p))]
    return out


@pytest.mark.gpu
def test_the_program_as_a_user_runs_it(model_dirs, tmp_path):
    """bin/smolmoe_b200 in a process of its own: tokens on stdout equal ``Model.generate``'s, the statistics line and
    the --stats and --token-ids files are well-formed."""
    from smolmoe_c99_b200 import Model
    prompts = _prompts("A", [5, 11, 17], 700)
    ids_file, stats_file, prompt_file = tmp_path / "ids.txt", tmp_path / "stats.json", tmp_path / "prompts.txt"
    prompt_file.write_text("".join(",".join(map(str, p)) + "\n" for p in prompts))
    proc = subprocess.run([sys.executable, BIN, model_dirs["A"], "--prompt-file", str(prompt_file), "--tokens", "8", "--dtype",
                           "float32", "--batch", "3", "--stop-ids", "", "--token-ids", str(ids_file), "--stats", str(stats_file)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [[int(t) for t in line.split()] for line in proc.stdout.strip().splitlines()]
    want = Model.from_folder(model_dirs["A"], "float32", batch=3).generate(prompts, tokens=8, stop_ids=())
    assert got == want
    stats = json.loads(stats_file.read_text())
    assert stats == json.loads(proc.stderr.strip().splitlines()[-1])
    assert stats["prompt_tokens"] == 33 and stats["generated_tokens"] == 24 and stats["processed_tokens"] == 33 + 21
    assert stats["decode_tokens_per_second"] > 0 and stats["prefill_tokens_per_second"] > 0 and stats["logits_hash"] == "0" * 16
    blocks = [b.split("\n") for b in ids_file.read_text().strip().split("\n\n")]
    assert [[int(t) for t in b] for b in blocks] == [p + g for p, g in zip(prompts, got)]
    # a model folder that is not there: a clean message, not a traceback
    bad = subprocess.run([sys.executable, BIN, str(tmp_path / "nowhere"), "--prompt", "1 2"], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "smolmoe:" in bad.stderr and "Traceback" not in bad.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_hash_and_perplexity(model_dirs, tmp_path, capsys, dtype):
    from smolmoe_c99_b200.engine.engine import Engine
    name = "B"
    prompts = _prompts(name, [9, 40, 23], 720)
    trace = tmp_path / "t.txt"
    base = [model_dirs[name], "--dtype", dtype, "--tokens", "0"] + _flags(prompts)
    _, _, stats = _main(base + ["--trace", str(trace), "--hash-logits", "--perplexity", "--batch", "1"], capsys)
    # the trace's rows are the step function's logits, as exact hexadecimal floats
    engine = Engine(model_dirs[name], dtype, max_tokens=1024)
    lines = trace.read_text().strip().split("\n")
    assert len(lines) == sum(len(p) for p in prompts)
    at, nll, count = 0, 0.0, 0
    for p in prompts:
        slot = engine.open_sequence()
        rows = engine.step([slot], [p], [list(range(len(p)))]).cpu()
        engine.close_sequence(slot)
        for pos in range(len(p)):
            fields = lines[at].split(" ")
            assert int(fields[0]) == pos
            assert torch.equal(torch.tensor([float.fromhex(f) for f in fields[1:]], dtype=torch.float32), rows[pos])
            at += 1
        want = plain_model.forward(model_dirs[name], p, round_like_bf16_engine=(dtype == "bfloat16")).double()
        for pos in range(len(p) - 1):
            nll += float(torch.logsumexp(want[pos], dim=0) - want[pos][p[pos + 1]])
            count += 1
    assert stats["perplexity_tokens"] == count
    assert abs(stats["nll"] - nll / count) <= (1e-6 if dtype == "float32" else 2e-3)
    assert abs(stats["perplexity"] - math.exp(stats["nll"])) < 1e-9
    # the hash does not depend on how the prompts are batched or cut into portions (bit for bit in 32-bit)
    hashes = {stats["logits_hash"]}
    for extra in (["--batch", "3"], ["--batch", "2", "--step-tokens", "7"], ["--batch", "3", "--profile"]):
        _, _, other = _main(base + ["--hash-logits"] + extra, capsys)
        if dtype == "float32":
            hashes.add(other["logits_hash"])
        if "--profile" in extra:
            # time per phase under the reference's keys (src/model.c:312-328); profiling changes no logit
            assert set(other["profile"]) == {"embed", "norm", "qkv", "rope", "attention", "attn_out", "ffn_up", "activation",
                                             "attn_quant", "ffn_down", "routing", "residual", "logits"}
            assert other["profile"]["qkv"] > 0 and other["profile"]["attention"] > 0 and other["profile"]["logits"] > 0
            assert other["profile"]["routing"] == 0 and sum(other["profile"].values()) < 10
            _, _, plain_run = _main(base + ["--hash-logits", "--batch", "3"], capsys)
            assert other["logits_hash"] == plain_run["logits_hash"]
    assert len(hashes) == 1 and stats["logits_hash"] != "0" * 16


def _read_trace(path):
    return torch.tensor([[float.fromhex(f) for f in line.split(" ")[1:]] for line in open(path).read().strip().split("\n")])


@pytest.mark.gpu
def test_plain_kernels_and_sampling_options(model_dirs, tmp_path, capsys):
    """--kernels plain computes the same function on the slow kernels; a sampling run repeats with its seed."""
    prompts = _prompts("D", [70, 9], 740)
    base = [model_dirs["D"], "--tokens", "6", "--stop-ids", ""] + _flags(prompts)
    _, fast, s_fast = _main(base + ["--trace", str(tmp_path / "fast.txt")], capsys)
    _, plain, s_plain = _main(base + ["--kernels", "plain", "--trace", str(tmp_path / "plain.txt")], capsys)
    assert s_fast["backend"].endswith("fast") and s_plain["backend"].endswith("plain")
    rows_fast, rows_plain = fast.strip().splitlines(), plain.strip().splitlines()
    assert len(rows_fast) == len(rows_plain) == 2 and all(len(r.split()) == 6 for r in rows_fast)
    a, b = _read_trace(tmp_path / "fast.txt"), _read_trace(tmp_path / "plain.txt")
    assert a.shape == b.shape == (79, TINY["D"]["vocab_size"]) and not torch.equal(a, b)
    assert float(((a - b).abs().max(dim=1).values / b.abs().max(dim=1).values).max()) <= 1e-2
    sample = base + ["--temperature", "0.8", "--top-k", "20", "--top-p", "0.9", "--seed", "7"]
    assert _main(sample, capsys)[1] == _main(sample, capsys)[1]
    assert _main(sample, capsys)[1] != _main(sample[:-1] + ["8"], capsys)[1]
