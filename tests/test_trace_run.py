"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
from compare import REL
from tiny import TINY, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _trace(requests, batches, prompt_lens):
    """Steps for batches that follow one another: prompts together, then one token each;
    a request is listed under "end" in the step that brings its last token."""
    steps, expect = [], []      # expect: per step, list of (request, position)
    for batch in batches:
        done = {r: prompt_lens[r] for r in batch}
        entries = [{"id": r, "tokens": requests[r][:prompt_lens[r]], "want": list(range(prompt_lens[r]))} for r in batch]
        # the second request of every batch asks for nothing in its prompt step
        if len(entries) > 1:
            entries[1]["want"] = []
        wanted = [(e["id"], p) for e in entries for p in e["want"]]
        steps.append({"step": len(steps), "entries": entries, "end": [r for r in batch if done[r] == len(requests[r])]})
        expect.append(wanted)
        live = [r for r in batch if done[r] < len(requests[r])]
        while live:
            entries = [{"id": r, "tokens": [requests[r][done[r]]], "want": [0]} for r in live]
            expect.append([(r, done[r]) for r in live])
            for r in live:
                done[r] += 1
            steps.append({"step": len(steps), "entries": entries, "end": [r for r in live if done[r] == len(requests[r])]})
            live = [r for r in live if done[r] < len(requests[r])]
    return steps, expect


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run(model_dirs, tmp_path, name, dtype):
    vocab = TINY[name]["vocab_size"]
    lengths = [9, 40, 23, 64, 5]
    requests = {f"q{i}": random_tokens(n, vocab, 30 + i) for i, n in enumerate(lengths)}
    batches = [["q0", "q1", "q2"], ["q3", "q4"], ["q1"]]
    prompt_lens = {r: max(1, len(t) - 7) for r, t in requests.items()}
    steps, expect = _trace(requests, batches, prompt_lens)
    out = tmp_path / "out"
    # 3 live requests of at most 64 tokens, each rounded up to a multiple of 64
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "192"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    want = {r: plain_model.forward(model_dirs[name], t, round_like_bf16_engine=(dtype == "bfloat16")) for r, t in requests.items()}
    for i, wanted in enumerate(expect):
        path = out / f"{i}.f32"
        if not wanted:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab))
        for row, (r, pos) in enumerate(wanted):
            bound = REL[dtype] * float(want[r][pos].abs().max())
            assert float((got[row] - want[r][pos]).abs().max()) <= bound, f"step {i}, request {r}, position {pos}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_takes_portions_and_requests_that_join(model_dirs, tmp_path, dtype):
    """A prompt in portions of 10 tokens; a second request whose prompt arrives while the first decodes."""
    vocab = TINY["B"]["vocab_size"]
    a, b = random_tokens(50, vocab, 71), random_tokens(30, vocab, 72)
    steps, expect = [], []
    for at in range(0, 40, 10):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": a[at:at + 10], "want": [0, 9]}], "end": []})
        expect.append([("a", at), ("a", at + 9)])
    steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[40]], "want": [0]},
                                                   {"id": "b", "tokens": b[:25], "want": [3, 24]}], "end": []})
    expect.append([("a", 40), ("b", 3), ("b", 24)])
    for k in range(5):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[41 + k]], "want": [0]},
                                                       {"id": "b", "tokens": [b[25 + k]], "want": [0]}],
                      "end": ["b"] if k == 4 else []})
        expect.append([("a", 41 + k), ("b", 25 + k)])
    steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": a[46:], "want": [3]}], "end": ["a"]})
    expect.append([("a", 49)])
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["B"], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = {"a": plain_model.forward(model_dirs["B"], a, round_like_bf16_engine=(dtype == "bfloat16")),
            "b": plain_model.forward(model_dirs["B"], b, round_like_bf16_engine=(dtype == "bfloat16"))}
    for i, wanted in enumerate(expect):
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(len(wanted), vocab))
        for row, (r, pos) in enumerate(wanted):
            bound = REL[dtype] * float(want[r][pos].abs().max())
            assert float((got[row] - want[r][pos]).abs().max()) <= bound, f"step {i}, request {r}, position {pos}"


def test_trace_run_refuses_more_tokens_than_it_was_sized_for(model_dirs, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": [64]}, {"id": "b", "tokens": [2] * 10, "want": []}], "end": []}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["A"], "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "128"],
                          input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "exceeds the cache" in proc.stderr      # 65 -> 128 and 10 -> 64 make 192 > 128
