"""The engine against the plain implementation under every way of cutting the work: each
request alone and whole; the last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again; prompts in
portions onto the cache; new requests that join running ones in one step; a sequence cut back
and fed again."""
import pytest
import torch

import plain_model
import replay
from compare import check_logits
from tiny import TINY, random_tokens

pytestmark = pytest.mark.gpu

# absolute bound for the few single rows compared below; whole runs are held to the bounds of compare.py
TOL = {"float32": 5e-6, "bfloat16": 1e-2}


def _requests(name, lengths, seed):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


def _plain(model_dir, requests, dtype):
    return {rid: plain_model.forward(model_dir, toks, round_like_bf16_engine=(dtype == "bfloat16"))
            for rid, toks in requests.items()}


def _engine(model_dir, dtype, max_tokens=4096):
    from smolmoe_c99_b200.engine.engine import Engine
    return Engine(model_dir, dtype, max_tokens=max_tokens)


def _check(got, want, dtype, what):
    """Largest difference against the row's largest logit, top-1 agreement outside near-ties and mean KL."""
    check_logits(got, want, dtype, what)


LENGTHS = {"A": [5, 11, 17, 64, 65, 100, 128], "B": [1, 23, 40, 41, 64, 96], "C": [3, 99, 100, 101, 129, 300],
           "D": [2, 127, 128, 129, 260, 700]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_all_cuts_agree_with_plain(model_dirs, name, dtype):
    requests = _requests(name, LENGTHS[name], 10)
    want = _plain(model_dirs[name], requests, dtype)
    engine = _engine(model_dirs[name], dtype)
    tol = dtype
    got_whole = replay.whole(engine, requests)
    _check(got_whole, want, tol, "whole")
    got_tail = replay.tail_decoded(engine, requests)
    _check(got_tail, want, tol, "tail decoded")
    ids = list(requests)
    batches = [{r: requests[r] for r in ids[:3]}, {r: requests[r] for r in ids[3:]}, {r: requests[r] for r in ids[:2]}]
    prompt_lens = {r: max(1, len(requests[r]) * 2 // 3) for r in ids}
    got_batched = replay.batched(engine, batches, prompt_lens)
    _check(got_batched, want, tol, "batched")
    assert engine.cache.slots.free_count == engine.cache.max_slots
    assert all(g.ledger.held_count == 0 for g in engine.cache.groups)
    if dtype == "float32":
        # the 32-bit path computes every output in an order that does not depend on the cut
        for rid in requests:
            assert torch.equal(got_whole[rid], got_tail[rid]), f"{rid}: whole and tail-decoded logits differ in bits"
            assert torch.equal(got_whole[rid], got_batched[rid]), f"{rid}: whole and batched logits differ in bits"


# ---- sequences that go on by any number of tokens, and mixed steps ------------------------------------------------
PORTION_LENGTHS = {"A": [5, 64, 65, 128], "B": [1, 41, 96], "C": [3, 100, 129, 300], "D": [2, 129, 260, 700]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompts_in_portions_onto_the_cache(model_dirs, name, dtype):
    """Portions of 1, 7, 64 and 100 tokens (B and C have windowed layers: a portion's first queries still see
    keys whose places in the ring its last tokens take), then the last tokens one by one."""
    requests = _requests(name, PORTION_LENGTHS[name], 70)
    want = _plain(model_dirs[name], requests, dtype)
    engine = _engine(model_dirs[name], dtype)
    got_whole = replay.whole(engine, requests) if dtype == "float32" else None
    for size, tail in ((1, 0), (7, 5), (64, 0), (100, 32)):
        got = replay.portions(engine, requests, size, tail)
        _check(got, want, dtype, f"portions of {size}")
        if dtype == "float32":
            for rid in requests:
                assert torch.equal(got[rid], got_whole[rid]), f"{rid}: portions of {size} and whole differ in bits"
    assert engine.cache.slots.free_count == engine.cache.max_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_new_requests_join_running_ones(model_dirs, name, dtype):
    """A mixed step: prompts (whole, and in portions of 9) beside the single tokens of requests that decode."""
    lens = PORTION_LENGTHS[name]
    requests = _requests(name, lens + lens[::-1][:2], 90)
    ids = list(requests)
    first, second = {r: requests[r] for r in ids[:2]}, {r: requests[r] for r in ids[2:]}
    prompt_lens = {r: max(1, len(requests[r]) * 3 // 4) for r in ids}
    want = _plain(model_dirs[name], requests, dtype)
    engine = _engine(model_dirs[name], dtype)
    got_whole = replay.whole(engine, requests) if dtype == "float32" else None
    for portion in (0, 9):
        got = replay.joined(engine, first, second, prompt_lens, after=3, portion=portion)
        _check(got, want, dtype, f"joined (portion {portion})")
        if dtype == "float32":
            for rid in requests:
                assert torch.equal(got[rid], got_whole[rid]), f"{rid}: joined and whole differ in bits"
    assert engine.cache.slots.free_count == engine.cache.max_slots
    assert all(g.ledger.held_count == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_cut_back_then_several_tokens(model_dirs, name, dtype):
    """``truncate`` marks the positions from n on as dead; feeding them again in one step gives the same logits."""
    requests = _requests(name, PORTION_LENGTHS[name][1:], 110)
    want = _plain(model_dirs[name], requests, dtype)
    engine = _engine(model_dirs[name], dtype)
    got = replay.truncated(engine, requests, {r: len(t) // 3 for r, t in requests.items()})
    _check(got, want, dtype, "cut back")


def test_a_step_over_max_step_tokens_is_refused_and_the_next_works(model_dirs):
    from smolmoe_c99_b200.engine.engine import Engine, StepError
    engine = Engine(model_dirs["A"], "float32", max_tokens=1024, max_step_tokens=16)
    a, b = engine.open_sequence(), engine.open_sequence()
    with pytest.raises(StepError, match="max_step_tokens"):
        engine.step([a, b], [[1] * 10, [2] * 7])
    assert engine.length(a) == 0 and engine.length(b) == 0
    toks = random_tokens(30, 256, 5)
    rows = [engine.step([a], [toks[i:i + 16]], [list(range(len(toks[i:i + 16])))]).cpu() for i in (0, 16)]
    want = plain_model.forward(model_dirs["A"], toks)
    assert float((torch.cat(rows) - want).abs().max()) <= TOL["float32"]
