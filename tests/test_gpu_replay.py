"""The engine against the plain implementation under every way of cutting the work: each
request alone and whole; the last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

import plain_model
import replay
from tiny import TINY, random_tokens

pytestmark = pytest.mark.gpu

# max |engine - plain| over all logits. float32: both sides compute in float with different
# summation orders; logits are O(1). bfloat16: the plain side rounds where the engine stores.
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


def _check(got, want, tol, what):
    for rid in want:
        assert got[rid].shape == want[rid].shape, f"{what} {rid}: shape {got[rid].shape} vs {want[rid].shape}"
        diff = (got[rid] - want[rid]).abs().max(dim=1).values
        worst = int(diff.argmax())
        assert float(diff.max()) <= tol, f"{what} {rid}: first position over tolerance " \
            f"{int((diff > tol).nonzero()[0])}, worst {float(diff.max()):.3g} at position {worst} of {len(diff)}"


LENGTHS = {"A": [5, 11, 17, 64, 65, 100, 128], "B": [1, 23, 40, 41, 64, 96], "C": [3, 99, 100, 101, 129, 300],
           "D": [2, 127, 128, 129, 260, 700]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_all_cuts_agree_with_plain(model_dirs, name, dtype):
    requests = _requests(name, LENGTHS[name], 10)
    want = _plain(model_dirs[name], requests, dtype)
    engine = _engine(model_dirs[name], dtype)
    tol = TOL[dtype]
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
