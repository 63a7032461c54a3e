"""Generation through the Python entry point, long decoding, the first tokens of a sequence and
slots that are used again, against the plain implementation."""
import pytest
import torch

import plain_model
from tiny import TINY, random_tokens

pytestmark = pytest.mark.gpu
TOL = {"float32": 5e-6, "bfloat16": 1e-2}


def _model(model_dir, dtype, name, batch=4, context=None):
    from smolmoe_c99_b200 import Model
    return Model.from_folder(model_dir, dtype, context=context or TINY[name]["max_position_embeddings"], batch=batch)


def _check_greedy(model_dir, dtype, prompt, tokens):
    """Every generated token is the plain implementation's best token, unless the plain margin
    at that place is within what rounding can move (then the continuation may differ)."""
    seq = list(prompt) + list(tokens)
    logits = plain_model.forward(model_dir, seq[:-1], round_like_bf16_engine=(dtype == "bfloat16"))
    for i, tok in enumerate(tokens):
        row = logits[len(prompt) - 1 + i]
        if int(row.argmax()) != tok:
            top = torch.topk(row, 2).values
            assert float(top[0] - top[1]) <= 2 * TOL[dtype], f"token {i}: {tok} vs plain {int(row.argmax())}"
            return


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    vocab = TINY[name]["vocab_size"]
    lengths = [5, 11, 17] if name == "A" else [1, 23]               # the batches BASELINE.json names
    prompts = [random_tokens(n, vocab, 50 + n) for n in lengths]
    model = _model(model_dirs[name], dtype, name)
    together = model.generate(prompts, tokens=8, stop_ids=())
    assert [len(t) for t in together] == [8] * len(prompts)
    for p, t in zip(prompts, together):
        _check_greedy(model_dirs[name], dtype, p, t)
    if dtype == "float32":
        alone = [model.generate([p], tokens=8, stop_ids=())[0] for p in prompts]
        assert alone == together                                  # what else is in the batch changes nothing
    assert model.engine.cache.slots.free_count == model.engine.cache.max_slots


def test_stop_ids_end_a_sequence_and_the_rest_goes_on(model_dirs):
    model = _model(model_dirs["A"], "float32", "A")
    prompts = [random_tokens(n, 256, 70 + n) for n in (4, 9, 6)]
    free_run = model.generate(prompts, tokens=12, stop_ids=())
    stop = free_run[1][3]                                         # request 1 ends at its fourth token
    out = model.generate(prompts, tokens=12, stop_ids=[stop], return_completions=True)
    assert out[1].tokens == free_run[1][:free_run[1].index(stop) + 1] and out[1].finish_reason == "stop"
    for i in (0, 2):
        cut = free_run[i].index(stop) + 1 if stop in free_run[i] else 12
        assert out[i].tokens == free_run[i][:cut]
    # the configuration's own eos id is the default stop
    assert model.engine.spec.stop_token_ids == (255,)


def test_temperature_sampling_repeats_with_its_seed_and_follows_the_plain_sampler(model_dirs):
    model = _model(model_dirs["B"], "float32", "B")
    prompts = [random_tokens(n, 384, 80 + n) for n in (1, 23)]
    a = model.generate(prompts, tokens=6, temperature=0.8, seed=5, stop_ids=())
    assert a == model.generate(prompts, tokens=6, temperature=0.8, seed=5, stop_ids=())
    assert a != model.generate(prompts, tokens=6, temperature=0.8, seed=6, stop_ids=())
    from smolmoe_c99_b200.sampling import sequence_seed
    for i, (p, toks) in enumerate(zip(prompts, a)):
        state, seq = sequence_seed(5, i), list(p)
        for tok in toks:                                           # teacher-forced along what the engine chose
            row = plain_model.forward(model_dirs["B"], seq)[-1]
            want, state = plain_model.sample(row.tolist(), 0.8, 40, 0.95, state)
            assert want == tok
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """700 positions, the last 550 one token at a time: the windowed group's ring of 128
    positions wraps four times, pages are added as the sequence grows."""
    from smolmoe_c99_b200.engine.engine import Engine
    toks = random_tokens(700, 300, 91)
    want = plain_model.forward(model_dirs["C"], toks, round_like_bf16_engine=(dtype == "bfloat16"))
    engine = Engine(model_dirs["C"], dtype, max_tokens=1024)
    slot = engine.open_sequence()
    rows = [engine.step([slot], [toks[:150]], [list(range(150))]).cpu()]
    for t in toks[150:]:
        rows.append(engine.step([slot], [[t]], [[0]]).cpu())
    got = torch.cat(rows)
    diff = (got - want).abs().max(dim=1).values
    assert float(diff.max()) <= TOL[dtype], f"first position over tolerance: {int((diff > TOL[dtype]).nonzero()[0])}"
    engine.close_sequence(slot)


def test_long_prompt_then_long_decoding_at_head_size_64(model_dirs):
    """A prompt of 1,500 positions through the tcgen05 prefill attention, then 120 tokens one at a time: the decode
    graph's span doubles on the way (2,048 is crossed at no point, 1,536 positions are in one span) and the cluster's
    CTAs hold their shares in one buffer."""
    from smolmoe_c99_b200.engine.engine import Engine
    toks = random_tokens(1620, 331, 77)
    want = plain_model.forward(model_dirs["D"], toks, round_like_bf16_engine=True)
    engine = Engine(model_dirs["D"], "bfloat16", max_tokens=4096)
    slot = engine.open_sequence()
    rows = [engine.step([slot], [toks[:1500]], [list(range(1500))]).cpu()]
    for t in toks[1500:]:
        rows.append(engine.step([slot], [[t]], [[0]]).cpu())
    engine.check_status()
    got = torch.cat(rows)
    diff = (got - want).abs().max(dim=1).values
    assert float(diff.max()) <= TOL["bfloat16"], f"first position over tolerance: {int((diff > TOL['bfloat16']).nonzero()[0])}"
    engine.close_sequence(slot)


def test_many_long_sequences_decode_with_streamed_attention(model_dirs):
    """More (sequence, kv head) pairs than the GPU holds clusters, hundreds of positions each: the decode attention
    streams every CTA's share tile by tile (TMA boxes of the paged pool). One sequence of the 110 is checked against
    the plain implementation through its prompt's end and 12 tokens one at a time; the others only share the batch."""
    import ctypes
    from smolmoe_c99_b200.engine.engine import Engine
    cfg = TINY["D"]
    n_seqs, n_prompt, n_more = 110, 890, 12
    engine = Engine(model_dirs["D"], "bfloat16", max_tokens=n_seqs * 960, max_slots=n_seqs)
    plan = (ctypes.c_int * 4)()
    ops = engine.runtime.ops
    ops._check(ops.lib.sm_attention_decode_plan(n_seqs, cfg["num_attention_heads"], cfg["num_key_value_heads"], 64, 0, 1024, plan))
    assert plan[1] == 0, f"this batch is meant for the streaming kernel, the plan is {list(plan)}"
    toks = random_tokens(n_prompt + n_more, cfg["vocab_size"], 91)
    want = plain_model.forward(model_dirs["D"], toks, round_like_bf16_engine=True)
    g = torch.Generator().manual_seed(4)
    others = [random_tokens(int(n), cfg["vocab_size"], 200 + i)
              for i, n in enumerate(torch.randint(300, 900, (n_seqs - 1,), generator=g))]
    slots = [engine.open_sequence() for _ in range(n_seqs)]
    at = 37                                           # the checked sequence sits in the middle of the batch
    prompts = others[:at] + [toks[:n_prompt]] + others[at:]
    first = engine.step(slots, prompts)               # the last position of every prompt
    rows = [first[at:at + 1].cpu()]
    feed = [[1 + (i % 7)] for i in range(n_seqs)]
    for t in toks[n_prompt:-1]:
        feed[at] = [t]
        rows.append(engine.step(slots, feed)[at:at + 1].cpu())
    engine.check_status()
    got = torch.cat(rows)
    diff = (got - want[n_prompt - 1:n_prompt - 1 + len(rows)]).abs().max(dim=1).values
    assert float(diff.max()) <= TOL["bfloat16"], f"first step over tolerance: {int((diff > TOL['bfloat16']).nonzero()[0])}"
    for s in slots:
        engine.close_sequence(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    from smolmoe_c99_b200.engine.engine import Engine
    engine = Engine(model_dirs[name], dtype, max_tokens=512)
    toks = random_tokens(4, TINY[name]["vocab_size"], 17)
    want = plain_model.forward(model_dirs[name], toks, round_like_bf16_engine=(dtype == "bfloat16"))
    for first in (1, 2, 3):                     # prompts of one, two and three tokens, then one by one
        slot = engine.open_sequence()
        rows = [engine.step([slot], [toks[:first]], [list(range(first))]).cpu()]
        rows += [engine.step([slot], [[t]], [[0]]).cpu() for t in toks[first:]]
        engine.close_sequence(slot)
        assert float((torch.cat(rows) - want).abs().max()) <= TOL[dtype], f"prompt of {first}"


def test_a_used_slot_shows_nothing_of_its_past(model_dirs):
    """Fill every page with a loud sequence, give the slots back, then run a quiet one in them."""
    from smolmoe_c99_b200.engine.engine import Engine
    engine = Engine(model_dirs["A"], "bfloat16", max_tokens=256, max_slots=2)
    loud = [random_tokens(128, 256, 5), random_tokens(128, 256, 6)]
    slots = [engine.open_sequence(), engine.open_sequence()]
    engine.step(slots, loud)
    for g in engine.cache.groups:
        g.k.mul_(50.0); g.v.mul_(50.0)          # what lies in the pages now would swamp any softmax
    for s in slots:
        engine.close_sequence(s)
    toks = random_tokens(70, 256, 8)
    want = plain_model.forward(model_dirs["A"], toks, round_like_bf16_engine=True)
    slot = engine.open_sequence()
    rows = [engine.step([slot], [toks[:20]], [list(range(20))]).cpu()]
    rows += [engine.step([slot], [[t]], [[0]]).cpu() for t in toks[20:]]
    assert float((torch.cat(rows) - want).abs().max()) <= TOL["bfloat16"]


def test_step_refuses_what_it_cannot_run(model_dirs):
    from smolmoe_c99_b200.engine.engine import Engine, StepError
    engine = Engine(model_dirs["A"], "float32", max_tokens=128, max_slots=2)
    s = engine.open_sequence()
    with pytest.raises(StepError, match="out of vocabulary"):
        engine.step([s], [[1, 256]])
    with pytest.raises(StepError, match="not open"):
        engine.step([5], [[1]])
    with pytest.raises(StepError, match="exceeds the cache"):
        engine.step([s], [[1] * 129])
    engine.step([s], [[1, 2, 3]])
    t = engine.open_sequence()
    with pytest.raises(StepError, match="appears twice"):
        engine.step([s, s], [[4], [5, 6]])
    with pytest.raises(StepError, match="wanted place"):
        engine.step([s], [[4]], [[1]])
    # after the refusals the engine still works (the reference: tests/test_errors.c); a sequence that goes on and
    # one that starts share a step
    assert engine.step([s, t], [[4], [5, 6]]).shape == (2, 256) and engine.length(s) == 4 and engine.length(t) == 2
