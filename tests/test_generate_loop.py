"""The generation loop's decisions, over a stand-in engine and sampler on the CPU."""
import pytest
import torch

from smolmoe_c99_b200.engine.generate import GenerationOptions, GenerationStats, TokenSink, generate


class FakeEngine:
    """Logits are one-hot: after token t the next token is (t + 1) % vocab."""

    def __init__(self, vocab=50, max_seq_len=64, slots=4):
        self.vocab, self.max_seq_len = vocab, max_seq_len
        self.free, self.open, self.lengths = list(range(slots)), set(), {}
        self.steps = []          # (kind, slots, tokens fed)
        self.max_open = 0

    def open_sequence(self):
        s = self.free.pop(0); self.open.add(s); self.lengths[s] = 0
        self.max_open = max(self.max_open, len(self.open))
        return s

    def close_sequence(self, slot):
        assert slot in self.open, "closed twice"
        self.open.remove(slot); self.free.append(slot); self.free.sort()

    def step(self, slots, tokens, want=None):
        if isinstance(tokens, torch.Tensor):
            fed = [[int(t)] for t in tokens.tolist()]
            self.steps.append(("decode", list(slots), fed))
        else:
            fed = [list(t) for t in tokens]
            self.steps.append(("prefill", list(slots), fed))
        for s, f in zip(slots, fed):
            assert s in self.open
            self.lengths[s] += len(f)
            assert self.lengths[s] <= self.max_seq_len
        logits = torch.zeros(len(slots), self.vocab)
        for i, f in enumerate(fed):
            logits[i, (f[-1] + 1) % self.vocab] = 1.0
        return logits

    def synchronize(self):
        pass


class FakeSampler:
    def new_states(self, indices):
        return torch.tensor(list(indices), dtype=torch.int32)

    def choose(self, logits, states):
        return logits.argmax(dim=1).to(torch.int32)

    @staticmethod
    def select(values, keep):
        return values[torch.tensor(list(keep), dtype=torch.long)]


def test_batches_follow_one_another_and_slots_are_used_again():
    eng = FakeEngine(slots=2)
    prompts = [[1, 2], [10], [20, 21, 22], [30], [40]]
    out = generate(eng, FakeSampler(), prompts, GenerationOptions(max_new_tokens=3, batch=2))
    assert [c.tokens for c in out] == [[3, 4, 5], [11, 12, 13], [23, 24, 25], [31, 32, 33], [41, 42, 43]]
    assert all(c.finish_reason == "length" for c in out)
    prefills = [s for s in eng.steps if s[0] == "prefill"]
    assert [p[2] for p in prefills] == [[[1, 2], [10]], [[20, 21, 22], [30]], [[40]]]     # whole prompts, unequal lengths
    assert [p[1] for p in prefills] == [[0, 1], [0, 1], [0]]                             # the same slots again
    assert eng.max_open == 2 and not eng.open


def test_the_last_token_is_not_fed_back():
    eng = FakeEngine()
    generate(eng, FakeSampler(), [[5]], GenerationOptions(max_new_tokens=4, batch=1))
    decodes = [s[2] for s in eng.steps if s[0] == "decode"]
    assert decodes == [[[6]], [[7]], [[8]]]            # 4 tokens come from 1 prefill and 3 decode steps
    assert eng.lengths[0] == 4


def test_stop_tokens_end_sequences_early_and_shrink_the_batch():
    eng = FakeEngine()
    prompts = [[1], [7], [20]]
    out = generate(eng, FakeSampler(), prompts, GenerationOptions(max_new_tokens=6, stop_token_ids=(3, 9), batch=3))
    assert [c.tokens for c in out] == [[2, 3], [8, 9], [21, 22, 23, 24, 25, 26]]         # the stop token is reported
    assert [c.finish_reason for c in out] == ["stop", "stop", "length"]
    decodes = [s for s in eng.steps if s[0] == "decode"]
    assert decodes[0][2] == [[2], [8], [21]]
    assert all(d[2][0][0] >= 22 and len(d[1]) == 1 for d in decodes[1:])               # the stop tokens were not fed back
    assert not eng.open


def test_prompt_and_new_tokens_must_fit():
    eng = FakeEngine(max_seq_len=8)
    with pytest.raises(ValueError, match="exceed the context"):
        generate(eng, FakeSampler(), [[1] * 6], GenerationOptions(max_new_tokens=3))
    assert not eng.steps and not eng.open
    with pytest.raises(ValueError, match="empty"):
        generate(eng, FakeSampler(), [[]], GenerationOptions())


def test_sink_sees_every_token_and_can_cancel():
    class Sink(TokenSink):
        def __init__(self):
            self.seen, self.calls = [], 0
        def on_token(self, request, token, last):
            self.seen.append((request, token, last))
        def should_stop(self):
            self.calls += 1
            return self.calls >= 2
    eng, sink = FakeEngine(), Sink()
    out = generate(eng, FakeSampler(), [[1], [5], [9]], GenerationOptions(max_new_tokens=5, batch=2), sink)
    assert sink.seen == [(0, 2, False), (1, 6, False), (0, 3, False), (1, 7, False)]
    assert [c.finish_reason for c in out] == ["cancelled"] * 3 and out[2].tokens == []
    assert not eng.open                                  # slots are given back on the way out


def test_slots_are_given_back_when_a_step_fails():
    class Broken(FakeEngine):
        def step(self, slots, tokens, want=None):
            if isinstance(tokens, torch.Tensor):
                raise RuntimeError("device fault")
            return super().step(slots, tokens, want)
    eng = Broken()
    with pytest.raises(RuntimeError, match="device fault"):
        generate(eng, FakeSampler(), [[1], [2]], GenerationOptions(max_new_tokens=3, batch=2))
    assert not eng.open and eng.free == [0, 1, 2, 3]


def test_stats_count_tokens():
    eng, stats = FakeEngine(), GenerationStats()
    ticks = iter(range(100))
    generate(eng, FakeSampler(), [[1, 2, 3], [4]], GenerationOptions(max_new_tokens=3, batch=2), stats=stats,
             clock=lambda: float(next(ticks)))
    assert stats.prompt_tokens == 4 and stats.generated_tokens == 6 and stats.decode_forwards == 4 and stats.batches == 1
    d = stats.as_dict()
    assert d["prefill_tokens_per_second"] == 4.0 and d["decode_tokens_per_second"] == 4.0


def test_zero_new_tokens():
    eng = FakeEngine()
    out = generate(eng, FakeSampler(), [[1]], GenerationOptions(max_new_tokens=0))
    assert out[0].tokens == [] and out[0].finish_reason == "length" and not eng.steps


class TwoHalfEngine(FakeEngine):
    """An engine that offers the one-token step in two halves, as the CUDA engine does."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.prepared, self.launched = 0, 0

    def prepare_decode(self, slots):
        self.prepared += 1
        return ("handle", tuple(slots), tuple(self.lengths[s] for s in slots))

    def launch_prepared(self, prepared, tokens):
        _, slots, starts = prepared
        assert tuple(self.lengths[s] for s in slots) == starts, "the sequences moved between the halves"
        self.launched += 1
        return self.step(list(slots), tokens)


def test_a_two_half_step_changes_no_decision():
    prompts = [[1], [7], [20]]
    opts = GenerationOptions(max_new_tokens=6, stop_token_ids=(9, 23), batch=3)
    plain, halves = FakeEngine(), TwoHalfEngine()
    want = generate(plain, FakeSampler(), prompts, opts)
    got = generate(halves, FakeSampler(), prompts, opts)
    assert [(c.tokens, c.finish_reason) for c in got] == [(c.tokens, c.finish_reason) for c in want]
    assert halves.steps == plain.steps                 # the same tokens fed to the same slots: no stop token, no last token
    assert halves.launched >= 1 and halves.prepared > halves.launched   # a step whose batch shrank was redone the plain way
    assert not halves.open


def test_an_engine_that_runs_ahead_of_the_host():
    """With ``runs_ahead`` the next step is launched before the host has read the chosen tokens. The completions are
    the same; a sequence that ended on a stop token has taken that one step into a slot that is closed right after;
    the last token the limit allows is still never fed; a row's logits of the step that ran ahead are dropped with
    its sequence."""
    class Ahead(TwoHalfEngine):
        runs_ahead = True

    prompts = [[1], [7], [20], [30]]
    opts = GenerationOptions(max_new_tokens=6, stop_token_ids=(9, 23), batch=4)
    plain, ahead = FakeEngine(), Ahead()
    want = generate(plain, FakeSampler(), prompts, opts)
    stats = GenerationStats()
    got = generate(ahead, FakeSampler(), prompts, opts, stats=stats)
    assert [(c.tokens, c.finish_reason) for c in got] == [(c.tokens, c.finish_reason) for c in want]
    assert [c.tokens for c in got] == [[2, 3, 4, 5, 6, 7], [8, 9], [21, 22, 23], [31, 32, 33, 34, 35, 36]]
    fed = [s for s in ahead.steps if s[0] == "decode"]
    # every step but the ones after a batch shrank came through launch_prepared, with the whole batch of that moment
    assert [tuple(f[0] for f in s[2]) for s in fed][:3] == [(2, 8, 21, 31), (3, 9, 22, 32), (4, 23, 33)]
    # the stop tokens 9 and 23 were fed once (the step that ran ahead) and their sequences closed; nothing followed them
    assert sum(1 for s in fed for f in s[2] if f[0] == 9) == 1 and sum(1 for s in fed for f in s[2] if f[0] == 23) == 1
    assert all(f[0] not in (10, 24) for s in fed for f in s[2])
    # the sixth token of a request is its last: never fed
    assert all(f[0] not in (7, 36) for s in fed for f in s[2])
    assert stats.generated_tokens == 6 + 2 + 3 + 6 and stats.decode_forwards == 4 + 3 + 2 + 2 + 2     # the forwards that counted
    assert not ahead.open and ahead.free == [0, 1, 2, 3]
