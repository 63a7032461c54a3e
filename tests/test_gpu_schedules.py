"""Whole-model checks of the schedules and dispatch branches that small batches never reach: decode batches of 12,
24 and 64 sequences (the kernels change at 8, 16 and 64 tokens), head size 128, the layer sizes of a real
checkpoint, a decode graph replayed with only some rows wanted, graphs dropped and captured again, and a one-token
step prepared ahead that finds the cache full. All against the plain implementation."""
import pytest
import torch

import plain_model
import replay
from compare import REL_WIDE, check_logits
from tiny import REAL_0_5B_2_LAYERS, TINY, random_tokens

pytestmark = pytest.mark.gpu
TOL = {"float32": 5e-6, "bfloat16": 1e-2}


def _plain(model_dir, requests, dtype):
    return {rid: plain_model.forward(model_dir, toks, round_like_bf16_engine=(dtype == "bfloat16"))
            for rid, toks in requests.items()}


def _check(got, want, dtype, what, bound=None):
    check_logits(got, want, dtype, what, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_wide_batches_of_unequal_lengths(model_dirs, name, dtype):
    """64 requests of 2 to 90 tokens. Batches of 12, 24 and 64 start together and decode their last 3 to 12 tokens,
    so the batch passes through many sizes as requests end; slots are used again from batch to batch."""
    from smolmoe_c99_b200.engine.engine import Engine
    vocab = TINY[name]["vocab_size"]
    g = torch.Generator().manual_seed(5)
    lengths = torch.randint(14, 91, (64,), generator=g).tolist()
    lengths[3], lengths[40] = 2, 13
    requests = {f"r{i}": random_tokens(n, vocab, 200 + i) for i, n in enumerate(lengths)}
    prompt_lens = {r: max(1, len(t) - 3 - (i % 10)) for i, (r, t) in enumerate(requests.items())}
    want = _plain(model_dirs[name], requests, dtype)
    engine = Engine(model_dirs[name], dtype, max_tokens=64 * 128, max_slots=64)
    ids = list(requests)
    first = {r: requests[r] for r in ids[:12]}
    got_whole, got_tail = replay.whole(engine, first), replay.tail_decoded(engine, first)
    _check(got_whole, {r: want[r] for r in first}, dtype, "whole")
    _check(got_tail, {r: want[r] for r in first}, dtype, "tail decoded")
    for batch_ids in (ids[:12], ids[12:36], ids):
        batch = {r: requests[r] for r in batch_ids}
        got = replay.batched(engine, [batch], prompt_lens)
        _check(got, {r: want[r] for r in batch}, dtype, f"batch of {len(batch)}")
        if dtype == "float32":
            for r in first:
                if r in got:
                    assert torch.equal(got[r], got_whole[r]), f"{r}: batch of {len(batch)} and whole differ in bits"
    assert engine.cache.slots.free_count == engine.cache.max_slots
    assert all(grp.ledger.held_count == 0 for grp in engine.cache.groups)
    engine.check_status()


@pytest.mark.parametrize("name", ["D", "E"])
def test_long_prompts_on_the_two_cta_products(model_dirs, name):
    """Steps of more than 160 tokens take the two-CTA products and the q/k/v epilogue that rotates and stores (head
    sizes 64 and 128): a whole prompt, the same prompt in two portions (the second reads the cache), and two prompts
    in one step, two prompts in three portions (the tcgen05 attention reads keys and values from the cache's pages),
    against the plain implementation; and against the same engine with those products switched off."""
    from smolmoe_c99_b200.engine.engine import Engine
    vocab, longest = TINY[name]["vocab_size"], TINY[name]["max_position_embeddings"]
    n = min(900, longest - 20)
    requests = {"long": random_tokens(n, vocab, 71), "other": random_tokens(n - 250, vocab, 72)}
    want = _plain(model_dirs[name], requests, "bfloat16")
    engine = Engine(model_dirs[name], "bfloat16", max_tokens=4096, max_slots=4, use_graphs=False)
    rows = list(range(0, n, 37)) + [n - 1]

    def run(lists, cuts):
        slots = [engine.open_sequence() for _ in lists]
        out = [[] for _ in lists]
        at = 0
        for cut in cuts + [None]:
            part = [t[at:cut] for t in lists]
            live = [i for i, t in enumerate(part) if t]
            want_rows = [[r - at for r in rows if at <= r < at + len(part[i])] for i in live]
            lg = engine.step([slots[i] for i in live], [part[i] for i in live], want_rows)
            k = 0
            for i, w in zip(live, want_rows):
                out[i].append(lg[k:k + len(w)].clone())
                k += len(w)
            at = cut
        for s in slots:
            engine.close_sequence(s)
        return [torch.cat(o).cpu() for o in out]

    def picked(rid):
        return want[rid][[r for r in rows if r < len(requests[rid])]]

    ops = engine.runtime.ops
    whole = run([requests["long"]], [])[0]
    portions = run([requests["long"]], [n - 520])[0]          # 520 tokens onto a cache of the rest
    thirds = run([requests["long"], requests["other"]], [n - 610, n - 290])     # unequal sequences go on together, twice
    both = run([requests["long"], requests["other"]], [])
    ops.gemm_pair_enable(False)
    try:
        single = run([requests["long"]], [])[0]
    finally:
        ops.gemm_pair_enable(True)
    engine.check_status()
    for what, got, rid in (("whole", whole, "long"), ("two portions", portions, "long"), ("two prompts", both[0], "long"),
                           ("three portions", thirds[0], "long"), ("three portions", thirds[1], "other"),
                           ("two prompts", both[1], "other"), ("one-CTA products", single, "long")):
        _check({rid: got}, {rid: picked(rid)}, "bfloat16", what)
    assert float((whole - single).abs().max()) <= 1e-2 * float(single.abs().max())


@pytest.fixture(scope="module")
def real_size_dir(tmp_path_factory):
    from smolmoe_c99_b200.config import config_from_json
    from smolmoe_c99_b200.weights import write_random_model
    return write_random_model(config_from_json(REAL_0_5B_2_LAYERS), str(tmp_path_factory.mktemp("real") / "m"), 7)


def _fnv1a64(t: torch.Tensor) -> int:
    """FNV-1a over the raw bits of float logits, as the reference hashes them (src/main.c:311-319)."""
    h = 0xCBF29CE484222325
    for b in t.contiguous().view(torch.uint8).flatten().tolist():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_against_plain(real_size_dir, dtype):
    """Qwen2.5-0.5B's layer sizes with 2 of its 24 layers: three requests whole, with the tail decoded, in a batch
    and in portions; and two runs give the same bits (the reference: tests/models.test.ts:85-94)."""
    from smolmoe_c99_b200.engine.engine import Engine
    vocab = REAL_0_5B_2_LAYERS["vocab_size"]
    requests = {f"r{i}": random_tokens(n, vocab, 300 + i) for i, n in enumerate([40, 129, 200])}
    want = _plain(real_size_dir, requests, dtype)
    engine = Engine(real_size_dir, dtype, max_tokens=1024, max_slots=4)
    got = {"whole": replay.whole(engine, requests), "tail": replay.tail_decoded(engine, requests),
           "batched": replay.batched(engine, [requests], {r: len(t) * 2 // 3 for r, t in requests.items()}),
           "portions": replay.portions(engine, requests, 64, 8)}
    for cut, g in got.items():
        _check(g, want, dtype, cut, REL_WIDE)
    if dtype == "float32":
        for r in requests:
            for cut in ("tail", "batched", "portions"):
                assert torch.equal(got[cut][r], got["whole"][r]), f"{r}: {cut} and whole differ in bits"
    again = replay.tail_decoded(engine, {"r1": requests["r1"]})["r1"]
    assert _fnv1a64(again[-4:]) == _fnv1a64(got["tail"]["r1"][-4:])      # run to run, bit for bit, in both dtypes
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_graph_replayed_with_some_rows_wanted(model_dirs, dtype):
    from smolmoe_c99_b200.engine.engine import Engine
    engine = Engine(model_dirs["D"], dtype, max_tokens=2048, max_slots=4)
    toks = [random_tokens(n, 331, 400 + n) for n in (30, 9, 50)]
    slots = [engine.open_sequence() for _ in toks]
    engine.step(slots, [t[:-3] for t in toks], [[]] * 3)
    every = engine.step(slots, [[t[-3]] for t in toks]).clone()            # captures the graph for three sequences
    some = engine.step(slots, [[t[-2]] for t in toks], [[0], [], [0]]).clone()
    assert engine.step(slots, [[t[-1]] for t in toks], [[], [], []]) is None
    want = [plain_model.forward(model_dirs["D"], t, round_like_bf16_engine=(dtype == "bfloat16")) for t in toks]
    assert every.shape[0] == 3 and some.shape[0] == 2
    for i in range(3):
        assert float((every[i].cpu() - want[i][-3]).abs().max()) <= TOL[dtype]
    assert float((some[0].cpu() - want[0][-2]).abs().max()) <= TOL[dtype]
    assert float((some[1].cpu() - want[2][-2]).abs().max()) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_prompt_steps_of_a_shape_seen_before_are_replayed(model_dirs, name, dtype):
    """The second step of a shape (the same numbers of tokens and wanted rows) is captured, later ones are replayed
    with other tokens, slots and starting positions: the logits are those of an engine without graphs, bit for
    bit, for whole prompts and for prompts that go on in portions (C has a windowed group: its portions stay eager),
    and the shapes kept are few."""
    from smolmoe_c99_b200.engine.engine import Engine, MAX_STEP_GRAPHS
    vocab = TINY[name]["vocab_size"]
    engine = Engine(model_dirs[name], dtype, max_tokens=4096, max_slots=8)
    plain = Engine(model_dirs[name], dtype, max_tokens=4096, max_slots=8, use_graphs=False)
    longest = TINY[name]["max_position_embeddings"] // 2          # every prompt goes on by as many tokens again
    shapes = [(min(70, longest), 5), (33,), (min(70, longest), 5), (min(129, longest), min(64, longest - 1), 3), (17,)]
    for round_ in range(4):
        for si, lens in enumerate(shapes):
            toks = [random_tokens(2 * n, vocab, 1000 * round_ + 10 * si + i) for i, n in enumerate(lens)]
            want = [[n - 1] if i % 2 == 0 else [0, n // 2] for i, n in enumerate(lens)]
            got = []
            for e in (engine, plain):
                # slots in another order every round, so that the replay brings other slots and pages
                spare = [e.open_sequence() for _ in range(round_ % 3)]
                slots = [e.open_sequence() for _ in lens]
                first = e.step(slots, [t[:n] for t, n in zip(toks, lens)], want).clone()
                second = e.step(slots, [t[n:] for t, n in zip(toks, lens)], want).clone()    # goes on from the cache
                got.append((first, second))
                for slot in slots + spare:
                    e.close_sequence(slot)
            assert torch.equal(got[0][0], got[1][0]), f"round {round_}, whole prompts {lens}"
            assert torch.equal(got[0][1], got[1][1]), f"round {round_}, portions {lens}"
    assert 0 < len(engine._step_graphs) <= MAX_STEP_GRAPHS
    assert not plain._step_graphs
    # and against the plain implementation once, through a replayed graph
    toks = random_tokens(33, vocab, 77)
    slot = engine.open_sequence()
    lg = engine.step([slot], [toks], [[32]]).cpu()
    ref = plain_model.forward(model_dirs[name], toks, round_like_bf16_engine=(dtype == "bfloat16"))
    assert float((lg[0] - ref[32]).abs().max()) <= TOL[dtype]


def test_graphs_are_dropped_and_captured_again(model_dirs, monkeypatch):
    """More batch sizes than graphs are kept: the oldest is dropped, and a step of its size captures it again."""
    from smolmoe_c99_b200.engine import engine as engine_module
    monkeypatch.setattr(engine_module, "MAX_GRAPHS", 2)
    engine = engine_module.Engine(model_dirs["A"], "bfloat16", max_tokens=2048, max_slots=4)
    toks = [random_tokens(40, 256, 500 + i) for i in range(4)]
    want = [plain_model.forward(model_dirs["A"], t, round_like_bf16_engine=True) for t in toks]
    slots = [engine.open_sequence() for _ in toks]
    engine.step(slots, [t[:20] for t in toks], [[]] * 4)
    at = 20
    for live in ([0, 1, 2, 3], [0, 1, 2], [0, 1], [0], [0, 1, 2, 3], [1, 3], [0, 1, 2, 3]):
        assert len(engine._graphs) <= 2
        lg = engine.step([slots[i] for i in live], [[toks[i][engine.length(slots[i])]] for i in live]).cpu()
        for row, i in enumerate(live):
            pos = engine.length(slots[i]) - 1
            assert float((lg[row] - want[i][pos]).abs().max()) <= TOL["bfloat16"], f"batch {live}, sequence {i}"
    assert len(engine._graphs) == 2


def test_a_prepared_step_that_finds_the_cache_full(model_dirs):
    """``prepare_decode`` gives up (None) when no page is left and changes nothing; ``step`` then refuses cleanly,
    and once a sequence has given its pages back the others go on with the right logits."""
    from smolmoe_c99_b200.engine.engine import Engine, StepError
    engine = Engine(model_dirs["A"], "bfloat16", max_tokens=128, max_slots=2, max_seq_len=128)   # two pages of 64
    toks = [random_tokens(70, 256, 600 + i) for i in range(2)]
    want = [plain_model.forward(model_dirs["A"], t, round_like_bf16_engine=True) for t in toks]
    a, b = engine.open_sequence(), engine.open_sequence()
    engine.step([a, b], [toks[0][:62], toks[1][:62]], [[], []])
    for k in (62, 63):                                                   # fills both pages; captures the graph
        lg = engine.step([a, b], [[toks[0][k]], [toks[1][k]]]).cpu()
        assert float((lg[0] - want[0][k]).abs().max()) <= TOL["bfloat16"]
    assert engine.prepare_decode([a, b]) is None                          # position 64 needs a third page
    held = [grp.ledger.held_count for grp in engine.cache.groups]
    with pytest.raises(StepError, match="exceeds the cache"):
        engine.step([a, b], [[toks[0][64]], [toks[1][64]]])
    assert [grp.ledger.held_count for grp in engine.cache.groups] == held and engine.length(a) == 64
    engine.close_sequence(b)
    lg = engine.step([a], [[toks[0][64]]]).cpu()
    assert float((lg[0] - want[0][64]).abs().max()) <= TOL["bfloat16"]


# ---- the whole decode step as one persistent kernel (an option: Ops.use_fused_decode) -----------------------------
FUSED_CONFIGS = {
    # widths that are multiples of 64 (the kernel's blocks of K), otherwise odd: 6 heads on 2 kv heads of 32, a window
    # of 70 from layer 1 on (a ring of 128 positions that wraps), untied head
    "F": dict(TINY["A"], hidden_size=192, intermediate_size=320, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=2, head_dim=32, vocab_size=331, max_position_embeddings=512, rms_norm_eps=1e-5,
              rope_theta=30000.0, tie_word_embeddings=False, use_sliding_window=True, sliding_window=70, max_window_layers=1),
    # head size 128, one kv head
    "G": dict(TINY["A"], hidden_size=256, intermediate_size=192, num_hidden_layers=2, num_attention_heads=2,
              num_key_value_heads=1, head_dim=128, vocab_size=515, max_position_embeddings=512, rms_norm_eps=2e-6,
              rope_theta=250000.0, tie_word_embeddings=True),
}


@pytest.mark.parametrize("name", ["F", "G", "real"])
def test_the_fused_decode_step(tmp_path, real_size_dir, name):
    """One persistent kernel for the whole decode step of up to 16 sequences: the same logits as the plain model,
    through captured graphs, with sequences of unequal lengths that end at different times."""
    from smolmoe_c99_b200.config import config_from_json
    from smolmoe_c99_b200.engine.engine import Engine
    from smolmoe_c99_b200.weights import write_random_model
    if name == "real":
        folder, vocab = real_size_dir, REAL_0_5B_2_LAYERS["vocab_size"]
    else:
        folder, vocab = write_random_model(config_from_json(FUSED_CONFIGS[name]), str(tmp_path / name), 21), FUSED_CONFIGS[name]["vocab_size"]
    engine = Engine(folder, "bfloat16", max_tokens=16 * 256, max_slots=16, kernels="fast")
    ops = engine.runtime.ops
    before = ops.use_fused_decode
    ops.use_fused_decode = True
    try:
        assert engine.model._fused_plan(engine.cache) is not None, "the model is the fused step's case"
        for n_seq in ((1, 5, 16) if name != "real" else (3,)):
            lengths = [20 + (41 * i) % 150 for i in range(n_seq)]
            requests = {f"r{i}": random_tokens(n, vocab, 800 + i) for i, n in enumerate(lengths)}
            prompt_lens = {r: len(t) - 4 - (i % 9) for i, (r, t) in enumerate(requests.items())}
            want = _plain(folder, requests, "bfloat16")
            launches = int(ops.lib.sm_launch_count())
            got = replay.batched(engine, [requests], prompt_lens)
            _check(got, want, "bfloat16", f"fused decode, {n_seq} sequences", REL_WIDE if name == "real" else None)
        engine.check_status()
    finally:
        ops.use_fused_decode = before
    # a model the fused step does not describe (a width that is no multiple of 64) goes kernel by kernel
    other = Engine(write_random_model(config_from_json(TINY["C"]), str(tmp_path / "c"), 2), "bfloat16", max_tokens=1024)
    assert other.model._fused_plan(other.cache) is None
