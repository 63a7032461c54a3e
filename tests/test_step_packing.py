"""How a step's sequences are packed for the kernels (host logic only): tokens one after another with each
token's position, slot, sequence end and sequence start; the prefill attention's query tiles; refusals."""
import pytest
import torch

from smolmoe_c99_b200.engine.batch import QUERY_TILE, pack_step

CPU = torch.device("cpu")


def _by_hand(slots, starts, token_lists):
    tokens, positions, token_slot, token_end, seq_start, cu = [], [], [], [], [], [0]
    for slot, start, toks in zip(slots, starts, token_lists):
        first = len(tokens)
        for i, t in enumerate(toks):
            tokens.append(t)
            positions.append(start + i)
            token_slot.append(slot)
            token_end.append(start + len(toks))
            seq_start.append(first)
        cu.append(len(tokens))
    return tokens, positions, token_slot, token_end, seq_start, cu


@pytest.mark.parametrize("lens", [[5], [3, 1, 70], [64, 65, 1, 2], [2, 9, 130, 1, 64, 7], [1] * 9])
def test_prompts_of_unequal_lengths(lens):
    """Up to four sequences are filled slice by slice, more with index arithmetic: both give what a loop gives."""
    slots = [7 - i if i < 7 else i for i in range(len(lens))]
    token_lists = [[(11 * i + j) % 97 for j in range(n)] for i, n in enumerate(lens)]
    step = pack_step(slots, [0] * len(lens), token_lists, CPU)
    tokens, positions, token_slot, token_end, seq_start, cu = _by_hand(slots, [0] * len(lens), token_lists)
    assert step.mode == "prefill" and step.n_seqs == len(lens) and step.n_tokens == sum(lens)
    assert step.tokens.tolist() == tokens and step.positions.tolist() == positions
    assert step.token_slot.tolist() == token_slot and step.token_end.tolist() == token_end
    assert step.token_seq_start.tolist() == seq_start and step.cu_seqlens.tolist() == cu
    assert step.slot_ids.tolist() == slots and step.seq_ends.tolist() == lens
    assert step.max_seq_len == max(lens)
    want_tiles = [[cu[i], n, q0] for i, n in enumerate(lens) for q0 in range(0, n, QUERY_TILE)]
    assert step.prefill_tiles.tolist() == want_tiles
    for t in (step.tokens, step.positions, step.token_slot, step.token_end, step.token_seq_start, step.cu_seqlens,
              step.slot_ids, step.seq_ends, step.prefill_tiles):
        assert t.dtype == torch.int32 and t.is_contiguous()


@pytest.mark.parametrize("n", [1, 3, 8])
def test_one_token_each(n):
    slots = list(range(n, 0, -1))
    starts = [10 * (i + 1) for i in range(n)]
    step = pack_step(slots, starts, [[i + 1] for i in range(n)], CPU)
    assert step.mode == "decode" and step.prefill_tiles is None
    assert step.tokens.tolist() == [i + 1 for i in range(n)]
    assert step.positions.tolist() == starts
    assert step.token_end.tolist() == [s + 1 for s in starts] == step.seq_ends.tolist()
    assert step.token_slot.tolist() == slots == step.slot_ids.tolist()
    assert step.token_seq_start.tolist() == list(range(n)) and step.cu_seqlens.tolist() == list(range(n + 1))
    assert step.max_seq_len == max(starts) + 1


@pytest.mark.parametrize("starts,lens", [([5], [2]), ([0, 5], [2, 1]), ([64, 0, 3, 200], [65, 7, 1, 130]),
                                         ([9, 8, 7, 6, 5, 0], [1, 1, 1, 1, 1, 70])])
def test_sequences_that_go_on_by_any_number_of_tokens(starts, lens):
    """A prompt in portions, a later message onto a live sequence, new sequences beside ones that decode: the
    same packing, with tiles that carry each sequence's first position and slot."""
    slots = [3 * i + 1 for i in range(len(lens))]
    token_lists = [[(7 * i + j) % 89 for j in range(n)] for i, n in enumerate(lens)]
    step = pack_step(slots, starts, token_lists, CPU)
    tokens, positions, token_slot, token_end, seq_start, cu = _by_hand(slots, starts, token_lists)
    assert step.mode == "extend" and step.prefill_tiles is None and step.seq_starts == starts
    assert step.tokens.tolist() == tokens and step.positions.tolist() == positions
    assert step.token_slot.tolist() == token_slot and step.token_end.tolist() == token_end
    assert step.token_seq_start.tolist() == seq_start and step.cu_seqlens.tolist() == cu
    assert step.slot_ids.tolist() == slots and step.seq_ends.tolist() == [s + n for s, n in zip(starts, lens)]
    assert step.max_seq_len == max(s + n for s, n in zip(starts, lens))
    want_tiles = [[cu[i], n, q0, starts[i], slots[i]] for i, n in enumerate(lens) for q0 in range(0, n, QUERY_TILE)]
    assert step.extend_tiles.tolist() == want_tiles and step.extend_tiles.dtype == torch.int32


def test_what_is_refused():
    with pytest.raises(ValueError, match="at least one sequence"):
        pack_step([], [], [], CPU)
    with pytest.raises(ValueError, match="at least one token"):
        pack_step([0, 1], [0, 0], [[1], []], CPU)
    with pytest.raises(ValueError, match="not negative"):
        pack_step([0], [-1], [[1, 2]], CPU)
