"""The GPU sampler against the plain restatement of the reference's rules (src/sampler.c)."""
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from smolmoe_c99_b200.kernels import get_ops
    return get_ops()


def _rows(n, vocab, seed, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, vocab, generator=g) * scale


def test_argmax_ties_and_bans(ops):
    logits = _rows(6, 1000, 1)
    logits[0, 10] = logits[0, 700] = 50.0            # a tie: the lower id wins
    logits[1, :] = 0.0                               # everything ties
    logits[2, 999] = 60.0
    banned = torch.zeros(1000, dtype=torch.uint8); banned[[10, 0, 999]] = 1
    got = ops.argmax(logits.cuda()).tolist()
    assert got == [plain_model.argmax(r.tolist()) for r in logits] and got[0] == 10 and got[1] == 0 and got[2] == 999
    got_b = ops.argmax(logits.cuda(), banned.cuda()).tolist()
    assert got_b == [plain_model.argmax(r.tolist(), banned.tolist()) for r in logits] and got_b[0] == 700 and got_b[1] == 1
    assert ops.argmax(logits.cuda(), torch.ones(1000, dtype=torch.uint8).cuda()).tolist() == [-1] * 6
    big = _rows(3, 151936, 2)                        # a vocabulary that is no power of two, many chunks
    assert ops.argmax(big.cuda()).tolist() == big.argmax(dim=1).tolist()
    assert ops.argmax(logits.cuda()).tolist() == got   # the scratch words are back to idle: a second call agrees


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 40, 0.95), (1.0, 0, 1.0), (0.3, 5, 0.5), (2.0, 0, 0.9),
                                                      (0.9, 1, 1.0), (1.0, 300, 1e-6), (1.3, 1000, 0.999)])
def test_sample_matches_the_plain_sampler(ops, temperature, top_k, top_p):
    vocab, rows = 300, 24
    logits = _rows(rows, vocab, 7)
    logits[3, 5] = logits[3, 6] = logits[3, 250] = float(logits[3].max()) + 1.0     # ties at the top
    logits[4] = torch.round(logits[4])                                               # many ties everywhere
    seeds = [1 + 7919 * i for i in range(rows)]
    states = torch.tensor(seeds, dtype=torch.int64).to(torch.int32).cuda()
    dev = logits.cuda()
    host_states = list(seeds)
    for draw in range(6):
        got = ops.sample(dev, states, temperature, top_k, top_p).tolist()
        want = []
        for r in range(rows):
            tok, host_states[r] = plain_model.sample(logits[r].tolist(), temperature, top_k, top_p, host_states[r])
            want.append(tok)
        assert got == want, f"draw {draw}"
        assert (states.cpu().to(torch.int64) & 0xFFFFFFFF).tolist() == host_states


def test_sample_with_bans_and_batch_independence(ops):
    vocab = 500
    logits = _rows(5, vocab, 9)
    banned = torch.zeros(vocab, dtype=torch.uint8); banned[logits.argmax(dim=1)] = 1
    states = torch.tensor([11, 22, 33, 44, 55], dtype=torch.int32).cuda()
    got = ops.sample(logits.cuda(), states.clone(), 0.7, 10, 0.9, banned.cuda()).tolist()
    want = [plain_model.sample(logits[r].tolist(), 0.7, 10, 0.9, s, banned.tolist())[0] for r, s in enumerate([11, 22, 33, 44, 55])]
    assert got == want and all(not banned[t] for t in got)
    # a row alone draws what it draws in the batch
    alone = ops.sample(logits[2:3].cuda(), torch.tensor([33], dtype=torch.int32).cuda(), 0.7, 10, 0.9, banned.cuda()).tolist()
    assert alone == [got[2]]


def test_sampler_options(ops):
    from smolmoe_c99_b200.sampling import Sampler, SamplingOptions, sequence_seed
    with pytest.raises(ValueError, match="temperature"):
        SamplingOptions(temperature=1e-7).validate()
    with pytest.raises(ValueError, match="top-p"):
        SamplingOptions(top_p=0.0).validate()
    with pytest.raises(ValueError, match="seed"):
        SamplingOptions(seed=0).validate()
    assert sequence_seed(1, 0) == 1 and sequence_seed(0xFFFFFFFF, 1) == 1
    s = Sampler(ops, 100, SamplingOptions(), torch.device("cuda"), banned_token_ids=[3])
    logits = torch.zeros(2, 100); logits[:, 3] = 9.0; logits[:, 8] = 5.0
    assert s.choose(logits.cuda(), s.new_states([0, 1])).tolist() == [8, 8]
