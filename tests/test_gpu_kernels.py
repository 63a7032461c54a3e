"""Each kernel alone against a plain float32 computation in PyTorch, at sizes other than
the engine's tiny configurations (widths and vocabularies that are no power of two, head
sizes in steps of 16, ragged tiles)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from smolmoe_c99_b200.kernels import get_ops
    return get_ops()


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("T,N,K", [(1, 896, 896), (8, 1152, 896), (64, 896, 4864), (3, 100, 72), (130, 300, 200),
                                   (2048, 896, 896), (500, 1000, 136), (17, 128, 64), (256, 256, 8), (33, 150, 1024),
                                   (64, 3584, 18944), (100, 896, 4864)])
@pytest.mark.parametrize("mode", ["store_f32", "store_bf16", "accumulate"])
@pytest.mark.parametrize("pairs", [True, False])
def test_gemm_tc(ops, T, N, K, mode, pairs):
    """``pairs``: above 64 tokens the two-CTA kernel (the default) or the one-CTA kernel."""
    if not pairs and T <= 160:
        pytest.skip("up to 160 tokens there is one kernel")
    ops.gemm_pair_enable(pairs)
    try:
        _gemm_tc_case(ops, T, N, K, mode)
    finally:
        ops.gemm_pair_enable(True)


def _gemm_tc_case(ops, T, N, K, mode):
    x, w = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05)
    bias = _rand((N,), torch.bfloat16, 3)
    want = x.float() @ w.float().T
    if mode == "accumulate":
        out = _rand((T, N), torch.float32, 4)
        want = want + out
        ops.gemm_tc(x, w, None, out, mode=1)
    else:
        out = torch.empty((T, N), dtype=torch.float32 if mode == "store_f32" else torch.bfloat16, device="cuda")
        want = want + bias.float()
        ops.gemm_tc(x, w, bias, out, mode=0)
    ops.check_error_flag()
    tol = 1e-3 * math.sqrt(K) * 0.05 + (0.0 if out.dtype == torch.float32 else 8e-3 * float(want.abs().max()))
    assert float((out.float() - want).abs().max()) <= tol


@pytest.mark.parametrize("T,H,K", [(1, 4864, 896), (8, 4864, 896), (64, 160, 96), (300, 520, 264), (2048, 1024, 128),
                                   (40, 202, 2048), (64, 18944, 3584), (70, 160, 1024), (112, 4864, 896), (129, 202, 264),
                                   (160, 520, 96)])
@pytest.mark.parametrize("pairs", [True, False])
def test_gemm_tc_gated(ops, T, H, K, pairs):
    """(a gated product goes to the two-CTA kernel from 112 tokens)"""
    if not pairs and T < 112:
        pytest.skip("up to 111 tokens there is one kernel")
    ops.gemm_pair_enable(pairs)
    try:
        _gemm_tc_gated_case(ops, T, H, K)
    finally:
        ops.gemm_pair_enable(True)


def _gemm_tc_gated_case(ops, T, H, K):
    x, w = _rand((T, K), torch.bfloat16, 5), _rand((2 * H, K), torch.bfloat16, 6, 0.05)
    g, u = x.float() @ w[:H].float().T, x.float() @ w[H:].float().T
    want = u * (g / (1 + torch.exp(-g)))
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x, w, None, out, mode=2, up_offset=H)
    ops.check_error_flag()
    assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("T,N,K", [(512, 896, 896), (2048, 896, 4864), (700, 200, 72), (1100, 1152, 896), (513, 136, 264),
                                   (4096, 2048, 128), (8192, 512, 64), (161, 896, 4864), (170, 136, 72), (300, 1152, 896),
                                   (120, 1152, 896), (112, 136, 72), (512, 896, 4864), (1000, 896, 4864), (256, 904, 2048),
                                   (300, 136, 1024), (700, 520, 4104)])
@pytest.mark.parametrize("mode", ["store_f32", "store_bf16", "accumulate", "gated"])
def test_gemm_pair(ops, T, N, K, mode):
    """Products of more than 160 tokens go to the kernel in which two CTAs share a tile of 256 tokens: against a float
    product, and against the one-CTA kernel on the same data. ("accumulate" with few tiles and a long K: two or four pairs
    of a cluster share a tile's K.)"""
    x = _rand((T, K), torch.bfloat16, 11)
    w = _rand((2 * N if mode == "gated" else N, K), torch.bfloat16, 12, 0.05)
    bias = _rand((N,), torch.bfloat16, 13)
    start = _rand((T, N), torch.float32, 14)

    def run():
        if mode == "gated":
            out = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
            return ops.gemm_tc(x, w, None, out, mode=2, up_offset=N)
        if mode == "accumulate":
            return ops.gemm_tc(x, w, None, start.clone(), mode=1)
        out = torch.empty((T, N), dtype=torch.float32 if mode == "store_f32" else torch.bfloat16, device="cuda")
        return ops.gemm_tc(x, w, bias, out, mode=0)

    if mode == "gated":
        g, u = x.float() @ w[:N].float().T, x.float() @ w[N:].float().T
        want = u * (g / (1 + torch.exp(-g)))
    else:
        want = x.float() @ w.float().T + (start if mode == "accumulate" else bias.float())
    got = run()
    ops.check_error_flag()
    ops.gemm_pair_enable(False)
    try:
        single = run()
        ops.check_error_flag()
    finally:
        ops.gemm_pair_enable(True)
    rounding = 0.0 if got.dtype == torch.float32 else 8e-3 * float(want.abs().max())
    tol = 1e-3 * math.sqrt(K) * 0.05 + rounding + (1e-3 if mode == "gated" else 0.0)
    assert float((got.float() - want).abs().max()) <= tol
    assert float((got.float() - single.float()).abs().max()) <= tol


def test_gemm_tc_refuses_unaligned_k(ops):
    from smolmoe_c99_b200.kernels import KernelError
    x, w = _rand((4, 100), torch.bfloat16, 1), _rand((16, 100), torch.bfloat16, 2)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_tc(x, w, None, torch.empty((4, 16), dtype=torch.float32, device="cuda"))
    # the dispatcher takes the CUDA-core kernel for it instead
    got = ops.linear(x, w, None, out_dtype=torch.float32)
    assert float((got - x.float() @ w.float().T).abs().max()) < 1e-3


@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("T,N,K", [(1, 70, 50), (65, 129, 33), (200, 64, 1000)])
def test_gemm_simt(ops, xd, wd, od, T, N, K):
    x, w, b = _rand((T, K), xd, 1), _rand((N, K), wd, 2, 0.05), _rand((N,), wd, 3)
    want = x.float() @ w.float().T + b.float()
    out = ops.gemm_simt(x, w, b, torch.empty((T, N), dtype=od, device="cuda"))
    tol = 2e-5 if od == torch.float32 else 8e-3 * float(want.abs().max())
    assert float((out.float() - want).abs().max()) <= tol
    # each output is one chain over k: more rows in the batch change no bit
    alone = ops.gemm_simt(x[:1].contiguous(), w, b, torch.empty((1, N), dtype=od, device="cuda"))
    assert torch.equal(alone[0], out[0])


# ---- attention ---------------------------------------------------------------------------
@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (14, 2, 64), (8, 2, 128), (3, 1, 48)])
@pytest.mark.parametrize("first", [3, 30, 2040])
def test_decode_attention_with_several_rows_of_a_sequence(ops, heads, kv_heads, hd, first):
    """A short later message: every new token of a sequence is a row of the decode kernel (``late``), each attending
    over the cache up to its own position, beside rows of another sequence; against the plain kernel."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    n_new, other = 9, 5
    longest = first + n_new
    pages_per_slot = -(-max(longest, 700) // PAGE_SIZE)
    g = torch.Generator().manual_seed(first)
    k_pool = _rand((2 * pages_per_slot, kv_heads, PAGE_SIZE, hd), torch.bfloat16, 31, 0.5)
    v_pool = _rand((2 * pages_per_slot, kv_heads, PAGE_SIZE, hd), torch.bfloat16, 32, 0.5)
    table = torch.randperm(2 * pages_per_slot, generator=g).to(torch.int32).view(2, pages_per_slot).cuda()
    positions = torch.tensor(list(range(first, first + n_new)) + list(range(600, 600 + other)), dtype=torch.int32).cuda()
    slots = torch.tensor([1] * n_new + [0] * other, dtype=torch.int32).cuda()
    q = _rand((n_new + other, heads, hd), torch.bfloat16, 33)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention_decode(q, positions, slots, scale, None, k_pool, v_pool, table, 0, kv_heads, max(longest, 605), late=True)
    ops.check_error_flag()
    want = ops.attention_plain(q, positions, scale, None, k_pool=k_pool, v_pool=v_pool, page_table=table, ring=0,
                               token_slot=slots, kv_heads=kv_heads)
    assert float((got.float() - want.float()).abs().max()) <= 1e-2



def _plain_attention(q, k, v, lens, window, scale):
    """q [T, H, hd], k/v [T, KH, hd] packed sequences; float64 reference on the CPU."""
    q, k, v = q.double().cpu(), k.double().cpu(), v.double().cpu()
    out = torch.zeros_like(q)
    H, KH = q.shape[1], k.shape[1]
    at = 0
    for n in lens:
        for pos in range(n):
            start = pos - window + 1 if (window and pos >= window) else 0
            for h in range(H):
                kh = h // (H // KH)
                s = (k[at + start:at + pos + 1, kh] @ q[at + pos, h]) * scale
                p = torch.softmax(s, dim=0)
                out[at + pos, h] = p @ v[at + start:at + pos + 1, kh]
        at += n
    return out.float()


def _packed_step(lens):
    from smolmoe_c99_b200.engine.batch import pack_step
    return pack_step(list(range(len(lens))), [0] * len(lens), [[0] * n for n in lens], torch.device("cuda"))


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (14, 2, 64), (6, 3, 80), (8, 2, 128), (2, 1, 40)])
@pytest.mark.parametrize("window", [None, 37, 100])
def test_attention_of_sequences_that_go_on_from_the_cache(ops, heads, kv_heads, hd, window):
    """Sequences at different points: one at its start, one that goes on by a single token, others by 7, 64 and 130
    tokens from positions that are no multiple of anything. Earlier keys and values lie in a paged cache (a ring for a
    window; every position written in order, so stale rows are real rows), the step's own come packed and are NOT in
    the cache yet. The tensor-core kernel and the plain kernel (bfloat16 and float) against the float64 formula; then
    kv_store puts the step's rows where they belong."""
    from types import SimpleNamespace
    from smolmoe_c99_b200.engine.batch import pack_step
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    starts, news = [0, 150, 33, 200, 70], [50, 1, 7, 64, 130]
    B, total = len(starts), [s + n for s, n in zip(starts, news)]
    ring = ((window + PAGE_SIZE - 1) // PAGE_SIZE) * PAGE_SIZE if window else 0
    pages_per_seq = (ring or 384) // PAGE_SIZE
    g = torch.Generator().manual_seed(31)
    table = torch.randperm(B * pages_per_seq, generator=g).to(torch.int32).view(B, pages_per_seq)
    k_pool = torch.zeros((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    ks = [torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16) for n in total]
    vs = [torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16) for n in total]
    qs = [torch.randn((n, heads, hd), generator=g).to(torch.bfloat16) for n in total]
    for b in range(B):
        for p in range(starts[b]):                    # the cache holds what earlier steps left, and nothing of this step
            idx = p % ring if ring else p
            page = int(table[b, idx // PAGE_SIZE])
            k_pool[page, :, idx % PAGE_SIZE] = ks[b][p]
            v_pool[page, :, idx % PAGE_SIZE] = vs[b][p]
    scale = 1.0 / math.sqrt(hd)
    want = torch.cat([_plain_attention(qs[b], ks[b], vs[b], [total[b]], window, scale)[starts[b]:] for b in range(B)])
    step = pack_step(list(range(B)), starts, [[0] * n for n in news], torch.device("cuda"))
    assert step.mode == "extend"
    q = torch.cat([qs[b][starts[b]:] for b in range(B)]).cuda()
    k = torch.cat([ks[b][starts[b]:] for b in range(B)]).cuda()
    v = torch.cat([vs[b][starts[b]:] for b in range(B)]).cuda()
    cache = SimpleNamespace(k_pool=k_pool.cuda(), v_pool=v_pool.cuda(), page_table=table.cuda(), ring=ring)
    if hd % 16 == 0:
        got = ops.attention_extend(q, k, v, step, scale, window, cache).float().cpu()
        assert float((got - want).abs().max()) <= 2e-2, "tensor-core kernel"
    plain = ops.attention_plain(q, step.positions, scale, window, k_packed=k, v_packed=v, token_seq_start=step.token_seq_start,
                                k_pool=cache.k_pool, v_pool=cache.v_pool, page_table=cache.page_table, ring=ring,
                                token_slot=step.token_slot).float().cpu()
    assert float((plain - want).abs().max()) <= 1e-2, "plain kernel, bfloat16"
    cache32 = SimpleNamespace(k_pool=k_pool.float().cuda(), v_pool=v_pool.float().cuda(), page_table=table.cuda(), ring=ring)
    plain32 = ops.attention_plain(q.float(), step.positions, scale, window, k_packed=k.float(), v_packed=v.float(),
                                  token_seq_start=step.token_seq_start, k_pool=cache32.k_pool, v_pool=cache32.v_pool,
                                  page_table=cache32.page_table, ring=ring, token_slot=step.token_slot).cpu()
    assert float((plain32 - want).abs().max()) <= 2e-5, "plain kernel, float"
    # the step's rows into the cache: every position of a sequence then lies where a later step looks for it
    for pools, kk, vv in ((cache, k, v), (cache32, k.float(), v.float())):
        ops.kv_store(kk, vv, step, pools)
        at = 0
        for b in range(B):
            first_kept = max(0, total[b] - ring) if ring else 0
            for p in list(range(first_kept, min(total[b], first_kept + 3))) + [total[b] - 1]:
                idx = p % ring if ring else p
                page = int(table[b, idx // PAGE_SIZE])
                assert torch.equal(pools.k_pool[page, :, idx % PAGE_SIZE].float().cpu(), ks[b][p].float()), (b, p)
                assert torch.equal(pools.v_pool[page, :, idx % PAGE_SIZE].float().cpu(), vs[b][p].float()), (b, p)
            at += news[b]


@pytest.mark.parametrize("heads,kv_heads,hd", [(14, 2, 64), (4, 4, 64), (8, 2, 128)])
@pytest.mark.parametrize("starts,news", [([700, 0, 33, 1000], [600, 130, 64, 530]), ([2000], [1000]), ([1, 127, 128], [300, 129, 257])])
@pytest.mark.parametrize("variant", [0, 1])
def test_attention_of_many_tokens_onto_the_cache(ops, heads, kv_heads, hd, starts, news, variant):
    """Prompt portions: sequences go on by hundreds of tokens from positions that are no multiple of a tile, and the
    cache holds the step's own keys and values already. The tcgen05 kernel reads every key from the paged pools (pages
    in a random order; rows past a sequence's end hold other numbers and must not count) and is compared with the
    plain kernel in float. One key far back stands out for one query of each sequence."""
    from types import SimpleNamespace
    from smolmoe_c99_b200.engine.batch import pack_step
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    B, total = len(starts), [s + n for s, n in zip(starts, news)]
    pages_per_seq = -(-max(total) // PAGE_SIZE) + 1
    g = torch.Generator().manual_seed(sum(news))
    table = torch.randperm(B * pages_per_seq, generator=g).to(torch.int32).view(B, pages_per_seq)
    k_pool = torch.randn((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), generator=g).to(torch.bfloat16)
    v_pool = torch.randn((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), generator=g).to(torch.bfloat16)
    qs = [torch.randn((n, heads, hd), generator=g).to(torch.bfloat16) for n in news]
    for b in range(B):
        # the last query of the sequence looks hard at one key near the sequence's start
        far = min(5, total[b] - 1)
        page = int(table[b, far // PAGE_SIZE])
        qs[b][-1] = k_pool[page, :, far % PAGE_SIZE].repeat_interleave(heads // kv_heads, dim=0) * 3.0
        # ... and the query before it at a key near the sequence's end: the scores of all earlier tiles are small beside
        # it, so the running reference moves late and what has been accumulated by then is rescaled
        if news[b] >= 2:
            near = total[b] - 3
            page = int(table[b, near // PAGE_SIZE])
            qs[b][-2] = k_pool[page, :, near % PAGE_SIZE].repeat_interleave(heads // kv_heads, dim=0) * 3.0
    step = pack_step(list(range(B)), starts, [[0] * n for n in news], torch.device("cuda"))
    assert step.mode == "extend"
    q = torch.cat(qs).cuda()
    assert q.shape[0] > ops.extend_rows_as_decode_tc
    packed = torch.empty((q.shape[0], kv_heads, hd), dtype=torch.bfloat16, device="cuda")     # not read
    cache = SimpleNamespace(k_pool=k_pool.cuda(), v_pool=v_pool.cuda(), page_table=table.cuda(), ring=0)
    scale = 1.0 / math.sqrt(hd)
    launches = int(ops.lib.sm_launch_count())
    ops.extend_tc_variant = variant          # one CTA an SM, or two (head size 64; 128 has the one form)
    try:
        got = ops.attention_extend(q, packed, packed, step, scale, None, cache, cache_written=True).float()
    finally:
        ops.extend_tc_variant = -1
    ops.check_error_flag()
    assert int(ops.lib.sm_launch_count()) == launches + 1
    want = ops.attention_plain(q.float(), step.positions, scale, None, k_pool=cache.k_pool.float(), v_pool=cache.v_pool.float(),
                               page_table=cache.page_table, ring=0, token_slot=step.token_slot, kv_heads=kv_heads)
    assert float((got - want).abs().max()) <= 2e-2
    at = 0
    for b in range(B):
        at += news[b]
        far = min(5, total[b] - 1)
        page = int(table[b, far // PAGE_SIZE])
        for h in (0, heads - 1):
            v_far = cache.v_pool[page, h // (heads // kv_heads), far % PAGE_SIZE].float()
            assert float((got[at - 1, h] - v_far).abs().max()) <= 5e-2, (b, h)
        if news[b] >= 2:
            near = total[b] - 3
            page = int(table[b, near // PAGE_SIZE])
            for h in (0, heads - 1):
                v_near = cache.v_pool[page, h // (heads // kv_heads), near % PAGE_SIZE].float()
                assert float((got[at - 2, h] - v_near).abs().max()) <= 5e-2, (b, h, "late key")


@pytest.mark.parametrize("T", [1, 5, 16])
@pytest.mark.parametrize("N,K", [(70, 50), (129, 1000), (16, 4864)])
def test_gemm_simt_for_few_tokens_gives_the_tile_kernels_bits(ops, T, N, K):
    """Up to 16 tokens take a kernel of their own in the 32-bit path; its sums are the tile kernel's, bit for bit (the
    same rows inside a batch of 64 go through the tile kernel)."""
    x, w, b = _rand((64, K), torch.float32, 1), _rand((N, K), torch.float32, 2, 0.1), _rand((N,), torch.float32, 3)
    big = ops.gemm_simt(x, w, b, torch.empty((64, N), dtype=torch.float32, device="cuda"))
    small = ops.gemm_simt(x[:T].contiguous(), w, b, torch.empty((T, N), dtype=torch.float32, device="cuda"))
    assert torch.equal(small, big[:T])
    want = x[:T].double() @ w.double().T + b.double()
    assert float((small.double() - want).abs().max()) <= 1e-5 * math.sqrt(K)
    acc = _rand((T, N), torch.float32, 4)
    acc_big = torch.cat([acc, torch.zeros((64 - T, N), device="cuda")]).contiguous()
    ops.gemm_simt(x[:T].contiguous(), w, None, acc, accumulate=True)
    ops.gemm_simt(x, w, None, acc_big, accumulate=True)
    assert torch.equal(acc, acc_big[:T])


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (14, 2, 64), (6, 3, 80), (8, 2, 128)])
@pytest.mark.parametrize("window", [None, 37])
def test_prefill_attention(ops, heads, kv_heads, hd, window):
    lens = [1, 63, 64, 65, 130]
    T = sum(lens)
    q, k, v = (_rand((T, n, hd), torch.bfloat16, s) for n, s in ((heads, 1), (kv_heads, 2), (kv_heads, 3)))
    scale = 1.0 / math.sqrt(hd)
    step = _packed_step(lens)
    want = _plain_attention(q, k, v, lens, window, scale)
    got = ops.attention_prefill_mma(q, k, v, step.prefill_tiles, scale, window).float().cpu()
    assert float((got - want).abs().max()) <= 2e-2
    plain = ops.attention_plain(q, step.positions, scale, window, k_packed=k, v_packed=v,
                                token_seq_start=step.token_seq_start).float().cpu()
    assert float((plain - want).abs().max()) <= 1e-2
    plain32 = ops.attention_plain(q.float(), step.positions, scale, window, k_packed=k.float(), v_packed=v.float(),
                                  token_seq_start=step.token_seq_start).cpu()
    assert float((plain32 - want).abs().max()) <= 2e-5


@pytest.mark.parametrize("heads,kv_heads,hd,variant", [(14, 2, 64, 0), (14, 2, 64, 1), (3, 1, 64, 0), (3, 1, 64, 1),
                                                       (4, 4, 128, -1), (6, 2, 128, -1)])
@pytest.mark.parametrize("window", [None, 37, 200])
def test_prefill_attention_tcgen05(ops, heads, kv_heads, hd, variant, window):
    """Sequences shorter than, equal to and longer than the tiles of 128; a window inside and across tiles."""
    lens = [1, 127, 128, 129, 300, 64]
    T = sum(lens)
    q, k, v = (_rand((T, n, hd), torch.bfloat16, s) for n, s in ((heads, 1), (kv_heads, 2), (kv_heads, 3)))
    scale = 1.0 / math.sqrt(hd)
    step = _packed_step(lens)
    want = _plain_attention(q, k, v, lens, window, scale)
    got = ops.attention_prefill_tcgen05(q, k, v, step.prefill_tiles, scale, window, variant=variant).float().cpu()
    ops.check_error_flag()
    assert float((got - want).abs().max()) <= 2e-2
    # it is the one the engine takes (whichever variant: they agree to rounding)
    assert float((ops.attention_prefill(q, k, v, step, scale, window).float().cpu() - got).abs().max()) <= 1e-2


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_prefill_attention_finds_a_far_key(ops, kernel):
    """One key far back among hundreds is made to dominate: its value must come through."""
    heads, kv_heads, hd, n = 2, 1, 64, 700
    run = ops.attention_prefill_mma if kernel == "mma" else ops.attention_prefill_tcgen05
    q, k, v = _rand((n, heads, hd), torch.bfloat16, 1, 0.1), _rand((n, kv_heads, hd), torch.bfloat16, 2, 0.1), \
        _rand((n, kv_heads, hd), torch.bfloat16, 3)
    far = 5
    k[far] = 0
    k[far, 0, 0] = 40.0
    q[n - 1, :, 0] = 40.0   # score 1600/8 = 200 for the far key, O(1) for the others
    # and one key in the query tile's last but one key tile dominates for another query: the running maximum moves
    # late, after tiles of small scores have been accumulated
    late = n - 140
    k[late] = 0
    k[late, 0, 1] = 40.0
    q[n - 2, :, 1] = 40.0
    step = _packed_step([n])
    got = run(q, k, v, step.prefill_tiles, 1.0 / math.sqrt(hd), None).float()
    assert float((got[n - 1, 0] - v[far, 0].float()).abs().max()) <= 2e-2
    assert float((got[n - 2, 0] - v[late, 0].float()).abs().max()) <= 2e-2
    # with a window that ends just after it, it is out of sight
    got_w = run(q, k, v, step.prefill_tiles, 1.0 / math.sqrt(hd), n - 1 - far).float()
    assert float((got_w[n - 1, 0] - v[far, 0].float()).abs().max()) > 0.1
    got_w1 = run(q, k, v, step.prefill_tiles, 1.0 / math.sqrt(hd), n - far).float()
    assert float((got_w1[n - 1, 0] - v[far, 0].float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (14, 2, 64), (9, 1, 128), (16, 1, 80),
                                               (4, 2, 256)])
@pytest.mark.parametrize("window", [None, 100])
def test_decode_attention_over_pages(ops, heads, kv_heads, hd, window):
    """Sequences of unequal lengths in scattered pages; the windowed case uses a ring."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    lens = [1, 64, 65, 129, 500]
    B = len(lens)
    ring = ((window + PAGE_SIZE - 1) // PAGE_SIZE) * PAGE_SIZE if window else 0
    pages_per_seq = (ring or max(lens) + PAGE_SIZE - 1) // PAGE_SIZE + 1
    n_pages = B * pages_per_seq + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(7)).tolist()
    table = torch.zeros((B + 2, pages_per_seq), dtype=torch.int32)
    slots = [4, 0, 2, 5, 1]
    for b, slot in enumerate(slots):
        table[slot] = torch.tensor(perm[b * pages_per_seq:(b + 1) * pages_per_seq], dtype=torch.int32)
    k_pool = torch.zeros((n_pages, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    ks, vs, qs = [], [], []
    for b, n in enumerate(lens):
        k, v = _rand((n, kv_heads, hd), torch.bfloat16, 10 + b).cpu(), _rand((n, kv_heads, hd), torch.bfloat16, 20 + b).cpu()
        ks.append(k); vs.append(v)
        for p in range(n):
            idx = p % ring if ring else p
            page = int(table[slots[b], idx // PAGE_SIZE])
            k_pool[page, :, idx % PAGE_SIZE] = k[p]
            v_pool[page, :, idx % PAGE_SIZE] = v[p]
        qs.append(_rand((1, heads, hd), torch.bfloat16, 30 + b))
    q = torch.cat(qs, dim=0)
    scale = 1.0 / math.sqrt(hd)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slot_ids = torch.tensor(slots, dtype=torch.int32).cuda()
    if hd > 128:
        from smolmoe_c99_b200.kernels import KernelError
        with pytest.raises(KernelError, match="outside this kernel"):   # refused, not wrong: the plain kernel takes it
            ops.attention_decode(q, positions, slot_ids, scale, window, k_pool.cuda(), v_pool.cuda(), table.cuda(), ring,
                                 kv_heads, max(lens))
        got = None
    else:
        got = ops.attention_decode(q, positions, slot_ids, scale, window, k_pool.cuda(), v_pool.cuda(), table.cuda(), ring,
                                   kv_heads, max(lens)).float().cpu()
    plain = ops.attention_plain(q, positions, scale, window, k_pool=k_pool.cuda(), v_pool=v_pool.cuda(),
                                page_table=table.cuda(), ring=ring, token_slot=slot_ids, kv_heads=kv_heads).float().cpu()
    for b, n in enumerate(lens):
        qq = torch.zeros((n, heads, hd), dtype=torch.bfloat16)
        qq[n - 1] = q[b].cpu()
        want = _plain_attention(qq, ks[b], vs[b], [n], window, scale)[n - 1]
        if got is not None:
            assert float((got[b] - want).abs().max()) <= 1e-2, f"cluster kernel, sequence {b}"
        assert float((plain[b] - want).abs().max()) <= 1e-2, f"plain kernel, sequence {b}"


@pytest.mark.parametrize("heads,kv_heads,hd", [(14, 2, 64), (8, 2, 128), (3, 1, 32)])
@pytest.mark.parametrize("lens,max_len", [([3000, 2500, 64, 1, 700], 4096), ([1500] * 3 + [40] * 37, 2048), ([4090], 4096)])
def test_decode_attention_long_contexts(ops, heads, kv_heads, hd, lens, max_len):
    """Shares of a cluster's CTAs that do not fit one buffer (chunks in flight), many sequences with one CTA each,
    and one sequence over the largest cluster: against the float64 formula for the newest position."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    B = len(lens)
    pages_per_seq = max_len // PAGE_SIZE
    g = torch.Generator().manual_seed(5)
    table = torch.randperm(B * pages_per_seq, generator=g).to(torch.int32).view(B, pages_per_seq)
    k_pool = torch.zeros((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    q = _rand((B, heads, hd), torch.bfloat16, 1).cpu()
    want = torch.zeros((B, heads, hd), dtype=torch.float64)
    scale = 1.0 / math.sqrt(hd)
    for b, n in enumerate(lens):
        k, v = _rand((n, kv_heads, hd), torch.bfloat16, 10 + b).cpu(), _rand((n, kv_heads, hd), torch.bfloat16, 50 + b).cpu()
        if n > 300:      # a far key that matters, so that a lost chunk shows
            k[7] = 0
            k[7, :, 0] = 30.0
            q[b, :, 0] = 2.0
        pages = table[b, :(n + PAGE_SIZE - 1) // PAGE_SIZE].long()
        padded = torch.zeros((len(pages) * PAGE_SIZE, kv_heads, hd), dtype=torch.bfloat16)
        padded[:n] = k
        k_pool[pages] = padded.view(len(pages), PAGE_SIZE, kv_heads, hd).permute(0, 2, 1, 3)
        padded = torch.zeros_like(padded)
        padded[:n] = v
        v_pool[pages] = padded.view(len(pages), PAGE_SIZE, kv_heads, hd).permute(0, 2, 1, 3)
        for h in range(heads):
            kh = h // (heads // kv_heads)
            p = torch.softmax((k[:, kh].double() @ q[b, h].double()) * scale, dim=0)
            want[b, h] = p @ v[:, kh].double()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slot_ids = torch.arange(B, dtype=torch.int32).cuda()
    got = ops.attention_decode(q.cuda(), positions, slot_ids, scale, None, k_pool.cuda(), v_pool.cuda(), table.cuda(), 0,
                               kv_heads, max_len).double().cpu()
    ops.check_error_flag()
    for b in range(B):
        assert float((got[b] - want[b]).abs().max()) <= 1e-2, f"sequence {b} of {lens[b]} positions"


@pytest.mark.parametrize("heads,kv_heads,hd", [(3, 1, 32), (10, 5, 48), (14, 2, 64), (6, 3, 96), (8, 2, 128), (12, 1, 64),
                                               (16, 1, 128), (9, 1, 80)])
@pytest.mark.parametrize("window", [None, 700])
def test_decode_attention_streamed_shares(ops, heads, kv_heads, hd, window):
    """More (sequence, kv head) pairs than the GPU holds clusters, each with hundreds of positions: every CTA streams
    its share tile by tile. Unequal lengths, scattered pages, a ring for the window (tiles then straddle pages and the
    ring's end), head sizes below their padded size; the newest position's row is the one read after the wait."""
    import ctypes
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    g = torch.Generator().manual_seed(11)
    B = 320 // kv_heads      # (the groups of more than 8 heads take two column tiles of the transposed product)
    lens = [int(x) for x in torch.randint(650, 1000, (B,), generator=g)]
    lens[0], lens[1], lens[2] = 1, 33, 999
    max_len = 1024
    ring = ((window + PAGE_SIZE - 1) // PAGE_SIZE) * PAGE_SIZE if window else 0
    pages_per_seq = (ring or max_len) // PAGE_SIZE
    plan = (ctypes.c_int * 4)()
    ops._check(ops.lib.sm_attention_decode_plan(B, heads, kv_heads, hd, int(window or 0), max_len, plan))
    assert plan[1] == 0, f"this case is meant for the streaming kernel, the plan is {list(plan)}"
    table = torch.randperm(B * pages_per_seq, generator=g).to(torch.int32).view(B, pages_per_seq)
    k_pool = torch.zeros((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    q = _rand((B, heads, hd), torch.bfloat16, 1).cpu()
    want = torch.zeros((B, heads, hd), dtype=torch.float64)
    scale = 1.0 / math.sqrt(hd)
    for b, n in enumerate(lens):
        k = torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16)
        v = torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16)
        first = max(0, n - window) if window else 0
        if n - first > 300:      # a far key that matters, so that a lost tile shows
            k[first + 5] = 0
            k[first + 5, :, 0] = 30.0
            q[b, :, 0] = 2.0
        where = torch.arange(first, n)
        idx = where % ring if ring else where
        pages = table[b, idx // PAGE_SIZE].long()
        k_pool[pages, :, idx % PAGE_SIZE] = k[first:]
        v_pool[pages, :, idx % PAGE_SIZE] = v[first:]
        for h in range(heads):
            kh = h // (heads // kv_heads)
            p = torch.softmax((k[first:, kh].double() @ q[b, h].double()) * scale, dim=0)
            want[b, h] = p @ v[first:, kh].double()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slot_ids = torch.arange(B, dtype=torch.int32).cuda()
    got = ops.attention_decode(q.cuda(), positions, slot_ids, scale, window, k_pool.cuda(), v_pool.cuda(), table.cuda(), ring,
                               kv_heads, max_len).double().cpu()
    ops.check_error_flag()
    worst = (got - want).abs().amax(dim=(1, 2))
    assert float(worst.max()) <= 1e-2, f"sequence {int(worst.argmax())} of {lens[int(worst.argmax())]} positions: {float(worst.max())}"


@pytest.mark.parametrize("heads,kv_heads,hd", [(14, 2, 64), (8, 2, 128), (3, 1, 32), (10, 5, 48)])
@pytest.mark.parametrize("window", [64, 100, 700, 704])
@pytest.mark.parametrize("many", [False, True])
def test_decode_attention_at_the_windows_lower_edge(ops, heads, kv_heads, hd, window, many):
    """The first key a query may see and the one just before it. Every position 0..n-1 is written into the ring in
    order, so the places outside the window hold real, older rows. A key that outweighs all others sits at the
    window's first position in the even sequences (its value must come through) and one position earlier in the
    odd ones (nothing of it may). Windows that fill their ring (64, 704) and windows that leave stale rows in it
    (100 in 128, 700 in 704); starts that are no multiple of 16; few sequences (one buffer per CTA) and many (shares
    streamed tile by tile)."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    g = torch.Generator().manual_seed(17)
    B = 320 // kv_heads if many else 4
    ring = ((window + PAGE_SIZE - 1) // PAGE_SIZE) * PAGE_SIZE
    lens = [int(x) for x in torch.randint(window + 1, window + 400, (B,), generator=g)]
    lens[0], lens[1] = window + 1, window + 2          # the window has just begun to slide
    pages_per_seq = ring // PAGE_SIZE
    table = torch.randperm(B * pages_per_seq, generator=g).to(torch.int32).view(B, pages_per_seq)
    k_pool = torch.zeros((B * pages_per_seq, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    q = torch.randn((B, heads, hd), generator=g).to(torch.bfloat16)
    q[:, :, 0] = 8.0
    want = torch.zeros((B, heads, hd), dtype=torch.float64)
    scale = 1.0 / math.sqrt(hd)
    for b, n in enumerate(lens):
        k = torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16)
        v = torch.randn((n, kv_heads, hd), generator=g).to(torch.bfloat16)
        start = n - window
        heavy = start if b % 2 == 0 else start - 1
        k[heavy] = 0
        k[heavy, :, 0] = 30.0                      # score 240 * scale against scores of a few units
        v[heavy] = 5.0
        for p in range(n):                         # in order: later positions take the places of earlier ones
            page = int(table[b, (p % ring) // PAGE_SIZE])
            k_pool[page, :, p % PAGE_SIZE] = k[p]
            v_pool[page, :, p % PAGE_SIZE] = v[p]
        for h in range(heads):
            kh = h // (heads // kv_heads)
            pr = torch.softmax((k[start:, kh].double() @ q[b, h].double()) * scale, dim=0)
            want[b, h] = pr @ v[start:, kh].double()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slot_ids = torch.arange(B, dtype=torch.int32).cuda()
    got = ops.attention_decode(q.cuda(), positions, slot_ids, scale, window, k_pool.cuda(), v_pool.cuda(), table.cuda(), ring,
                               kv_heads, max(lens)).double().cpu()
    ops.check_error_flag()
    plain = ops.attention_plain(q.cuda(), positions, scale, window, k_pool=k_pool.cuda(), v_pool=v_pool.cuda(),
                                page_table=table.cuda(), ring=ring, token_slot=slot_ids, kv_heads=kv_heads).double().cpu()
    for b in range(B):
        if b % 2 == 0:
            assert float((want[b] - 5.0).abs().max()) < 1e-3           # the case is what it is meant to be
        else:
            assert float(want[b].abs().max()) < 4.5
    for name, out in (("cluster kernel", got), ("plain kernel", plain)):
        worst = (out - want).abs().amax(dim=(1, 2))
        b = int(worst.argmax())
        assert float(worst.max()) <= 2e-2, f"{name}: sequence {b} ({lens[b]} positions, heavy key " \
            f"{'at' if b % 2 == 0 else 'before'} the window's start): off by {float(worst.max()):.3g}"


# ---- products over a handful of tokens -----------------------------------------------------
@pytest.mark.parametrize("T", [1, 3, 8, 9, 16, 32])
@pytest.mark.parametrize("N,K", [(896, 896), (100, 72), (151, 4864), (1000, 136)])
def test_gemm_skinny_store_and_accumulate(ops, T, N, K):
    x, w, b = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05), _rand((N,), torch.bfloat16, 3)
    want = x.float() @ w.float().T
    out = ops.gemm_skinny(x, w, b, torch.empty((T, N), dtype=torch.float32, device="cuda"))
    tol = 1e-3 * math.sqrt(K) * 0.05
    assert float((out - (want + b.float())).abs().max()) <= tol
    res = _rand((T, N), torch.float32, 4)
    want_acc = want + res
    ops.gemm_skinny(x, w, None, res, mode=1)
    assert float((res - want_acc).abs().max()) <= tol
    # the same rows alone give the same bits: a row's sum does not depend on the batch
    alone = ops.gemm_skinny(x[:1].contiguous(), w, b, torch.empty((1, N), dtype=torch.float32, device="cuda"))
    assert torch.equal(alone[0], out[0])


def test_which_kernel_takes_a_product_over_few_tokens(ops):
    """Up to 8 tokens: the weight-streaming kernel, unless plain rows would take three rounds or more. 9 to 16: only
    if its CTAs hold their share of K at once. More: the tcgen05 kernel. The output head (thousands of row tiles): the tcgen05 kernel."""
    def x(T, K):
        return torch.zeros((T, K), dtype=torch.bfloat16, device="cuda")

    def w(N, K):
        return torch.empty((N, K), dtype=torch.bfloat16, device="cuda")
    assert ops._skinny_ok(x(8, 896), w(896, 896)) and ops._skinny_ok(x(8, 8960), w(1536, 8960))   # one round, two rounds
    assert not ops._skinny_ok(x(8, 18944), w(3584, 18944))                # four rounds of plain rows: the tcgen05 kernel
    assert ops._skinny_ok(x(16, 896), w(1152, 896))                       # one round at 16 tokens
    assert not ops._skinny_ok(x(16, 896), w(2 * 4864, 896), gated=True)   # two rounds: 32 weight rows beside 16 tokens
    assert not ops._skinny_ok(x(16, 3584), w(4608, 3584))
    assert not ops._skinny_ok(x(17, 896), w(896, 896))
    assert not ops._skinny_ok(x(8, 896), w(151936, 896))
    assert not ops._skinny_ok(x(8, 896).float(), w(896, 896))              # the 32-bit path never takes it


@pytest.mark.parametrize("T,H,K", [(1, 4864, 896), (8, 160, 96), (13, 520, 264), (3, 48, 4104), (32, 40, 2056)])
def test_gemm_skinny_norm_prologue_and_gate(ops, T, H, K):
    from smolmoe_c99_b200.kernels.ops import NormedRows
    res = _rand((T, K), torch.float32, 7)
    nw = (_rand((K,), torch.bfloat16, 8, 0.2).float() + 1).to(torch.bfloat16)
    w = _rand((2 * H, K), torch.bfloat16, 6, 0.05)
    eps = 1e-5
    xn = ops.rmsnorm(res, nw, eps, torch.bfloat16)   # the stand-alone kernel
    ref = res * torch.rsqrt((res * res).mean(dim=1, keepdim=True) + eps) * nw.float()
    assert float((xn.float() - ref).abs().max()) <= 8e-3 * float(ref.abs().max())
    g, u = xn.float() @ w[:H].float().T, xn.float() @ w[H:].float().T
    want = u * (g / (1 + torch.exp(-g)))
    lazy = NormedRows(ops, res, nw, eps, torch.bfloat16)
    got = ops.gemm_skinny(lazy, w, None, torch.empty((T, H), dtype=torch.bfloat16, device="cuda"), mode=2, up_offset=H)
    assert float((got.float() - want).abs().max()) <= 1e-2 * float(want.abs().max()) + 1e-3


def _torch_qkv_rope_pools(x, w, b, positions, slots, table, cos, sin, heads, kv_heads, hd, n_pages):
    """Product, bias, rotation of q and k on pairs (i, i + hd/2) and the cache cells they belong in, computed
    with PyTorch in float (no kernel of the library): returns q [T, heads, hd] and the two expected pools."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    T = x.shape[0]
    qkv = x.float() @ w.float().T + b.float()
    q, k, v = qkv.split([heads * hd, kv_heads * hd, kv_heads * hd], dim=1)
    c, s_ = cos[positions.long()][:, None, :], sin[positions.long()][:, None, :]

    def rot(t):
        lo, hi = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([lo * c - hi * s_, lo * s_ + hi * c], dim=-1)

    q, k, v = rot(q.view(T, heads, hd)), rot(k.view(T, kv_heads, hd)), v.reshape(T, kv_heads, hd)
    k_pool = torch.zeros((n_pages, kv_heads, PAGE_SIZE, hd), dtype=torch.float32, device=x.device)
    v_pool = torch.zeros_like(k_pool)
    for t in range(T):
        pos, slot = int(positions[t]), int(slots[t])
        page = int(table[slot, pos // PAGE_SIZE])
        k_pool[page, :, pos % PAGE_SIZE] = k[t]
        v_pool[page, :, pos % PAGE_SIZE] = v[t]
    return q, k_pool, v_pool


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (3, 1, 32), (14, 2, 64), (5, 5, 48)])
def test_fused_qkv_matches_the_separate_kernels(ops, heads, kv_heads, hd):
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    T, K = 5, 96
    N = (heads + 2 * kv_heads) * hd
    x, w, b = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.1), _rand((N,), torch.bfloat16, 3)
    positions = torch.tensor([0, 7, 63, 64, 130], dtype=torch.int32).cuda()
    slots = torch.tensor([2, 0, 4, 1, 3], dtype=torch.int32).cuda()
    table = torch.randperm(20, generator=torch.Generator().manual_seed(3)).to(torch.int32).view(5, 4).cuda()
    half = hd // 2
    ang = torch.arange(200, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                                                                        -torch.arange(half, dtype=torch.float64) * 2 / hd)
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    pools = [torch.zeros((20, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    ends = positions + 1
    qkv = ops.gemm_simt(x, w, b, torch.empty((T, N), dtype=torch.float32, device="cuda"))
    q_ref, _, _ = ops.rope_store(qkv, positions, cos, sin, heads, kv_heads, hd, hd, torch.bfloat16, False, pools[0], pools[1],
                                 table, 0, slots, ends)
    q = ops.qkv_rope_store_fused(x, w, b, positions, cos, sin, heads, kv_heads, hd, hd, pools[2], pools[3], table, 0, slots)
    assert q is not None
    assert float((q.float() - q_ref.float()).abs().max()) <= 2e-2
    assert float((pools[2].float() - pools[0].float()).abs().max()) <= 2e-2
    assert float((pools[3].float() - pools[1].float()).abs().max()) <= 2e-2
    assert int((pools[2] != 0).sum()) == int((pools[0] != 0).sum())   # the same cells were written
    # and against a computation that uses no kernel of the library
    q_t, k_t, v_t = _torch_qkv_rope_pools(x, w, b, positions, slots, table, cos, sin, heads, kv_heads, hd, 20)
    tol = 8e-3 * float(q_t.abs().max())
    assert float((q.float() - q_t).abs().max()) <= tol
    assert float((pools[2].float() - k_t).abs().max()) <= tol and float((pools[3].float() - v_t).abs().max()) <= tol
    assert torch.equal(pools[2] != 0, k_t != 0) and torch.equal(pools[3] != 0, v_t != 0)


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (3, 1, 32), (14, 2, 64), (8, 2, 128), (28, 4, 128)])
@pytest.mark.parametrize("T,K", [(17, 96), (40, 896), (64, 3584), (100, 896), (160, 264)])
def test_fused_qkv_on_the_tcgen05_kernel_matches_the_separate_kernels(ops, heads, kv_heads, hd, T, K):
    """17 to 160 tokens: bias, rotation and the cache write happen where the split-K cluster of the tcgen05 kernel adds
    its sums up (one split included). Unequal positions, scattered pages, row counts that are no multiple of 128."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    N = (heads + 2 * kv_heads) * hd
    x, w, b = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05), _rand((N,), torch.bfloat16, 3)
    g = torch.Generator().manual_seed(9)
    positions = torch.randint(0, 4 * PAGE_SIZE, (T,), generator=g).to(torch.int32).cuda()
    slots = torch.randperm(T, generator=g).to(torch.int32).cuda()
    table = torch.randperm(T * 4, generator=g).to(torch.int32).view(T, 4).cuda()
    half = hd // 2
    ang = torch.arange(4 * PAGE_SIZE, dtype=torch.float64)[:, None] * torch.pow(
        torch.tensor(10000.0, dtype=torch.float64), -torch.arange(half, dtype=torch.float64) * 2 / hd)
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    pools = [torch.zeros((T * 4, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    qkv = ops.gemm_simt(x, w, b, torch.empty((T, N), dtype=torch.float32, device="cuda"))
    q_ref, _, _ = ops.rope_store(qkv, positions, cos, sin, heads, kv_heads, hd, hd, torch.bfloat16, False, pools[0], pools[1],
                                 table, 0, slots, positions + 1)
    q = ops.qkv_rope_store_fused(x, w, b, positions, cos, sin, heads, kv_heads, hd, hd, pools[2], pools[3], table, 0, slots)
    ops.check_error_flag()
    import ctypes
    tile_n, splits = ctypes.c_int(), ctypes.c_int()
    ops._check(ops.lib.sm_gemm_tc_plan(T, N, K, 0, ctypes.byref(tile_n), ctypes.byref(splits)))
    if splits.value > 8:      # K split more ways than a cluster has CTAs (a few rows, a long K): left to the separate kernels
        assert q is None and float(pools[2].abs().max()) == 0.0
        return
    assert q is not None, "the fused tcgen05 path did not take this shape"
    tol = 1e-3 * math.sqrt(K) * 0.05 + 8e-3 * float(q_ref.float().abs().max())
    assert float((q.float() - q_ref.float()).abs().max()) <= tol
    assert float((pools[2].float() - pools[0].float()).abs().max()) <= tol
    assert float((pools[3].float() - pools[1].float()).abs().max()) <= tol
    assert int((pools[2] != 0).sum()) == int((pools[0] != 0).sum())   # the same cells were written
    assert int((pools[3] != 0).sum()) == int((pools[1] != 0).sum())
    # and against a computation that uses no kernel of the library. Two tokens may share a cell here (positions
    # and pages are drawn at random), so cells are compared where exactly one token writes
    q_t, k_t, v_t = _torch_qkv_rope_pools(x, w, b, positions, slots, table, cos, sin, heads, kv_heads, hd, T * 4)
    assert float((q.float() - q_t).abs().max()) <= tol
    cells = [(int(table[int(slots[t]), int(positions[t]) // PAGE_SIZE]), int(positions[t]) % PAGE_SIZE) for t in range(T)]
    once = [c for c in cells if cells.count(c) == 1]
    assert len(once) >= T - 4
    for page, row in once:
        assert float((pools[2][page, :, row].float() - k_t[page, :, row]).abs().max()) <= tol
        assert float((pools[3][page, :, row].float() - v_t[page, :, row]).abs().max()) <= tol


@pytest.mark.parametrize("heads,kv_heads,hd", [(14, 2, 64), (3, 1, 128), (8, 2, 128), (5, 3, 64), (4, 0, 64)])
@pytest.mark.parametrize("T,K,ring", [(512, 896, 0), (777, 136, 0), (2048, 896, 0), (900, 264, 256), (161, 896, 0), (200, 136, 128),
                                      # up to 160 tokens the small kernel's epilogue does it, for a handful of tokens
                                      # the weight-streaming kernel's
                                      (20, 896, 0), (100, 136, 0), (160, 264, 128), (5, 96, 0), (12, 264, 128)])
def test_fused_qkv_of_many_tokens(ops, heads, kv_heads, hd, T, K, ring):
    """More than 160 tokens: bias, rotation, the packed keys and values and the cache write in the epilogue of the
    two-CTA product, against PyTorch in float. Two sequences that go on from unequal positions, scattered pages; with
    a ring, the positions that it has no place for any more must not be written."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    N = (heads + 2 * kv_heads) * hd
    x, w, b = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05), _rand((N,), torch.bfloat16, 3)
    first = T // 3
    starts, lens = [37, 0], [first, T - first]
    positions = torch.cat([torch.arange(s0, s0 + n) for s0, n in zip(starts, lens)]).to(torch.int32).cuda()
    token_slot = torch.cat([torch.full((n,), slot) for slot, n in zip([1, 0], lens)]).to(torch.int32).cuda()
    token_end = torch.cat([torch.full((n,), s0 + n) for s0, n in zip(starts, lens)]).to(torch.int32).cuda()
    pages_per_slot = (ring or (max(s0 + n for s0, n in zip(starts, lens)) + PAGE_SIZE)) // PAGE_SIZE + (0 if ring else 1)
    g = torch.Generator().manual_seed(9)
    table = torch.randperm(2 * pages_per_slot, generator=g).to(torch.int32).view(2, pages_per_slot).cuda()
    n_pos = int(positions.max()) + 1
    half = hd // 2
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * torch.pow(
        torch.tensor(1e6, dtype=torch.float64), -torch.arange(half, dtype=torch.float64) * 2 / hd)
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    kvh = max(kv_heads, 1)
    k_pool = torch.zeros((2 * pages_per_slot, kvh, PAGE_SIZE, hd), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    got = ops.qkv_rope_store_many(x, w, b, positions, cos, sin, heads, kv_heads, hd, hd, want_packed=True, k_pool=k_pool,
                                  v_pool=v_pool, page_table=table, ring=ring, token_slot=token_slot, token_end=token_end)
    ops.check_error_flag()
    assert got is not None, "the two-CTA kernel did not take this product"
    q, kp, vp = got
    qkv = x.float() @ w.float().T + b.float()
    q_t, k_t, v_t = qkv.split([heads * hd, kv_heads * hd, kv_heads * hd], dim=1)
    c, s_ = cos[positions.long()][:, None, :], sin[positions.long()][:, None, :]

    def rot(t):
        lo, hi = t[..., :half], t[..., half:]
        return torch.cat([lo * c - hi * s_, lo * s_ + hi * c], dim=-1)

    q_t = rot(q_t.reshape(T, heads, hd))
    tol = 1e-3 * math.sqrt(K) * 0.05 + 8e-3 * float(q_t.abs().max())
    assert float((q.float() - q_t).abs().max()) <= tol
    if not kv_heads:
        assert kp is None and vp is None and float(k_pool.abs().max()) == 0.0
        return
    k_t, v_t = rot(k_t.reshape(T, kv_heads, hd)), v_t.reshape(T, kv_heads, hd)
    assert float((kp.float() - k_t).abs().max()) <= tol and float((vp.float() - v_t).abs().max()) <= tol
    want_k, want_v = torch.zeros_like(k_pool, dtype=torch.float32), torch.zeros_like(v_pool, dtype=torch.float32)
    for t in range(T):
        pos, slot, end = int(positions[t]), int(token_slot[t]), int(token_end[t])
        if ring and pos < end - ring:
            continue
        idx = pos % ring if ring else pos
        page = int(table[slot, idx // PAGE_SIZE])
        want_k[page, :, idx % PAGE_SIZE] = k_t[t]
        want_v[page, :, idx % PAGE_SIZE] = v_t[t]
    assert float((k_pool.float() - want_k).abs().max()) <= tol and float((v_pool.float() - want_v).abs().max()) <= tol
    assert torch.equal(k_pool != 0, want_k != 0) and torch.equal(v_pool != 0, want_v != 0)


def test_fused_qkv_refuses_heads_that_straddle_tiles(ops):
    """Head sizes that do not divide 128 are left to the separate kernels."""
    from smolmoe_c99_b200.kernels import PAGE_SIZE
    heads, kv_heads, hd, T, K = 5, 5, 48, 20, 96
    N = (heads + 2 * kv_heads) * hd
    x, w = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05)
    positions = torch.arange(T, dtype=torch.int32).cuda()
    table = torch.arange(T, dtype=torch.int32).view(T, 1).cuda()
    cos = torch.ones((PAGE_SIZE, hd // 2), device="cuda"); sin = torch.zeros_like(cos)
    pool = torch.zeros((T, kv_heads, PAGE_SIZE, hd), dtype=torch.bfloat16, device="cuda")
    assert ops.qkv_rope_store_fused(x, w, None, positions, cos, sin, heads, kv_heads, hd, hd, pool, pool.clone(), table, 0,
                                    positions) is None
    assert float(pool.abs().max()) == 0.0
