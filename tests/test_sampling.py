"""Top-k / top-p sampling: the numpy restatement of the reference's tail on CPU (known answers of the generator,
properties), the kernel against it on GPU, vocab shards played in sequence on one GPU."""
import numpy as np
import pytest

import oracle_np as onp


def test_generator_and_seed_known_answers():
    # splitmix64 and xorshift64* have published reference outputs: splitmix64 of 0 is 0xE220A8397B1DCDAF,
    # and the xorshift64* multiplier is the one of Vigna's paper; the draw is the upper half of the product
    assert onp.splitmix64(0) == 0xE220A8397B1DCDAF
    r, st = onp.rng_next(1)
    x = 1
    x ^= x >> 12; x = (x ^ (x << 25)) & ((1 << 64) - 1); x ^= x >> 27
    assert st == x and r == ((x * 2685821657736338717) & ((1 << 64) - 1)) >> 32
    assert onp.rng_next(st)[1] != st


def test_restatement_properties():
    rng = np.random.default_rng(5)
    logits = onp.f32_to_bf16(rng.standard_normal(5000).astype(np.float32) * 3)
    v = onp.bf16_to_f32(logits)
    tok, st, _ = onp.sample_topk_topp(logits, 0.8, 1.0, 1, 77)            # top_k = 1: greedy, generator untouched
    assert tok == onp.greedy(logits) and st == 77
    tok, st, _ = onp.sample_topk_topp(logits, 0.0, 0.9, 50, 77)           # temperature 0: greedy
    assert tok == onp.greedy(logits) and st == 77
    kth = np.sort(v)[-40]
    seen = set()
    state = onp.splitmix64(11)
    for _ in range(200):
        tok, state, _ = onp.sample_topk_topp(logits, 1.0, 1.0, 40, state)
        assert v[tok] >= kth                                            # always one of the 40 strongest
        seen.add(tok)
    assert len(seen) > 5
    tok, _, _ = onp.sample_topk_topp(logits, 1.0, 1e-6, 40, 123)          # a tiny top_p keeps the strongest only
    assert tok == onp.greedy(logits)


def _cfg(torch, rows):
    a = np.zeros((len(rows), 6), dtype=np.uint32)
    for i, (temp, top_p, top_k) in enumerate(rows):
        a[i, 0] = np.float32(temp).view(np.uint32); a[i, 1] = np.float32(top_p).view(np.uint32); a[i, 2] = top_k
        a[i, 3] = np.float32(1.0).view(np.uint32)
    return torch.from_numpy(a.view(np.int32)).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [122753, 4099, 100])
def test_kernel_matches_restatement(pkg, vocab):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(vocab)
    rows = [(0.7, 0.9, 40), (1.0, 1.0, 128), (1.3, 0.5, 8), (0.8, 0.95, 1), (0.0, 0.9, 50), (1.0, 0.999, 300), (0.5, 1.0, 2), (2.0, 0.3, 64)]
    M = len(rows)
    logits = onp.f32_to_bf16(rng.standard_normal((M, vocab)).astype(np.float32) * 2.5)
    logits[2, 10:60] = logits[2].max()                 # a plateau of equal strongest values: ties go to the lower indices
    logits[5, :] = onp.f32_to_bf16(np.float32([1.0]))[0]  # every logit equal
    d_logits = torch.from_numpy(logits.view(np.int16)).cuda()
    states = [onp.splitmix64(1000 + m) for m in range(M)]
    d_rng = torch.from_numpy(np.array(states, dtype=np.uint64).view(np.int64)).cuda()
    d_out = torch.full((M,), -7, dtype=torch.int32, device="cuda")
    cfg = _cfg(torch, rows)
    for step in range(6):                              # the generator state advances on the device from draw to draw
        pkg.sample_topk_topp(d_logits, M, vocab, vocab, cfg, d_rng, d_out)
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        new_states = d_rng.cpu().numpy().view(np.uint64)
        for m, (temp, top_p, top_k) in enumerate(rows):
            want, st, margin = onp.sample_topk_topp(logits[m], temp, top_p, top_k, states[m])
            assert int(new_states[m]) == st, (m, step)
            states[m] = st
            if margin > 1e-5:                          # an exp that differs in the last bit cannot move a draw this far from a boundary
                assert int(got[m]) == want, (m, step, int(got[m]), want)
            v = onp.bf16_to_f32(logits[m])
            k = max(1, min(top_k, 128))
            assert v[got[m]] >= np.sort(v)[-min(k, vocab)]


@pytest.mark.gpu
def test_sharded_ranks_in_sequence_draw_the_same_token(pkg):
    """Two vocab shards on one GPU, the 'ranks' launched one after the other.  Every rank stores its candidates into
    BOTH exchange regions, so the rank that runs second finds everything and must return the restatement's token over
    the whole vocabulary; the rank that runs first finds nothing from its peer and, with a short limit, gives up: token
    -1, failure word set, generator untouched, exchange number still advanced."""
    torch = pytest.importorskip("torch")
    vocab, M, world = 9000, 3, 2
    rng = np.random.default_rng(42)
    logits = onp.f32_to_bf16(rng.standard_normal((M, vocab)).astype(np.float32) * 2.5)
    split = 4504                                       # shard boundary (a multiple of 8)
    shards = [np.ascontiguousarray(logits[:, :split]), np.ascontiguousarray(logits[:, split:])]
    rows = [(0.9, 0.9, 50), (1.0, 1.0, 128), (0.7, 0.8, 5)]
    cfg = _cfg(torch, rows)
    nbytes = pkg.sampling_exchange_bytes(4, world)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    peers = torch.tensor([r.data_ptr() for r in regions], dtype=torch.int64, device="cuda")
    steps = [torch.tensor([1, 0], dtype=torch.int32, device="cuda") for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    states = [onp.splitmix64(500 + m) for m in range(M)]
    rngs = [torch.from_numpy(np.array(states, dtype=np.uint64).view(np.int64)).cuda() for _ in range(world)]
    outs = [torch.full((M,), -7, dtype=torch.int32, device="cuda") for _ in range(world)]
    d_sh = [torch.from_numpy(s.view(np.int16)).cuda() for s in shards]
    bases, widths = [0, split], [split, vocab - split]

    def run(rank, timeout_ns=0):
        pkg.sample_topk_topp_sharded(d_sh[rank], M, widths[rank], widths[rank], bases[rank], cfg, rngs[rank], outs[rank], peers,
                                     regions[rank], 4, steps[rank], rank, world, status, timeout_ns=timeout_ns)
        torch.cuda.synchronize()

    run(1, timeout_ns=2_000_000)                        # rank 0 has not delivered: bounded wait, -1, sticky word
    assert status.item() == 1 and outs[1].tolist() == [-1, -1, -1] and steps[1].tolist() == [2, 0]
    status.zero_()
    run(0)                                             # rank 1's candidates of exchange 1 are there: rank 0 completes exchange 1
    assert status.item() == 0 and steps[0].tolist() == [2, 0]
    want = [onp.sample_topk_topp(logits[m], *rows[m], states[m]) for m in range(M)]
    for m in range(M):
        if want[m][2] > 1e-5:
            assert outs[0][m].item() == want[m][0]
    # exchange 2 the other way round: rank 0 first (gives up), then rank 1 (finds rank 0's candidates of exchange 2)
    run(0, timeout_ns=2_000_000)
    assert status.item() == 1
    status.zero_()
    run(1)                                             # its generator has not drawn yet: the first call gave up before the draw
    assert status.item() == 0 and steps[1].tolist() == [3, 0]
    st1 = rngs[1].cpu().numpy().view(np.uint64)
    for m in range(M):
        w2 = onp.sample_topk_topp(logits[m], *rows[m], states[m])
        assert int(st1[m]) == w2[1]
        if w2[2] > 1e-5:
            assert outs[1][m].item() == w2[0]
