"""CPU, two gloo ranks: the N-sharded path end to end on the host -- shard the
weights the way bench.py does, compute each shard with the CPU oracle, all-gather
the outputs, and compare with the unsharded oracle; reduce the per-rank argmax
pairs with the reference's tie rule.  No GPU and no product kernel is involved:
this covers the host-side logic of the multi-GPU path."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_sharding():
    spec = importlib.util.spec_from_file_location("mc_sharding", os.path.join(ROOT, "minicpm5-5080fast_b200", "sharding.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shard_rows_cover_exactly():
    sh = _load_sharding()
    for n in (2304, 3456, 5760, 122753, 17, 8):
        for world in (1, 2, 4, 8):
            spans = [sh.shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            per = spans[0][2]
            assert per % 8 == 0 and per * world >= n
            assert all(s[1] - s[0] == per for s in spans if s[1] < n)
    assert sh.shard_rows(122753, 8, 7) == (107464, 122753, 15352)


def test_reduce_argmax_pairs_tie_rule():
    sh = _load_sharding()
    assert sh.reduce_argmax_pairs([1.0, 3.0, 3.0, 2.0], [10, 700, 300, 5]) == (3.0, 300)
    assert sh.reduce_argmax_pairs([float("nan"), 1.0], [0, 9]) == (1.0, 9)
    assert sh.reduce_argmax_pairs([float("-inf")] * 2, [4, 2]) == (float("-inf"), 2)


def _worker(rank, world, port, q):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import torch.distributed as dist
    import oracle_np as onp
    sh = _load_sharding()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        K, N, I, V = 256, 1000, 96, 4099             # N, V not multiples of the shard pitch
        w = onp.seeded_bf16(1, (N, K), 0.02)
        wgu = onp.seeded_bf16(2, (2 * I, K), 0.02)
        wv = onp.seeded_bf16(3, (V, K), 0.02)
        x = onp.seeded_bf16(4, (K,), 1.0)

        def gather(shard_u16, per):
            mine = torch.zeros(2 * per, dtype=torch.uint8)          # gloo has no 16-bit integers: ship bytes
            mine[:2 * shard_u16.size] = torch.from_numpy(np.ascontiguousarray(shard_u16).view(np.uint8))
            full = torch.zeros(world * 2 * per, dtype=torch.uint8)
            dist.all_gather_into_tensor(full, mine)
            return full.numpy().view(np.uint16)

        # plain linear
        lo, hi, per = sh.shard_rows(N, world, rank)
        y = gather(onp.linear_bf16(w[lo:hi], x), per)[:N]
        ok1 = np.array_equal(y, onp.linear_bf16(w, x))
        # gate_up sharded by pairs, SwiGLU before the gather
        lo, hi, per = sh.shard_gate_up(I, world, rank)
        w_sh = np.concatenate([wgu[:I][lo:hi], wgu[I:][lo:hi]])
        mid = gather(onp.gate_up_swiglu_bf16(w_sh, x), per)[:I]
        ok2 = np.array_equal(mid, onp.gate_up_swiglu_bf16(wgu, x))
        # vocab-parallel lm_head: only (value, index) pairs travel
        lo, hi, per = sh.shard_rows(V, world, rank)
        logits = onp.linear_bf16(wv[lo:hi], x)
        lf = onp.bf16_to_f32(logits)
        pair = torch.tensor([float(lf.max()), float(int(lf.argmax()) + lo)] if lf.size else [float("-inf"), 2.0 ** 31 - 1],
                            dtype=torch.float64)
        pairs = torch.zeros(world * 2, dtype=torch.float64)
        dist.all_gather_into_tensor(pairs, pair)
        v, i = sh.reduce_argmax_pairs(pairs[0::2].tolist(), pairs[1::2].tolist())
        ok3 = i == onp.greedy(onp.linear_bf16(wv, x))
        q.put((rank, bool(ok1), bool(ok2), bool(ok3)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_gloo_sharded_linears_match_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in res), res
