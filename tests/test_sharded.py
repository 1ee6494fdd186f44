"""N-sharded linears whose output exchange runs inside the GEMV kernel.

One GPU is enough for the kernels themselves: the ranks of a small "world" are run one
after another in one process, all "peer" buffers being local, in an order in which every
wait is already satisfied when its kernel starts (no kernel ever waits for a later
launch).  The whole sharded stack, where ranks do wait for each other, runs as one
process per GPU and is skipped with fewer than two devices."""
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle_np as onp
from parity import check_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sharded_layout_cpu(pkg):
    from importlib import import_module
    sh = import_module("minicpm5-5080fast_b200.sharding")
    L, H, Q, I, V = 2, 256, 384, 512, 1001
    one = pkg.stack_desc(L, H, Q, I, V)
    assert pkg.stack_exchange_bytes(one) == 0
    for world in (2, 4, 8):
        total_lm = 0
        for rank in range(world):
            d = pkg.stack_desc(L, H, Q, I, V, fp8=True, world=world, rank=rank)
            rows = lambda n: (lambda lo, hi, per: hi - lo)(*sh.shard_rows(n, world, rank))
            assert pkg.stack_section(d, 0, "qkv")[1] == rows(Q) * H
            assert pkg.stack_section(d, 1, "o")[1] == rows(H) * H
            assert pkg.stack_section(d, 0, "gate_up")[1] == 2 * rows(I) * H
            assert pkg.stack_section(d, 0, "gate_up_scale")[1] == 2 * rows(I) * 4
            assert pkg.stack_section(d, 0, "down")[1] == rows(H) * I
            assert pkg.stack_section(d, 0, "norm1")[1] == H * 2          # norm weights are not sharded
            total_lm += pkg.stack_section(d, 0, "lm_head")[1]
            assert pkg.stack_exchange_bytes(d) > 0 and pkg.stack_exchange_bytes(d) % 256 == 0
        assert total_lm == V * H
    with pytest.raises(pkg.McError):
        pkg.stack_sizes(pkg.stack_desc(L, H, Q, I, V, world=2, rank=2))
    with pytest.raises(pkg.McError):
        pkg.stack_sizes(pkg.stack_desc(L, H, Q, I, V, world=9, rank=0))
    with pytest.raises(pkg.McError):                                  # 8 ranks x pitch 8 > 40 rows: a rank would own nothing
        pkg.stack_sizes(pkg.stack_desc(L, 40, 48, 64, V, world=8, rank=0))


@pytest.fixture(scope="module")
def g(pkg):
    torch = pytest.importorskip("torch")
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert pkg.device_check()["cc"][0] == 10
    import gpu_util
    return gpu_util


class World:
    """A few ranks in one process: per rank a gathered vector of tagged words."""

    def __init__(self, torch, world, pitch):
        self.world, self.pitch = world, pitch
        self.gathered = [torch.zeros(world * pitch, dtype=torch.int32, device="cuda") for _ in range(world)]
        self.step = torch.ones(1, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def producer(self, pkg, rank, seq=5):
        return pkg.shard_io(self.world, rank, self.step, self.status, out_slot=self.pitch, out_seq=(1, seq),
                            out_peer=[t.data_ptr() for t in self.gathered])

    def consumer(self, pkg, rank, seq=5, timeout_ns=0):
        return pkg.shard_io(self.world, rank, self.step, self.status, in_seq=(1, seq), timeout_ns=timeout_ns)

    def values(self, rank, n):
        """(bf16 bits, tags) of the first n words of a rank's gathered vector."""
        w = self.gathered[rank].cpu().numpy().view(np.uint32)[:n]
        return (w & 0xFFFF).astype(np.uint16), (w >> 16)


def _shards(n, world):
    pitch = ((n + world - 1) // world + 7) // 8 * 8
    return pitch, [(min(n, r * pitch), min(n, (r + 1) * pitch)) for r in range(world)]


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("world", [2, 3])
def test_push_then_consume(pkg, g, fp8, world):
    import torch
    N, K = 992, 512
    w = onp.seeded_bf16(910, (N, K), 0.02)
    x = onp.seeded_bf16(911, (K,), 1.0)
    q, sc = onp.make_fp8_weight(w) if fp8 else (w, None)
    ref = onp.linear_fp8(q, sc, x) if fp8 else onp.linear_bf16(w, x)
    pitch, spans = _shards(N, world)
    wd = World(torch, world, pitch)
    dx = g.dev(x)
    for r, (lo, hi) in enumerate(spans):
        pkg.gemv_sharded(0, 0, g.dev(q[lo:hi]), g.dev(sc[lo:hi]) if fp8 else None, dx, None, None, None, None, hi - lo, K,
                         0.0, wd.producer(pkg, r))
    g.sync()
    whole = g.empty_u16(N)                                   # the same linear, not sharded
    if fp8:
        pkg.launch_gemv_fp8(g.dev(q), g.dev(sc), dx, whole, N, K)
    else:
        pkg.launch_decode_gemv(g.dev(q), dx, whole, N, K)
    g.sync()
    for r in range(world):
        got, tags = wd.values(r, N)
        assert np.all(tags == 5), "every word carries the exchange's sequence tag"
        check_close(got, ref, what="sharded push rank %d" % r)
        assert np.array_equal(got, g.host_u16(whole)), "a row's result must not depend on the sharding"
    assert wd.status.item() == 0

    # consumer: residual add + RMSNorm prologue over the gathered vector, output local
    N2 = 264
    w2 = onp.seeded_bf16(912, (N2, N), 0.02)
    q2, sc2 = onp.make_fp8_weight(w2) if fp8 else (w2, None)
    dq2, dsc2 = g.dev(q2), (g.dev(sc2) if fp8 else None)
    res_in = g.dev(onp.seeded_bf16(913, (N,), 1.0))
    nw = g.dev(onp.f32_to_bf16(1.0 + 0.1 * np.random.default_rng(914).standard_normal(N).astype(np.float32)))
    outs = []
    for kind in ("sharded", "plain"):
        res_out, y = g.empty_u16(N), g.empty_u16(N2)
        addend = g.dev(wd.values(0, N)[0])
        if kind == "sharded":
            pkg.gemv_sharded(1, 0, dq2, dsc2, res_in, wd.gathered[0], nw, res_out, y, N2, N, 1e-6, wd.consumer(pkg, 0))
        elif fp8:
            pkg.launch_gemv_fp8_prologue(dq2, dsc2, res_in, addend, nw, res_out, y, N2, N, 1e-6)
        else:
            pkg.launch_gemv_rows_prologue(dq2, res_in, addend, nw, res_out, y, N2, N, 1e-6)
        g.sync()
        outs.append((g.host_u16(res_out), g.host_u16(y)))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert wd.status.item() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_push_swiglu_pairs(pkg, g, fp8):
    import torch
    I, K, world = 520, 256, 2
    gate, up = onp.seeded_bf16(920, (I, K), 0.02), onp.seeded_bf16(921, (I, K), 0.02)
    x = onp.seeded_bf16(922, (K,), 1.0)
    il = np.empty((2 * I, K), dtype=np.uint16)
    il[0::2], il[1::2] = gate, up
    q, sc = onp.make_fp8_weight(il) if fp8 else (il, None)
    lin = (lambda m, s: onp.linear_fp8(m, s, x)) if fp8 else (lambda m, s: onp.linear_bf16(m, x))
    full = lin(q, sc)
    ref = onp.swiglu_bf16(full[0::2], full[1::2])
    pitch, spans = _shards(I, world)
    wd = World(torch, world, pitch)
    dx = g.dev(x)
    for r, (lo, hi) in enumerate(spans):
        pkg.gemv_sharded(0, 1, g.dev(q[2 * lo:2 * hi]), g.dev(sc[2 * lo:2 * hi]) if fp8 else None, dx, None, None, None, None,
                         2 * (hi - lo), K, 0.0, wd.producer(pkg, r))
    g.sync()
    for r in range(world):
        got, tags = wd.values(r, I)
        assert np.all(tags == 5)
        check_close(got, ref, what="sharded swiglu rank %d" % r)
    assert np.array_equal(wd.values(0, I)[0], wd.values(1, I)[0])


@pytest.mark.gpu
def test_wait_is_bounded_and_sticky(pkg, g):
    """Words whose tag never becomes current: the consumer gives up after the limit, records it, and
    the context stays usable; later waits give up at once."""
    import time
    import torch
    N, K = 64, 256
    wd = World(torch, 2, 128)
    w = g.dev(onp.seeded_bf16(930, (N, K), 0.02))
    y = g.empty_u16(N)
    pkg.gemv_sharded(0, 0, w, None, wd.gathered[0], None, None, None, y, N, K, 0.0, wd.consumer(pkg, 0, timeout_ns=5_000_000))
    g.sync()
    assert wd.status.item() == 1
    t0 = time.perf_counter()
    for _ in range(20):                                      # 20 x 1 s if the failure were not sticky
        pkg.gemv_sharded(0, 0, w, None, wd.gathered[0], None, None, None, y, N, K, 0.0, wd.consumer(pkg, 0))
    g.sync()
    assert time.perf_counter() - t0 < 2.0
    # the context is healthy: an ordinary call still gives the right answer
    x = onp.seeded_bf16(931, (K,), 1.0)
    pkg.launch_decode_gemv(w, g.dev(x), y, N, K)
    g.sync()
    check_close(g.host_u16(y), onp.linear_bf16(onp.seeded_bf16(930, (N, K), 0.02), x), what="after timeout")


@pytest.mark.gpu
def test_peer_argmax_reduces_pairs(pkg, g):
    import torch
    world = 4
    pairs = torch.zeros(8, dtype=torch.int64, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # ranks 0, 2, 3 have delivered already; this process plays rank 1.  Tie between 1 and 3 -> lower index wins.
    vals, idxs = [1.5, 2.25, -3.0, 2.25], [7, 90, 5, 40]
    for r in (0, 2, 3):
        pairs[r] = int(np.float32(vals[r]).view(np.uint32)) | (idxs[r] << 32)
        flags[r] = 1
    table_p = torch.tensor([pairs.data_ptr()] * world, dtype=torch.int64, device="cuda")
    table_f = torch.tensor([flags.data_ptr()] * world, dtype=torch.int64, device="cuda")
    val = torch.tensor([vals[1]], dtype=torch.float32, device="cuda")
    idx = torch.tensor([idxs[1]], dtype=torch.int32, device="cuda")
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    tv = torch.zeros(1, dtype=torch.float32, device="cuda")
    pkg.peer_argmax(val, idx, table_p, table_f, pairs, flags, step, 1, world, status, tok, tv)
    g.sync()
    assert tok.item() == 40 and tv.item() == 2.25 and step.item() == 2 and status.item() == 0
    assert flags[1].item() == world                          # every "peer" is this buffer: four arrivals
    # next step: nobody else delivers -> bounded wait, sticky failure, step still advances
    pkg.peer_argmax(val, idx, table_p, table_f, pairs, flags, step, 1, world, status, tok, tv, timeout_ns=2_000_000)
    g.sync()
    assert status.item() == 1 and step.item() == 3


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_sharded_batched_stack_two_gpus(pkg, g, fp8):
    """M = 8 on two GPUs: the tensor-core GEMMs store into every rank's [M, width] buffers themselves and the consumers wait
    for their arrival counters; one step with 3 rows in between (e4m3: CUDA-core kernels + gather kernels) on the same stack;
    logits within tolerance of one GPU."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29743", os.path.join(ROOT, "tests", "sharded_worker.py"), "--rows", "8", "--mix"] + (["--fp8"] if fp8 else [])
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "SHARDED-OK" in out.stdout, out.stdout[-2000:]


@pytest.mark.gpu
def test_peer_allgather_rows_and_batched_argmax(pkg, g):
    """One GPU, world of two played in sequence: 2-D scatter into both 'ranks' buffers, then the M-row pair reduce."""
    import torch
    M, width, pitch = 3, 40, 24                      # rank 0 owns columns [0, 24), rank 1 [24, 40)
    bufs = [torch.zeros((M, width), dtype=torch.int16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tb = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    tf = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device="cuda")
    shards = [torch.arange(M * 24, dtype=torch.int16, device="cuda").reshape(M, 24) + 100,
              torch.arange(M * 16, dtype=torch.int16, device="cuda").reshape(M, 16) + 1000]
    # rank 1 first with a short limit: rank 0 has not delivered -> bounded wait runs out, data still lands
    pkg.peer_allgather_rows(shards[1], M, 32, width * 2, pitch * 2, tb, tf, flags[1], epochs[1], 1, 2, timeout_ns=2_000_000, status=status)
    g.sync()
    assert status.item() == 1 and epochs[1].item() == 1
    # sticky: with the failure word set, a second gather does not wait again (its limit is 5 s here),
    # still delivers and still advances its epoch
    import time
    t0 = time.perf_counter()
    pkg.peer_allgather_rows(shards[1], M, 32, width * 2, pitch * 2, tb, tf, flags[1], epochs[1], 1, 2, timeout_ns=5_000_000_000, status=status)
    g.sync()
    assert time.perf_counter() - t0 < 1.0 and status.item() == 1 and epochs[1].item() == 2
    status.zero_()
    pkg.peer_allgather_rows(shards[0], M, 48, width * 2, pitch * 2, tb, tf, flags[0], epochs[0], 0, 2, status=status)
    g.sync()
    assert status.item() == 0
    want = torch.cat((shards[0], shards[1]), dim=1)
    assert torch.equal(bufs[0], want) and torch.equal(bufs[1], want)
    # M-row greedy reduce: this process plays rank 0 of two, rank 1's pairs are already there
    pairs = torch.zeros(2 * M, dtype=torch.int64, device="cuda")
    pflags = torch.zeros(8, dtype=torch.int32, device="cuda")
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    other_v, other_i = [0.5, 3.0, -1.0], [900, 901, 902]
    for m in range(M):
        pairs[M + m] = int(np.float32(other_v[m]).view(np.uint32)) | (other_i[m] << 32)
    pflags[1] = 1
    tp = torch.tensor([pairs.data_ptr()] * 2, dtype=torch.int64, device="cuda")
    tfl = torch.tensor([pflags.data_ptr()] * 2, dtype=torch.int64, device="cuda")
    val = torch.tensor([1.5, 3.0, -2.0], dtype=torch.float32, device="cuda")
    idx = torch.tensor([10, 11, 12], dtype=torch.int32, device="cuda")
    tok = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    tv = torch.zeros(M, dtype=torch.float32, device="cuda")
    pkg.peer_argmax(val, idx, tp, tfl, pairs, pflags, step, 0, 2, status, tok, tv, n_rows=M)
    g.sync()
    assert tok.tolist() == [10, 11, 902] and tv.tolist() == [1.5, 3.0, -1.0] and step.item() == 2 and status.item() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_sharded_stack_two_gpus(pkg, g, fp8):
    """One process per GPU: tokens and logits of the sharded stack equal the one-GPU stack's."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(ROOT, "tests", "sharded_worker.py")] + (["--fp8"] if fp8 else [])
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "SHARDED-OK" in out.stdout, out.stdout[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("N,K", [(3456, 2304), (2304, 5760), (20003, 2304)])
def test_row_results_do_not_depend_on_the_shard(pkg, g, fp8, N, K):
    """What lets a sharded run be checked bit for bit against one GPU: a row's M = 1 result is the same whichever rows
    travel with it.  The benchmark's shapes (and a ragged vocabulary-like height) cut for 2, 4 and 8 ranks pick other
    tile shapes, thread counts and rows per warp than the whole matrix; every shard must reproduce its rows exactly."""
    from importlib import import_module
    sh = import_module("minicpm5-5080fast_b200.sharding")
    w = onp.seeded_bf16(960 + N, (N, K), 0.02)
    x = onp.seeded_bf16(961 + N, (K,), 1.0)
    dx = g.dev(x)
    if fp8:
        q, sc = onp.make_fp8_weight(w)

    def run(lo, hi):
        dy = g.empty_u16(hi - lo)
        if fp8:
            pkg.launch_gemv_fp8(g.dev(q[lo:hi]), g.dev(sc[lo:hi]), dx, dy, hi - lo, K)
        else:
            pkg.launch_decode_gemv(g.dev(w[lo:hi]), dx, dy, hi - lo, K)
        g.sync()
        return g.host_u16(dy)

    full = run(0, N)
    for world in (2, 4, 8):
        for rank in range(world):
            lo, hi, _ = sh.shard_rows(N, world, rank)
            assert np.array_equal(run(lo, hi), full[lo:hi]), f"world {world} rank {rank}"
