"""One rank of the sharded-stack test (launched under torch.distributed.run, one process per GPU).

Every rank builds its shard of the same seeded model, binds an exchange region in
symmetric (peer-mapped) memory, steps the sharded stack, and compares tokens and its
logits shard with the one-GPU stack run on its own device."""
import argparse
import ctypes
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import oracle_np as onp   # noqa: E402
import stack_util as su   # noqa: E402


def upload_shard(pkg, torch, desc, w, fp8, world, rank):
    sh = importlib.import_module("minicpm5-5080fast_b200.sharding")
    wbytes, sbytes = pkg.stack_sizes(desc)
    arena = torch.zeros(wbytes, dtype=torch.uint8, device="cuda")
    scratch = torch.zeros(sbytes, dtype=torch.uint8, device="cuda")

    def put(layer, name, arr):
        off, n = pkg.stack_section(desc, layer, name)
        b = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        assert b.size == n, (name, b.size, n)
        arena[off:off + n] = torch.from_numpy(b).cuda()

    def put_mat(layer, name, mat, pairs=False):
        if pairs:
            I = mat.shape[0] // 2
            lo, hi, _ = sh.shard_rows(I, world, rank)
            il = np.empty((2 * (hi - lo), mat.shape[1]), dtype=mat.dtype)
            il[0::2], il[1::2] = mat[:I][lo:hi], mat[I:][lo:hi]
            part = il
        else:
            lo, hi, _ = sh.shard_rows(mat.shape[0], world, rank)
            part = mat[lo:hi]
        if fp8:
            q, sc = onp.make_fp8_weight(part)          # per-row scales: quantising a shard == a shard of the quantised
            put(layer, name, q)
            put(layer, name + "_scale", sc)
        else:
            put(layer, name, part)

    for l, lay in enumerate(w["layers"]):
        put_mat(l, "qkv", lay["qkv"]); put_mat(l, "o", lay["o"]); put_mat(l, "gate_up", lay["gate_up"], pairs=True)
        put_mat(l, "down", lay["down"]); put(l, "norm1", lay["norm1"]); put(l, "norm2", lay["norm2"])
    put_mat(0, "lm_head", w["lm_head"]); put(0, "final_norm", w["final_norm"])
    return arena, scratch


def read_logits(pkg, torch, st, n):
    out = torch.empty(n, dtype=torch.int16, device="cuda")
    ctypes.CDLL("libcudart.so").cudaMemcpy(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(pkg.stack_logits_ptr(st)),
                                            ctypes.c_size_t(n * 2), 3)
    return out.cpu().numpy().view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--rows", type=int, default=1, help="batch rows M")
    ap.add_argument("--mix", action="store_true", help="second trial with 3 rows: another kernel family (and exchange form) on the same stack")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = importlib.import_module("minicpm5-5080fast_b200")
    sh = importlib.import_module("minicpm5-5080fast_b200.sharding")
    layers, H, Q, I, V = 3, 512, 768, 1024, 4099
    w = su.make_weights(layers, H, Q, I, V)
    fp8 = args.fp8

    # the one-GPU stack on this device: the reference for tokens and logits
    MAXB = args.rows
    M = MAXB
    d1 = pkg.stack_desc(layers, H, Q, I, V, fp8=fp8, max_batch=M)
    a1, s1 = su.upload(pkg, torch, d1, w, fp8)
    st1 = pkg.stack_create(d1, a1, s1)

    dW = pkg.stack_desc(layers, H, Q, I, V, fp8=fp8, max_batch=M, world=world, rank=rank)
    aW, sW = upload_shard(pkg, torch, dW, w, fp8, world, rank)
    stW = pkg.stack_create(dW, aW, sW)
    region = symm.empty(pkg.stack_exchange_bytes(dW), dtype=torch.uint8, device="cuda")
    region.zero_()
    handle = symm.rendezvous(region, dist.group.WORLD)
    stream = torch.cuda.Stream()
    pkg.stack_bind_exchange(stW, [int(p) for p in handle.buffer_ptrs], timeout_ns=0, stream=stream)
    torch.cuda.synchronize()
    dist.barrier()

    lo, hi, _ = sh.shard_rows(V, world, rank)
    ok = True
    for trial in range(4):                                  # eager, capture, replay, replay with a new input
        M = 3 if (args.mix and trial == 1 and MAXB > 3) else MAXB
        x = onp.seeded_bf16(700 + (trial == 3), (M, H), 1.0)
        hx = torch.from_numpy(x.view(np.int16)).pin_memory()
        t1 = torch.full((M,), -1, dtype=torch.int32).pin_memory()
        tW = torch.full((M,), -2, dtype=torch.int32).pin_memory()
        pkg.stack_step_host(st1, hx, M, t1, stream)
        pkg.stack_step_host(stW, hx, M, tW, stream)
        full = read_logits(pkg, torch, st1, M * V).reshape(M, V)
        mine = read_logits(pkg, torch, stW, M * (hi - lo)).reshape(M, hi - lo)
        if M == 1:
            # one row: a row's arithmetic order does not depend on the sharding -> bit-equal
            if int(t1[0]) != int(tW[0]) or int(tW[0]) != onp.greedy(full[0]):
                ok = False
                print(f"rank {rank} trial {trial}: token {int(tW[0])} vs one-GPU {int(t1[0])} vs greedy {onp.greedy(full[0])}", flush=True)
            if not np.array_equal(mine, full[:, lo:hi]):
                ok = False
                print(f"rank {rank} trial {trial}: logits shard differs in {(mine != full[:, lo:hi]).sum()} of {hi - lo}", flush=True)
        else:
            # batched: the tensor-core kernel splits K by the matrix height, so shards round differently: tolerance
            gf, rf = onp.bf16_to_f32(mine).astype(np.float64), onp.bf16_to_f32(full[:, lo:hi]).astype(np.float64)
            rel = np.sqrt(((gf - rf) ** 2).sum() / max((rf ** 2).sum(), 1e-30))
            if not rel < 1e-2:
                ok = False
                print(f"rank {rank} trial {trial}: logits shard relL2 {rel:.3e}", flush=True)
            ff = onp.bf16_to_f32(full).astype(np.float64)
            for m in range(M):
                top = np.sort(ff[m])[-2:]
                if top[1] - top[0] > 0.05 and int(tW[m]) != int(np.argmax(ff[m])):
                    ok = False
                    print(f"rank {rank} trial {trial} row {m}: token {int(tW[m])} vs {int(np.argmax(ff[m]))}", flush=True)
                if not (0 <= int(tW[m]) < V):
                    ok = False
                    print(f"rank {rank} trial {trial} row {m}: token {int(tW[m])} out of range", flush=True)
    if pkg.stack_exchange_status(stW, stream) != 0:
        ok = False
        print(f"rank {rank}: a bounded wait ran out", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    if rank == 0 and int(flag) == 1:
        print("SHARDED-OK", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
