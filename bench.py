#!/usr/bin/env python
"""Benchmark of the B200 decode linear-layer path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|ref_gpu]
                    [--workload stream|qkv|gate_up|down|lm_head] [--dtype bf16|fp8] [--m M]

One "step" of the default workload is one pass of the full 40-layer decode
weight stream (per layer: fused qkv 2304->3456, o 2304->2304, gate_up
2304->11520 with SwiGLU, down 5760->2304; then lm_head 2304->122753 with the
greedy argmax) on seeded synthetic weights, M activation rows (default 1).  The
metric is the HBM throughput of that stream: algorithmic bytes (every weight,
scale, input and output counted once) divided by device time.  With N > 1 the
matrices are sharded along N (output rows) over the ranks, every output is
exchanged inside the producing kernel (peer stores over NVLink; NCCL only for
rendezvous and barriers), and the aggregate over all ranks is reported (strong
scaling: the total work is fixed).

What is timed is also checked: the token of the graph replay must equal the
eager step's, the logits must match a plain fp32 PyTorch statement of the same
chain on the same weights, and with N > 1 rank 0 also runs the one-GPU stack
and compares token and logits shard with the sharded run.  A mismatch exits
non-zero without a JSON line.  After the headline the default run measures the
single-linear configurations (one entry each under "configs").

`--impl reference` times the reference's own CPU implementation of the same
linears (its native cross-check compiled in place under oracle/_ref for bf16;
the C restatement of its fp8 statement for fp8) on the host cores, on a bounded
sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L, H, QKV, I, V = 40, 2304, 3456, 5760, 122753
if os.environ.get("MC_LAYERS"):          # profiler captures only: a shorter stack keeps the capture small
    L = int(os.environ["MC_LAYERS"])
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


import importlib.util as _ilu

_spec = _ilu.spec_from_file_location("mc_sharding", os.path.join(ROOT, "minicpm5-5080fast_b200", "sharding.py"))
_sh = _ilu.module_from_spec(_spec)
_spec.loader.exec_module(_sh)
roundup, shard_rows = _sh.roundup, _sh.shard_rows


def linear_bytes(n, k, m, wb, n_out=None):
    """Algorithmic bytes of one linear call: weights + row scales (fp8) + x + y."""
    n_out = n if n_out is None else n_out
    return n * k * wb + (4 * n if wb == 1 else 0) + 2 * m * k + 2 * m * n_out


def stream_bytes(m, wb, world=1, rank=0):
    tot = 0
    for n, k, pair in ((QKV, H, False), (H, H, False), (2 * I, H, True), (H, I, False)):
        if pair:
            lo, hi, _ = shard_rows(n // 2, world, rank)
            rows = 2 * (hi - lo)
            tot += L * linear_bytes(rows, k, m, wb, rows // 2)
        else:
            lo, hi, _ = shard_rows(n, world, rank)
            tot += L * linear_bytes(hi - lo, k, m, wb)
    lo, hi, _ = shard_rows(V, world, rank)
    return tot + linear_bytes(hi - lo, H, m, wb)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0, t1):
        """Keeps the samples taken between two wall-clock instants (the timed region)."""
        self.t0, self.t1 = t0, t1

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.th.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        t0, t1 = getattr(self, "t0", 0.0), getattr(self, "t1", float("inf"))
        inside = [r for (t, r) in self.rows if t0 <= t <= t1]
        for r in (inside or [r for (_, r) in self.rows]):
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# reference arm / cpu baseline (host cores)
# ------------------------------------------------------------------------------------------
def cpu_reference(dtype, m, budget_s, steps=1, warmup=0):
    """Times the reference's CPU implementation on one transformer layer's four
    linears (a bounded sample of the stream).  Returns (GB/s by algorithmic
    bytes, info).  Only this function and the tests execute anything of oracle/."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_np as onp
    # 1/40 of the stream: one layer's four linears and one fortieth of the lm_head rows
    shapes = [(QKV, H), (H, H), (2 * I, H), (H, I), ((V + L - 1) // L, H)]
    wb = 2 if dtype == "bf16" else 1
    sample_bytes = sum(linear_bytes(n, k, m, wb, n // 2 if i == 2 else n) for i, (n, k) in enumerate(shapes))
    ws = [onp.seeded_bf16(50 + i, s, 0.02) for i, s in enumerate(shapes)]
    xs = [onp.seeded_bf16(60 + i, (m, s[1]), 1.0) for i, s in enumerate(shapes)]
    ref_so = os.path.join(ROOT, "oracle", "_ref", "libref_native.so")
    port_so = os.path.join(ROOT, "oracle", "libcpu_ref.so")
    if dtype == "bf16" and os.path.exists(ref_so):
        lib = ctypes.CDLL(ref_so)
        lib.ref_native_threads.restype = ctypes.c_uint32
        cores, kind = int(lib.ref_native_threads()), "reference"

        def run():
            for w, x in zip(ws, xs):
                y = np.empty(w.shape[0], np.uint16)
                for r in range(m):
                    lib.ref_native_gemv(x[r].ctypes.data_as(ctypes.c_void_p), w.ctypes.data_as(ctypes.c_void_p),
                                        w.shape[0], w.shape[1], y.ctypes.data_as(ctypes.c_void_p))
    else:
        if not os.path.exists(port_so):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "libcpu_ref.so"])
        lib = ctypes.CDLL(port_so)
        cores, kind = os.cpu_count() or 1, "port"
        qs = [onp.make_fp8_weight(w) for w in ws] if dtype == "fp8" else None

        def run():
            for i, (w, x) in enumerate(zip(ws, xs)):
                y = np.empty((m, w.shape[0]), np.uint16)
                if dtype == "fp8":
                    q, sc = qs[i]
                    lib.oracle_linear_fp8(q.ctypes.data_as(ctypes.c_void_p), sc.ctypes.data_as(ctypes.c_void_p),
                                          x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p), None,
                                          m, w.shape[0], w.shape[1], 0, cores)
                else:
                    lib.oracle_linear_bf16(w.ctypes.data_as(ctypes.c_void_p), x.ctypes.data_as(ctypes.c_void_p),
                                           y.ctypes.data_as(ctypes.c_void_p), None, m, w.shape[0], w.shape[1], 0, cores)
    for _ in range(max(1, warmup)):
        run()
    t0 = time.perf_counter()
    n = 0
    while True:
        run()
        n += 1
        dt = time.perf_counter() - t0
        if n >= steps and (dt >= budget_s or steps > 1):
            break
    per = dt / n
    info = {"value": sample_bytes / per / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"1/40 of the stream (one layer: qkv, o, gate_up, down; {shapes[4][0]} of the lm_head rows), M={m}, {n} passes, {per * 1e3:.1f} ms per pass",
            "ms_per_pass": per * 1e3, "cpu_model": cpu_model()}
    if budget_s > 0:
        # second CPU figure: the reference's numpy statement (tools/reference_forward.py:158-172 restated in
        # oracle_np: upcast W and x to fp32 on every call, BLAS matmul, round to bf16) on the same sample
        qs2 = [onp.make_fp8_weight(w) for w in ws] if dtype == "fp8" else None

        def run_np():
            for i, (w, x) in enumerate(zip(ws, xs)):
                onp.linear_fp8(qs2[i][0], qs2[i][1], x) if dtype == "fp8" else onp.linear_bf16(w, x)
        run_np()
        t0, k = time.perf_counter(), 0
        while True:
            run_np()
            k += 1
            dtn = time.perf_counter() - t0
            if dtn >= min(3.0, budget_s):
                break
        info["numpy"] = {"value": sample_bytes / (dtn / k) / 1e9, "unit": "GB/s", "threads": os.cpu_count() or 1,
                         "ms_per_pass": dtn / k * 1e3, "what": "numpy fp32 matmul with per-call upcast of W, same sample"}
    return info


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    info = cpu_reference(args.dtype, args.m, budget_s=0.0, steps=max(args.steps, 1), warmup=max(args.warmup, 1))
    wb = 2 if args.dtype == "bf16" else 1
    line = {
        "impl": "reference", "metric": "decode_linear_hbm_throughput", "value": info["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": info["ms_per_pass"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": workload_name(args), "sample": info["sample"]},
        "cpu_baseline": {k: info[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": info["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_name(args):
    if getattr(args, "workload", "stream") != "stream":
        n, k, kind = Single.SHAPES[args.workload]
        extra = {0: "", 1: " + SwiGLU epilogue", 2: " + fused argmax"}[kind]
        w8 = ", W8A8 (activations quantised per row)" if args.dtype == "fp8" and args.m > 1 and os.environ.get("MC_W8A8", "0") == "1" else ""
        return f"single linear {args.workload} {k}->{n}{extra}, {args.dtype}{w8}, M={args.m}, rotating weight copies"
    return (f"config5 full {L}-layer decode weight stream (qkv 2304->3456, o 2304->2304, gate_up 2304->11520 + SwiGLU, "
            f"down 5760->2304, lm_head 2304->122753 + argmax), {args.dtype}, M={args.m}")


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class Stream:
    """Device-resident sharded weights of the synthetic stack plus the launch
    sequence of one decode step through the C ABI."""

    def __init__(self, pkg, torch, dtype, m, world, rank, dist):
        self.pkg, self.torch, self.m, self.world, self.rank, self.dist = pkg, torch, m, world, rank, dist
        self.fp8 = dtype == "fp8"
        dev = "cuda"
        g = torch.Generator(device=dev)
        g.manual_seed(20260908 + 5000)            # same seed on every rank: shards of one logical model
        self.layers = []
        self.handle = None
        self.desc = None
        # MC_GATHER: "fused" (default) = the library's sharded stack, outputs exchanged inside the GEMV
        # kernels; "peer" = per-call launches + the library's peer all-gather kernel; "nccl" = per-call
        # launches + ncclAllGather.  The last two are kept as comparison arms.
        self.gather_mode = os.environ.get("MC_GATHER", "fused") if world > 1 else None
        if world == 1 or self.gather_mode == "fused":
            # the weights live in the library's own arena layout (this rank's shard of it) and the
            # step is the library's decode-stack object (C ABI)
            self.desc = pkg.stack_desc(L, H, QKV, I, V, fp8=self.fp8, max_batch=max(m, 1), graph=True,
                                       world=world, rank=rank)
            wbytes, sbytes = pkg.stack_sizes(self.desc)
            self.arena = torch.zeros(wbytes, dtype=torch.uint8, device=dev)
            self.scratch = torch.zeros(sbytes, dtype=torch.uint8, device=dev)

        def place(layer, name, t):
            """Copies a generated tensor to its arena section and returns a view of it there."""
            if self.desc is None or t is None:
                return t
            off, n = pkg.stack_section(self.desc, layer, name)
            flat = t.contiguous().view(torch.uint8).reshape(-1)
            assert flat.numel() == n, (name, flat.numel(), n)
            self.arena[off:off + n].copy_(flat)
            return self.arena[off:off + n].view(t.dtype).view(t.shape)

        def bf16_bits(t):
            return t.to(torch.bfloat16).view(torch.int16)

        def make(n, k, lo, hi, pairs=False):
            """Rows [lo,hi) of a logical [n,k] N(0,0.02) matrix (drawn whole so every
            rank sees the same model), gate/up interleaved when pairs."""
            w = torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02
            w = w.to(torch.bfloat16).to(torch.float32)
            if pairs:
                half = n // 2
                w = torch.stack((w[:half][lo:hi], w[half:][lo:hi]), dim=1).reshape(-1, k)
            else:
                w = w[lo:hi]
            if not self.fp8:
                return bf16_bits(w).contiguous(), None
            sc = (w.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
            q = (w / sc[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
            return q, sc.contiguous()

        def placed(li, name, ws):
            w, sc = ws
            return place(li, name, w), place(li, name + "_scale", sc)

        for li in range(L):
            lay = {}
            lo, hi, _ = shard_rows(QKV, world, rank); lay["qkv"] = placed(li, "qkv", make(QKV, H, lo, hi))
            lo, hi, _ = shard_rows(H, world, rank); lay["o"] = placed(li, "o", make(H, H, lo, hi))
            lo, hi, _ = shard_rows(I, world, rank); lay["gu"] = placed(li, "gate_up", make(2 * I, H, lo, hi, pairs=True))
            lo, hi, _ = shard_rows(H, world, rank); lay["down"] = placed(li, "down", make(H, I, lo, hi))
            lay["n1"] = place(li, "norm1", bf16_bits(1.0 + 0.1 * torch.randn(H, generator=g, device=dev)))
            lay["n2"] = place(li, "norm2", bf16_bits(1.0 + 0.1 * torch.randn(H, generator=g, device=dev)))
            self.layers.append(lay)
        lo, hi, per = shard_rows(V, world, rank)
        self.v_lo, self.v_rows, self.v_per = lo, hi - lo, per
        self.lm = placed(0, "lm_head", make(V, H, lo, hi))
        self.nf = place(0, "final_norm", bf16_bits(1.0 + 0.1 * torch.randn(H, generator=g, device=dev)))
        if self.desc is not None:
            self.handle = pkg.stack_create(self.desc, self.arena, self.scratch)
            if world > 1:
                # exchange region in symmetric (peer-mapped) memory, same size on every rank
                import torch.distributed._symmetric_memory as symm
                self.region = symm.empty(pkg.stack_exchange_bytes(self.desc), dtype=torch.uint8, device=dev)
                self.region.zero_()
                hnd = symm.rendezvous(self.region, dist.group.WORLD)
                pkg.stack_bind_exchange(self.handle, [int(p) for p in hnd.buffer_ptrs])
                torch.cuda.synchronize()
                dist.barrier()
        z = lambda *s: torch.zeros(s, dtype=torch.int16, device=dev)
        self.per = {"qkv": shard_rows(QKV, world, 0)[2], "o": shard_rows(H, world, 0)[2],
                    "mid": shard_rows(I, world, 0)[2], "down": shard_rows(H, world, 0)[2]}
        gx = torch.Generator(device="cpu")
        gx.manual_seed(20260908 + 5999)           # the same activation on every rank
        self.x_in = torch.randn((m, H), generator=gx).to(torch.bfloat16).view(torch.int16).to(dev)
        self.res = [z(m, H), z(m, H)]
        self.qkv_s, self.qkv = z(m, self.per["qkv"]), z(world, m, self.per["qkv"])
        self.o_s, self.o = z(m, self.per["o"]), z(world, m, self.per["o"])
        self.mid_s, self.mid = z(m, self.per["mid"]), z(world, m, self.per["mid"])
        self.dn_s, self.dn = z(m, self.per["down"]), z(world, m, self.per["down"])
        self.logits = z(m, max(self.v_rows, 8))
        self.stage = torch.empty(pkg.argmax_stage_bytes(max(m, 1)), dtype=torch.uint8, device=dev)
        self.tok = torch.zeros(m, dtype=torch.int32, device=dev)
        self.val = torch.zeros(m, dtype=torch.float32, device=dev)
        self.pair = torch.zeros((world, m, 2), dtype=torch.float32, device=dev)
        self.launches = 0
        self.peer = None
        if world > 1 and m == 1 and self.gather_mode == "peer":
            try:
                self._setup_peer(dev)
            except Exception as e:      # no symmetric memory on this stack: NCCL all-gather, same kernels otherwise
                self.peer = None
                self.peer_error = f"{type(e).__name__}: {e}"[:120]
        if m != 1:
            if world != 1 and self.handle is None:
                raise SystemExit("bench: the batched (M > 1) sharded stream runs through the library's stack (MC_GATHER=fused)")
            if m > 64:
                raise SystemExit("bench: M <= 64")
            self.h = z(m, H)
            self.ctx = z(m, H)
            self.qkv_m, self.o_m, self.mid_m, self.dn_m = z(m, QKV), z(m, H), z(m, I), z(m, H)
            self.logits = z(m, V)

    def logits_view(self):
        """The bf16 logits [M, rows of this rank's vocab shard] the last step of the stack wrote."""
        if self.handle is None:
            return self.logits[:, :self.v_rows]
        off = self.pkg.stack_logits_ptr(self.handle) - self.scratch.data_ptr()
        n = self.m * self.v_rows
        return self.scratch[off:off + 2 * n].view(self.torch.int16).view(self.m, self.v_rows)

    def reference_logits(self, x_bits):
        """Plain PyTorch fp32 statement of the same chain on the same device-resident weights (one GPU):
        every stored intermediate rounded to bf16 where the library stores bf16.  The checker, never timed."""
        torch = self.torch
        assert self.world == 1
        bf = lambda t: t.to(torch.bfloat16).to(torch.float32)
        bits = lambda t: t.view(torch.bfloat16).to(torch.float32)

        def lin(ws, v):
            w, sc = ws
            if sc is None:
                return bf(v @ bits(w).T)
            return bf((v @ w.view(torch.float8_e4m3fn).to(torch.float32).T) * sc[None, :])

        def rms(v, nw):
            return bf(v * torch.rsqrt((v * v).mean(dim=1, keepdim=True) + 1e-6) * bits(nw)[None, :])

        res = bits(x_bits)
        for lay in self.layers:
            qkv = lin(lay["qkv"], rms(res, lay["n1"]))
            res = bf(res + lin(lay["o"], qkv[:, :H].contiguous()))
            gu = lin(lay["gu"], rms(res, lay["n2"]))           # rows interleaved: gate_j, up_j
            g, u = gu[:, 0::2], gu[:, 1::2]
            res = bf(res + lin(lay["down"], bf(g / (1.0 + torch.exp(-g)) * u)))
        return lin(self.lm, rms(res, self.nf))

    def _setup_peer(self, dev):
        """Gathered buffers in symmetric (peer-mapped) memory + flag arrays for the library's own
        all-gather kernel (mc_sm100_peer_allgather)."""
        import torch.distributed._symmetric_memory as symm
        torch, world, rank = self.torch, self.world, self.rank
        slots = {"qkv": self.per["qkv"] * 2, "o": self.per["o"] * 2, "mid": self.per["mid"] * 2,
                 "dn": self.per["down"] * 2, "pair": 16}
        off, cur = {}, 256                                # [0,256): flag array (world x uint32)
        for k, b in slots.items():
            off[k] = cur
            cur += (b * world + 255) // 256 * 256
        t = symm.empty(cur, dtype=torch.uint8, device=dev)
        t.zero_()
        h = symm.rendezvous(t, self.dist.group.WORLD)
        ptrs = [int(p) for p in h.buffer_ptrs]
        self.sym = t
        i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)
        self.peer = {"slots": slots, "flags": i64(ptrs), "my_flags": t[:256].view(torch.int32),
                     "bufs": {k: i64([p + off[k] for p in ptrs]) for k in slots},
                     "epoch": torch.zeros(1, dtype=torch.int32, device=dev),
                     "status": torch.zeros(1, dtype=torch.int32, device=dev)}
        view = lambda k, n: t[off[k]:off[k] + slots[k] * world].view(torch.int16).view(world, 1, n)
        self.qkv, self.o = view("qkv", self.per["qkv"]), view("o", self.per["o"])
        self.mid, self.dn = view("mid", self.per["mid"]), view("dn", self.per["down"])
        self.pair = t[off["pair"]:off["pair"] + 16 * world].view(torch.float32).view(world, 4)
        self.pair_shard = torch.zeros(4, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        self.dist.barrier()

    def peer_gather(self, key, shard):
        pr = self.peer
        nbytes = shard.numel() * shard.element_size()
        self.pkg.peer_allgather(shard, nbytes, pr["slots"][key], pr["bufs"][key], pr["flags"], pr["my_flags"],
                                pr["epoch"], self.rank, self.world, status=pr["status"], pdl=True)
        self.extra_launches += 1

    def gather(self, full, shard, key=None):
        if self.world > 1 and self.peer is not None and key is not None:
            self.peer_gather(key, shard)
            return full.view(-1)
        if self.world > 1:
            # NCCL has no 16-bit integer type: the same bits travel as bf16
            self.dist.all_gather_into_tensor(full.view(-1).view(self.torch.bfloat16), shard.view(-1).view(self.torch.bfloat16))
            return full.view(-1)
        return shard.view(-1)

    def step_batched(self, pdl=True):
        """M > 1: the reference's BatchGroup sequence (native/runtime/batch_group.cpp:745-807):
        separate residual+RMSNorm kernels between the batched GEMMs."""
        p, fp8, m = self.pkg, self.fp8, self.m
        res = self.res[0]
        res.copy_(self.x_in)
        addend, n = None, 0

        def linear(ws, x, y, N, K):
            w, s = ws
            if fp8:
                p.launch_gemv_fp8_rows_m(w, s, x, y, m, N, K, pdl=pdl)
            else:
                p.gemm_bf16(None, None, 0, m, N, K, w, x, y)

        for lay in self.layers:
            p.launch_residual_rmsnorm_rows(res, addend, lay["n1"], self.h, m, H, 1e-6, pdl=pdl)
            linear(lay["qkv"], self.h, self.qkv_m, QKV, H)
            self.ctx.copy_(self.qkv_m[:, :H])            # stand-in for attention (not a kernel of this library)
            linear(lay["o"], self.ctx, self.o_m, H, H)
            p.launch_residual_rmsnorm_rows(res, self.o_m, lay["n2"], self.h, m, H, 1e-6, pdl=pdl)
            w, s = lay["gu"]
            p.launch_gate_up_swiglu(w, s, self.h, self.mid_m, m, 2 * I, H, pdl=pdl)
            linear(lay["down"], self.mid_m, self.dn_m, H, I)
            addend = self.dn_m
            n += 6
        p.launch_residual_rmsnorm_rows(res, addend, self.nf, self.h, m, H, 1e-6, pdl=pdl)
        w, s = self.lm
        if m <= 8:
            p.launch_lm_head_argmax(w, s, self.h, self.logits, V, m, V, H, 0, self.stage, self.tok, self.val, pdl=pdl)
        else:
            linear(self.lm, self.h, self.logits, V, H)
            p.launch_argmax_bf16(self.logits, m, V, V, 0, self.stage, self.tok, self.val, pdl=pdl)
        self.launches = n + 4
        return self.tok

    def step_stack(self):
        """One GPU: the whole step through the C ABI's decode-stack object."""
        m = self.m
        self.pkg.stack_step(self.handle, self.x_in, m, self.tok)
        self.launches = (1 if (m == 1 and self.world == 1 and CHAIN[0]) else (4 * L + 2 + (1 if self.world > 1 else 0)) if m == 1
                         else (6 * L + 1 + (2 if m <= 4 else 3) + ((4 * L + 1) if self.world > 1 else 0)))
        return self.tok

    def step(self, pdl=True):
        if self.handle is not None:
            return self.step_stack()
        if self.m != 1:
            return self.step_batched(pdl)
        p, fp8 = self.pkg, self.fp8
        self.extra_launches = 0
        ra, rb = self.res                    # residual ping-pong: qkv reads ra -> writes rb, gate_up reads rb -> writes ra
        addend = None
        x_res = self.x_in
        n = 0
        for lay in self.layers:
            w, s = lay["qkv"]
            (p.launch_gemv_fp8_prologue(w, s, x_res, addend, lay["n1"], rb, self.qkv_s, w.shape[0], H, 1e-6, pdl=pdl) if fp8
             else p.launch_gemv_rows_prologue(w, x_res, addend, lay["n1"], rb, self.qkv_s, w.shape[0], H, 1e-6, pdl=pdl))
            qkv = self.gather(self.qkv, self.qkv_s, "qkv")
            w, s = lay["o"]
            (p.launch_gemv_fp8(w, s, qkv, self.o_s, w.shape[0], H, pdl=pdl) if fp8
             else p.launch_decode_gemv(w, qkv, self.o_s, w.shape[0], H, pdl=pdl))
            o = self.gather(self.o, self.o_s, "o")
            w, s = lay["gu"]
            p.launch_gate_up_swiglu_prologue(w, s, rb, o, lay["n2"], ra, self.mid_s, w.shape[0], H, 1e-6, pdl=pdl)
            mid = self.gather(self.mid, self.mid_s, "mid")
            w, s = lay["down"]
            (p.launch_gemv_fp8(w, s, mid, self.dn_s, w.shape[0], I, pdl=pdl) if fp8
             else p.launch_decode_gemv(w, mid, self.dn_s, w.shape[0], I, pdl=pdl))
            addend = self.gather(self.dn, self.dn_s, "dn")
            x_res = ra
            n += 4
        a = rb
        w, s = self.lm
        p.launch_lm_head_argmax_prologue(w, s, x_res, addend, self.nf, a, self.logits, self.v_rows, H, 1e-6,
                                         self.v_lo, self.stage, self.tok, self.val, pdl=pdl)
        n += 2
        if self.world > 1:
            # (value, index) of every shard to every rank, then the same tie rule
            if self.peer is not None:
                self.pair_shard[0:1].copy_(self.val)
                self.pair_shard[1:2].copy_(self.tok.to(self.torch.float32))
                self.peer_gather("pair", self.pair_shard)
            else:
                mine = self.torch.stack((self.val, self.tok.to(self.torch.float32)), dim=1)
                self.dist.all_gather_into_tensor(self.pair.view(-1), mine.view(-1))
        n += self.extra_launches
        self.launches = n
        return self.tok


class Single:
    """One linear of the stream in isolation: `copies` distinct weight copies
    (more than twice the L2 size in total) are visited round-robin so that every
    call streams its weights from HBM; one step = one visit of every copy."""

    SHAPES = {"qkv": (QKV, H, 0), "o": (H, H, 0), "gate_up": (2 * I, H, 1), "down": (H, I, 0), "lm_head": (V, H, 2)}

    def __init__(self, pkg, torch, name, dtype, m, l2_bytes):
        self.pkg, self.m, self.name = pkg, m, name
        n, k, kind = self.SHAPES[name]
        self.n, self.k, self.kind, self.fp8 = n, k, kind, dtype == "fp8"
        wb = 1 if self.fp8 else 2
        per = n * k * wb
        self.copies = int(max(2, min(64, (2 * l2_bytes + per - 1) // per + 1)))
        g = torch.Generator(device="cuda"); g.manual_seed(7)
        self.w, self.s = [], []
        for _ in range(self.copies):
            w = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            if self.fp8:
                w32 = w.to(torch.float32)
                sc = (w32.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
                self.w.append((w32 / sc[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).contiguous())
                self.s.append(sc.contiguous())
            else:
                self.w.append(w.view(torch.int16).contiguous()); self.s.append(None)
        self.x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16).view(torch.int16)
        n_out = n // 2 if kind == 1 else n
        self.n_out = n_out
        self.y = torch.zeros((m, n_out), dtype=torch.int16, device="cuda")
        self.stage = torch.empty(pkg.argmax_stage_bytes(max(m, 1)), dtype=torch.uint8, device="cuda")
        self.tok = torch.zeros(m, dtype=torch.int32, device="cuda")
        self.ws_bytes = pkg.gemm_workspace_bytes(m, n, k)
        self.ws = torch.empty(max(self.ws_bytes, 16), dtype=torch.uint8, device="cuda")
        self.launches = 0
        self.w8a8 = os.environ.get("MC_W8A8", "0") == "1"      # e4m3, M > 1: quantised activations instead of weight-only
        self.xq = torch.empty((m, k), dtype=torch.uint8, device="cuda")
        self.xs = torch.empty(m, dtype=torch.float32, device="cuda")
        self.bytes_per_call = linear_bytes(n, k, m, wb, n_out)
        self.hints = os.environ.get("MC_HINTS", "1") == "1"     # each call names the next copy's weights (L2 prefetch)

    def call(self, i, pdl=True):
        """The linear on weight copy i; tells the kernel which copy comes next (L2 prefetch)."""
        p, m, n, k = self.pkg, self.m, self.n, self.k
        w, s = self.w[i], self.s[i]
        if self.hints:
            p.hint_next_weights(self.w[(i + 1) % self.copies])
        if self.kind == 1:
            p.launch_gate_up_swiglu(w, s, self.x, self.y, m, n, k, pdl=pdl)
        elif self.kind == 2 and m <= 8:
            p.launch_lm_head_argmax(w, s, self.x, self.y, n, m, n, k, 0, self.stage, self.tok, None, pdl=pdl)
        elif self.fp8 and self.w8a8 and m > 1:
            # the reference's batched e4m3 path: per-row activation quantiser + W8A8 GEMM (tcgen05 kind::f8f6f4)
            p.gemm_fp8(None, self.ws, self.ws_bytes, m, n, k, w, s, self.x, self.y, self.xq, self.xs)
        elif self.fp8:
            (p.launch_gemv_fp8(w, s, self.x, self.y, n, k, pdl=pdl) if m == 1
             else p.launch_gemv_fp8_rows_m(w, s, self.x, self.y, m, n, k, pdl=pdl))
        else:
            (p.launch_decode_gemv(w, self.x, self.y, n, k, pdl=pdl) if m == 1
             else p.gemm_bf16(None, self.ws, self.ws_bytes, m, n, k, w, self.x, self.y))

    def step(self, pdl=True):
        for i in range(self.copies):
            self.call(i, pdl)
        self.launches = self.copies * (2 if self.kind == 2 or (self.fp8 and self.w8a8 and self.m > 1) else 1)
        return self.tok

    def check(self, torch):
        """One call on copy 0 against a plain fp32 PyTorch statement of the same linear (relative L2 error
        and largest relative error over elements that are not tiny); returns the figures, raises on a miss."""
        self.call(0, pdl=False)
        torch.cuda.synchronize()
        x = self.x.view(torch.bfloat16).to(torch.float32)
        if self.fp8 and self.w8a8 and self.m > 1:
            # W8A8: the statement quantises the activation rows the way the library does (scale = max|row| / 448, e4m3)
            sc = (x.abs().amax(dim=1, keepdim=True) / 448.0).clamp_min(1e-30)
            x = (x / sc).to(torch.float8_e4m3fn).to(torch.float32) * sc
        if self.fp8:
            ref = (x @ self.w[0].view(torch.float8_e4m3fn).to(torch.float32).T) * self.s[0][None, :]
        else:
            ref = x @ self.w[0].view(torch.bfloat16).to(torch.float32).T
        if self.kind == 1:
            rb = ref.to(torch.bfloat16).to(torch.float32)
            g, u = rb[:, 0::2], rb[:, 1::2]
            ref = g / (1.0 + torch.exp(-g)) * u
        got = self.y.view(torch.bfloat16).to(torch.float32)
        d = (got - ref).double()
        rel = float(torch.sqrt((d * d).sum() / (ref.double() ** 2).sum()))
        rms = float(torch.sqrt((ref.double() ** 2).mean()))
        big = ref.abs() >= rms * 2.0 ** -7
        # half a bf16 unit of rounding on either side is 2^-8; a SwiGLU output carries its inputs' rounding too
        max_rel = float((d.abs()[big] / ref.abs().double()[big]).max())
        tol = 2e-2 if self.kind == 1 else 1e-2
        if not (rel <= 1e-2 and max_rel <= tol):
            raise SystemExit(f"bench: {self.name} {'fp8' if self.fp8 else 'bf16'} M={self.m} differs from the fp32 statement: "
                             f"relL2={rel:.3e} max_rel={max_rel:.3e}")
        if self.kind == 2 and self.m <= 8:
            want = got.argmax(dim=1).to(torch.int32)
            vals = got.gather(1, self.tok.long()[:, None])[:, 0]
            if not bool(((self.tok == want) | (vals == got.max(dim=1).values)).all()):
                raise SystemExit(f"bench: lm_head argmax M={self.m} is not the maximum of its own logits")
        return {"rel_l2": rel, "max_rel": max_rel}


CHAIN = [False]       # whether M = 1 steps of a one-GPU stack run as one persistent kernel (library default: no)


def set_chain(pkg, on):
    pkg.debug_set_chain(on)
    CHAIN[0] = bool(on)


def apply_prefetch_env(pkg):
    """MC_PREFETCH="mode[,chunk[,evict_first[,cap_mb]]]" overrides the library's L2-prefetch defaults (A/B runs)."""
    if os.environ.get("MC_MMA_ROWS") is not None:    # MC_MMA_ROWS=0: bf16 batched linears on the tcgen05 kernel only
        pkg.debug_set_mma_rows(int(os.environ["MC_MMA_ROWS"]))
    if os.environ.get("MC_CHAIN") is not None:       # MC_CHAIN=0: one kernel per linear instead of the one-launch M = 1 chain
        set_chain(pkg, os.environ["MC_CHAIN"] != "0")
    v = os.environ.get("MC_PREFETCH")
    if not v:
        return "default"
    f = [int(x) for x in v.split(",")] + [-1, -1, 0]
    pkg.debug_set_prefetch(mode=f[0], chunk_bytes=f[1], evict_first=f[2], cap_bytes=(f[3] << 20) if f[3] > 0 else 0)
    return v


def time_graph(torch, stream, st, steps, warmup, use_graph=True, barrier=None):
    """Captures one step of `st`, replays it warmup + steps times; returns (ms for `steps` steps, launch mode, run)."""
    barrier = barrier or torch.cuda.synchronize
    graph, mode = None, "eager+pdl"
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                st.step()
            mode = "cuda-graph+pdl"
        except Exception as e:                      # capture not possible: same kernels, eager launches
            graph, mode = None, f"eager+pdl (graph capture failed: {type(e).__name__})"
            torch.cuda.synchronize()
    run = (lambda: graph.replay()) if graph is not None else (lambda: st.step())
    barrier()
    for _ in range(max(warmup, 3)):
        run()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record(stream)
    for _ in range(steps):
        run()
    ev1.record(stream)
    barrier()
    return ev0.elapsed_time(ev1), mode, run, (t0, time.time())


# DRAM bytes per launch over algorithmic bytes, from the ncu captures summarised under profiles/ (read + write,
# one launch, cold L2).  A shape without a capture reports "modelled" with the family's ratio.
TRAFFIC = {
    # (kernel family, workload, dtype): (DRAM bytes / algorithmic bytes, source)
    ("gemv_fast_kernel", "qkv", "bf16"): (1.0006, "profiles/gemv_fast_bf16_qkv_3456x2304.md"),
    ("gemv_fast_kernel", "o", "bf16"): (1.0011, "profiles/gemv_fast_bf16_o_2304x2304.md"),
    ("gemv_fast_kernel", "gate_up", "bf16"): (1.0002, "profiles/gemv_fast_bf16_gate_up_11520x2304.md"),
    ("gemv_fast_kernel", "down", "bf16"): (1.0007, "profiles/gemv_fast_bf16_down_2304x5760.md"),
    ("gemv_fast_kernel", "gate_up", "fp8"): (1.0006, "profiles/gemv_fast_fp8_gate_up_11520x2304.md"),
    ("gemv_fast_kernel", "lm_head", "bf16"): (1.0079, "profiles/gemv_fast_bf16_lm_head_122753x2304.md"),
    ("gemv_fast_kernel", "lm_head", "fp8"): (1.0158, "profiles/gemv_fast_fp8_lm_head_122753x2304.md"),
    ("skinny_gemm_kernel", "down", "bf16"): (0.9996, "profiles/skinny_gemm_bf16_down_m16_2304x5760.md (M = 16; M = 64: 0.9916)"),
    ("skinny_gemm_kernel", "down", "fp8"): (1.0025, "profiles/skinny_gemm_fp8_weight_only_down_m8_2304x5760.md (M = 8)"),
    ("gemm_mma_rows_kernel", "down", "bf16"): (1.0008, "profiles/gemm_mma_rows_bf16_down_m8_2304x5760.md (M = 8)"),
    ("skinny_gemm_kernel", "down", "fp8_w8a8"): (1.0019, "profiles/skinny_gemm_w8a8_down_m8_2304x5760.md (M = 8; the GEMM launch, its activation already quantised)"),
    ("decode_chain_kernel", "stream", "bf16"): (1.0048, "profiles/decode_chain_persistent_kernel_bf16_fp8_m1.md (4 layers + lm_head captured, scaled by bytes)"),
    # the whole bf16 M = 1 step: byte-weighted mean of its five kernels' ratios
    ("gemv_fast_kernel", "stream", "bf16"): (1.0013, "byte-weighted over profiles/gemv_fast_bf16_{qkv,o,gate_up,down,lm_head}_*.md"),
}


def traffic_for(kernel, workload, dtype, algorithmic_bytes):
    if dtype == "fp8" and kernel == "skinny_gemm_kernel" and os.environ.get("MC_W8A8", "0") == "1":
        dtype = "fp8_w8a8"
    hit = TRAFFIC.get((kernel, workload, dtype))
    if hit is not None:
        return algorithmic_bytes * hit[0], f"ncu dram__bytes_read.sum + dram__bytes_write.sum, {hit[1]}"
    return None, "no ncu capture of this kernel and shape"


def kernel_name(workload, dtype, m):
    if m == 1 and workload == "stream" and CHAIN[0]:
        return "decode_chain_kernel"
    if m == 1:
        return "gemv_fast_kernel"
    if dtype == "fp8" and m <= 3:
        return "gemv_rows_kernel"
    if (dtype == "bf16" and 2 <= m <= 8 and workload in Single.SHAPES and Single.SHAPES[workload][2] == 0
            and Single.SHAPES[workload][0] <= 16 * 148 and os.environ.get("MC_MMA_ROWS", "8") != "0"):
        return "gemm_mma_rows_kernel"       # a weight of at most 16 rows per SM: the register-streaming mma.sync kernel
    return "skinny_gemm_kernel"


def run_configs(pkg, torch, info, stream, peak, steps=12):
    """The single-linear configurations: qkv bf16 M=1; gate_up + SwiGLU e4m3 M=1; down_proj bf16 and e4m3 for
    M in {1..64}; lm_head bf16 M in {1, 8}.  Each entry: us per call, GB/s, fraction of the measured copy peak
    and of 8 TB/s, kernel, and the parity of one call against the fp32 PyTorch statement."""
    plan = [("config1", "qkv", "bf16", 1), ("config2", "gate_up", "fp8", 1)]
    plan += [("config3", "down", d, m) for d in ("bf16", "fp8") for m in (1, 2, 4, 8, 16, 32, 64)]
    plan += [("config4", "lm_head", "bf16", 1), ("config4", "lm_head", "bf16", 8), ("config4", "lm_head", "fp8", 1)]
    plan += [("layer", "o", "bf16", 1), ("layer", "gate_up", "bf16", 1), ("layer", "qkv", "fp8", 1), ("layer", "o", "fp8", 1),
             ("layer", "gate_up", "bf16", 8), ("layer", "gate_up", "fp8", 8)]
    out = []
    for cfg, name, dtype, m in plan:
        sg = Single(pkg, torch, name, dtype, m, info["l2_bytes"])
        par = sg.check(torch)
        sg.step()
        stream.synchronize()
        ms, mode, run, _ = time_graph(torch, stream, sg, steps, 3)
        us = ms * 1e3 / (steps * sg.copies)
        gbs = sg.bytes_per_call / (us * 1e-6) / 1e9
        kern = kernel_name(name, dtype, m)
        traffic, src = traffic_for(kern, name, dtype, sg.bytes_per_call)
        out.append({"config": cfg, "linear": name, "N": sg.n, "K": sg.k, "dtype": dtype, "M": m, "us_per_call": us, "GBps": gbs,
                    "frac_of_measured": gbs / peak, "frac_of_8TBs": gbs / NOMINAL_HBM_GBS, "kernel": kern,
                    "bytes_per_call": sg.bytes_per_call, "weight_copies": sg.copies, "launch": mode,
                    "next_weights_hint": sg.hints, "parity_checked": "fp32 statement", "rel_l2": par["rel_l2"],
                    "max_rel": par["max_rel"], "traffic": traffic, "traffic_source": src})
        del sg, run
        torch.cuda.empty_cache()
    return out


def run_stream_configs(pkg, torch, args, stream, peak, steps=20):
    """The other whole-step streams next to the headline: e4m3 and bf16, M = 1 and M = 8, each checked like the
    headline before it is timed, and the M = 1 step as ONE persistent kernel (the library's alternative launch form,
    off by default).  One entry each: ms per step, GB/s, fraction of the measured copy peak."""
    import copy
    plan = [("bf16", 1, False), ("fp8", 1, False), ("bf16", 8, False), ("fp8", 8, False), ("bf16", 1, True), ("fp8", 1, True)]
    out = []
    for dtype, m, chain in plan:
        if (dtype, m, chain) == (args.dtype, args.m, False):
            continue                                  # the headline itself
        a = copy.copy(args)
        a.dtype, a.m = dtype, m
        set_chain(pkg, chain)
        try:
            st = Stream(pkg, torch, dtype, m, 1, 0, None)
            st.step()
            stream.synchronize()
            tok, logits = st.tok.clone(), st.logits_view().clone()
            par = check_stream(pkg, torch, st, a, 1, 0, stream, tok, logits)
            ms, mode, run, _ = time_graph(torch, stream, st, steps, 3)
            stream.synchronize()
            if not torch.equal(st.tok, tok) or not torch.equal(st.logits_view(), logits):
                raise SystemExit(f"bench: {dtype} M={m} stream: graph replay differs from the eager step")
            if pkg.stack_exchange_status(st.handle, stream) != 0:
                raise SystemExit(f"bench: {dtype} M={m} stream: a bounded wait ran out")
            nbytes = stream_bytes(m, 2 if dtype == "bf16" else 1, 1, 0)
            gbs = nbytes / (ms / steps * 1e-3) / 1e9
            out.append({"config": "config5", "stream": f"40 layers + lm_head, {dtype}, M={m}", "dtype": dtype, "M": m,
                        "launch_form": "one persistent kernel per step" if chain else "one kernel per linear",
                        "ms_per_step": ms / steps, "GBps": gbs, "frac_of_measured": gbs / peak, "frac_of_8TBs": gbs / NOMINAL_HBM_GBS,
                        "launch": mode, "tokens_per_s": m * 1e3 / (ms / steps), "parity_checked": "fp32 statement + graph replay",
                        "rel_l2": par.get("rel_l2_vs_fp32_statement"), "cosine": par.get("cosine")})
            pkg.stack_destroy(st.handle)
            del st, run
            torch.cuda.empty_cache()
        finally:
            set_chain(pkg, False)
    return out


def check_stream(pkg, torch, st, args, world, rank, stream, tok_eager, logits_eager):
    """What the timed graph computes, against (a) the eager step, (b) at one GPU the fp32 PyTorch statement of
    the chain, (c) at N > 1 the one-GPU stack built on rank 0 from the same seeds.  Returns the figures."""
    res = {}
    if world == 1:
        ref = st.reference_logits(st.x_in)
        got = logits_eager.view(torch.bfloat16).to(torch.float32)
        d = (got - ref).double()
        rel = float(torch.sqrt((d * d).sum() / (ref.double() ** 2).sum()))
        cos = float((got.double() * ref.double()).sum() / torch.sqrt((got.double() ** 2).sum() * (ref.double() ** 2).sum()))
        res.update(rel_l2_vs_fp32_statement=rel, cosine=cos)
        # 40 layers of bf16-rounded intermediates: last-bit differences upstream move the logits a little
        if not (rel < 5e-2 and cos > 0.999):
            raise SystemExit(f"bench: logits differ from the fp32 statement of the chain: relL2={rel:.3e} cos={cos:.6f}")
        top2 = ref.topk(2, dim=1).values
        clear = (top2[:, 0] - top2[:, 1]) > 0.05
        want = ref.argmax(dim=1).to(torch.int32)
        if not bool(((tok_eager == want) | ~clear).all()):
            raise SystemExit(f"bench: token {tok_eager.tolist()} differs from the fp32 statement's {want.tolist()}")
        own = got.argmax(dim=1).to(torch.int32)
        if not bool(((tok_eager == own) | (got.gather(1, tok_eager.long()[:, None])[:, 0] == got.max(dim=1).values)).all()):
            raise SystemExit("bench: the token is not the maximum of the step's own logits")
        res["tokens"] = tok_eager.tolist()
    elif rank == 0:
        one = Stream(pkg, torch, args.dtype, args.m, 1, 0, None)
        one.x_in.copy_(st.x_in)
        one.step()
        stream.synchronize()
        full = one.logits_view()
        mine = full[:, st.v_lo:st.v_lo + st.v_rows]
        same_tok = bool(torch.equal(one.tok, tok_eager))
        if args.m == 1:
            same = bool(torch.equal(mine, logits_eager))          # a row's arithmetic does not depend on the sharding
            res.update(one_gpu_token_equal=same_tok, one_gpu_logits_shard_equal=same, tokens=tok_eager.tolist())
        else:
            # batched: a shard of N / world rows is cut into other K splits than the whole matrix, so sums run in another
            # order and 40 layers of bf16-rounded intermediates drift a little apart: tolerance of the fp32-statement check,
            # token equality wherever the one-GPU run's two best logits are clearly apart
            a, b = mine.view(torch.bfloat16).float(), logits_eager.view(torch.bfloat16).float()
            rel = float(torch.sqrt(((a - b) ** 2).sum() / (a ** 2).sum()))
            top2 = full.view(torch.bfloat16).float().topk(2, dim=1).values
            clear = (top2[:, 0] - top2[:, 1]) > 0.05
            same_tok = bool(((one.tok == tok_eager) | ~clear).all())
            same = rel < 5e-2
            res.update(one_gpu_token_equal_where_clear=same_tok, rel_l2_vs_one_gpu_logits_shard=rel, tokens=tok_eager.tolist())
        if not (same_tok and same):
            raise SystemExit(f"bench: sharded run differs from the one-GPU stack (token equal: {same_tok}, logits shard equal: {same})")
        pkg.stack_destroy(one.handle)
        del one
        torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    pkg = importlib.import_module("minicpm5-5080fast_b200")
    pkg.lib()          # fails loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    info = pkg.device_check()
    prefetch = apply_prefetch_env(pkg)
    wb = 2 if args.dtype == "bf16" else 1
    single = args.workload != "stream"
    if single and world > 1:
        raise SystemExit("bench: single-linear workloads run on one GPU")
    st = (Single(pkg, torch, args.workload, args.dtype, args.m, info["l2_bytes"]) if single
          else Stream(pkg, torch, args.dtype, args.m, world, rank, dist))
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    parity = {}
    with torch.cuda.stream(stream), ClockSampler(local) as clk:
        if single:
            parity = st.check(torch)
        barrier()                                   # sharded kernels wait (bounded) for their peers: start together
        st.step()                                   # eager once: sets attributes
        stream.synchronize()
        if not single:
            tok_eager = st.tok.clone()
            logits_eager = st.logits_view().clone()
            parity = check_stream(pkg, torch, st, args, world, rank, stream, tok_eager, logits_eager)
        ms, mode, run, (t_wall0, t_wall1) = time_graph(torch, stream, st, args.steps, args.warmup, bool(args.graph), barrier)
        clk.window(t_wall0, t_wall1)
        if not single:
            # the last timed replay computed the same step as the eager one
            stream.synchronize()
            if not torch.equal(st.tok, tok_eager) or not torch.equal(st.logits_view(), logits_eager):
                raise SystemExit(f"bench: graph replay differs from the eager step (tokens {st.tok.tolist()} vs {tok_eager.tolist()})")
            parity["graph_replay_equals_eager"] = True
        # ---- end to end: host input -> device -> linears -> result back on the host, every step
        x_dev = st.x if single else st.x_in
        res_dev = st.y if single else st.tok
        hx = x_dev.cpu().pin_memory()
        hres = torch.zeros(tuple(res_dev.shape), dtype=res_dev.dtype).pin_memory()
        if not single and st.handle is not None:
            # the user-facing call: host activations in, host tokens out, one C-ABI call per step
            def e2e_step():
                pkg.stack_step_host(st.handle, hx, args.m, hres, stream)
        else:
            def e2e_step():
                x_dev.copy_(hx, non_blocking=True)
                run()
                hres.copy_(res_dev, non_blocking=True)
                stream.synchronize()
        barrier()
        for _ in range(3):
            e2e_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        if not single and st.handle is not None:
            if not torch.equal(hres, tok_eager.cpu()):
                raise SystemExit(f"bench: the host-buffer step returned {hres.tolist()}, the eager step {tok_eager.tolist()}")
            parity["host_step_equals_eager"] = True

    if getattr(st, "peer", None) is not None and int(st.peer["status"].item()) != 0:
        raise SystemExit("bench: a bounded wait of the peer all-gather kernel ran out (a rank fell behind or died)")
    if not single and st.handle is not None and pkg.stack_exchange_status(st.handle, stream) != 0:
        raise SystemExit("bench: a bounded wait ran out inside a kernel of the stack (a rank fell behind or died, or a pipeline stalled)")
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    if single:
        total_bytes = st.bytes_per_call * st.copies
    else:
        total_bytes = sum(stream_bytes(args.m, wb, world, r) for r in range(world))
    per_step_ms = ms / args.steps
    value = total_bytes / (per_step_ms * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = value / world
    if rank == 0:
        configs = None
        if world == 1 and not single and args.configs:
            with torch.cuda.stream(stream):
                configs = run_configs(pkg, torch, info, stream, peak)
                if L == 40:
                    configs += run_stream_configs(pkg, torch, args, stream, peak)
        cpu = cpu_reference(args.dtype, args.m, budget_s=10.0) if world == 1 and not args.no_cpu else None
        kern = kernel_name(args.workload, args.dtype, args.m)
        per_launch_bytes = (total_bytes / world) / (1 if not single else st.copies)
        traffic, traffic_src = traffic_for(kern, args.workload, args.dtype, per_launch_bytes)
        line = {
            "metric": "decode_linear_hbm_throughput", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if wb == 2 else "fp8_e4m3_weight_only(fp32 acc)",
            "data": "synthetic", "parity_checked": True, "parity": parity,
            "config": {"workload": workload_name(args), "launch": mode, "parallelism": f"N-sharded x{world}",
                       "gather": (None if world == 1 else
                                  "inside the GEMV kernels: every output word stored to all peers over NVLink with its sequence tag (symmetric memory)" if st.handle is not None else
                                  "peer-store kernel over NVLink (symmetric memory)" if getattr(st, "peer", None) else
                                  "nccl all_gather" + (" (" + getattr(st, "peer_error", "") + ")" if getattr(st, "peer_error", "") else "")),
                       "l2": ("every call reads a different weight copy; the copies together exceed twice the L2" if single
                              else "inputs larger than L2: every step streams its own weights from HBM once"),
                       "l2_prefetch": prefetch,
                       "bytes_per_step": total_bytes, "calls_per_step": st.launches if not single else st.copies,
                       "us_per_call": per_step_ms * 1e3 / (st.copies if single else st.launches),
                       "tokens_per_s": None if single else args.m * 1e3 / per_step_ms},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(hx.numel() * 2),
                    "d2h_bytes_per_step": int(hres.numel() * hres.element_size()), "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": st.launches * args.steps,
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_kind": f"{peak_kind} copy bandwidth", "frac_of_nominal_8TBs": per_gpu / NOMINAL_HBM_GBS,
                         "kernel": kern + (" (one launch per call)" if single else " (whole step: every launch of the chain)"),
                         "traffic": traffic, "traffic_source": traffic_src},
        }
        if configs is not None:
            line["configs"] = configs
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample") if k in cpu}
            for k in ("cpu_model", "numpy"):
                if k in cpu:
                    line["cpu_baseline"][k] = cpu[k]
        print(json.dumps(line), flush=True)
    if dist is not None:
        # leave without the communicator teardown (it can block behind captured work on this stack)
        del run
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


def run_ref_gpu(args):
    """Comparison arm on the same GPU: per shape and M, this library against (i) the reference's own GEMV kernels
    (native/kernels/sm120/gemv.cu, gemv_fp8.cu) compiled unmodified for sm_100a and (ii) the cuBLASLt call of its
    batched path (native/runtime/gemm.cpp:67-128), all three with the same rotation of weight copies and the same
    graph replay.  Needs oracle/_ref/libref_gpu.so (oracle/Makefile, target ref_gpu); prints one JSON line."""
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
    if not os.path.exists(so):
        print(json.dumps({"impl": "ref_gpu", "unavailable": "oracle/_ref/libref_gpu.so has not been built (make -C oracle ref_gpu needs the reference tree)"}))
        return
    pkg = importlib.import_module("minicpm5-5080fast_b200")
    pkg.lib()
    ref = ctypes.CDLL(so)
    vp, u32 = ctypes.c_void_p, ctypes.c_uint32
    ref.ref_gpu_last_error.restype = ctypes.c_char_p
    ref.ref_gpu_decode_gemv.argtypes = [vp, vp, vp, u32, u32, vp, ctypes.c_int]
    ref.ref_gpu_gemv_fp8.argtypes = [vp, vp, vp, vp, u32, u32, vp, ctypes.c_int]
    ref.ref_gpu_gemv_fp8_rows_m.argtypes = [vp, vp, vp, vp, u32, u32, u32, vp, ctypes.c_int]
    ref.ref_cublaslt_gemm_bf16.argtypes = [vp, vp, ctypes.c_size_t, u32, u32, u32, vp, vp, vp]
    torch.cuda.set_device(0)
    info = pkg.device_check()
    peak, _ = measured_peak()
    stream = torch.cuda.Stream()
    ws = torch.empty(16 << 20, dtype=torch.uint8, device="cuda")      # the reference's 16 MB GEMM workspace
    plan = [("config1", "qkv", "bf16", 1), ("layer", "o", "bf16", 1), ("layer", "gate_up_plain", "bf16", 1), ("config2", "gate_up_plain", "fp8", 1)]
    plan += [("config3", "down", d, m) for d in ("bf16", "fp8") for m in (1, 2, 4, 8, 16, 32, 64)]
    plan += [("config4", "lm_head_plain", "bf16", 1), ("config4", "lm_head_plain", "bf16", 8)]
    Single.SHAPES["gate_up_plain"] = (2 * I, H, 0)          # the reference has no SwiGLU epilogue: plain [2I] output on both sides
    Single.SHAPES["lm_head_plain"] = (V, H, 0)
    rows = []

    class Arm:
        def __init__(self, sg, call):
            self.sg, self.call, self.copies = sg, call, sg.copies

        def step(self):
            for i in range(self.copies):
                self.call(i)

    with torch.cuda.stream(stream):
        sp = stream.cuda_stream
        for cfg, name, dtype, m in plan:
            sg = Single(pkg, torch, name, dtype, m, info["l2_bytes"])
            sg.hints = False
            y_ref = torch.zeros_like(sg.y)
            arms = {"ours": Arm(sg, lambda i: sg.call(i))}
            if dtype == "bf16":
                arms["cublaslt"] = Arm(sg, lambda i: _ck(ref.ref_cublaslt_gemm_bf16(sp, ws.data_ptr(), ws.numel(), m, sg.n, sg.k, sg.w[i].data_ptr(),
                                                                                   sg.x.data_ptr(), y_ref.data_ptr()), "cublasLt"))
                if m == 1:
                    arms["ref_simt_sm100a"] = Arm(sg, lambda i: _ck(ref.ref_gpu_decode_gemv(sg.w[i].data_ptr(), sg.x.data_ptr(), y_ref.data_ptr(), sg.n,
                                                                                           sg.k, sp, 1), ref.ref_gpu_last_error()))
            elif m == 1:
                arms["ref_simt_sm100a"] = Arm(sg, lambda i: _ck(ref.ref_gpu_gemv_fp8(sg.w[i].data_ptr(), sg.s[i].data_ptr(), sg.x.data_ptr(), y_ref.data_ptr(),
                                                                                    sg.n, sg.k, sp, 1), ref.ref_gpu_last_error()))
            elif m <= 8:
                arms["ref_simt_sm100a"] = Arm(sg, lambda i: _ck(ref.ref_gpu_gemv_fp8_rows_m(sg.w[i].data_ptr(), sg.s[i].data_ptr(), sg.x.data_ptr(),
                                                                                           y_ref.data_ptr(), m, sg.n, sg.k, sp, 1), ref.ref_gpu_last_error()))
            entry = {"config": cfg, "linear": name.replace("_plain", ""), "N": sg.n, "K": sg.k, "dtype": dtype, "M": m,
                     "bytes_per_call": sg.bytes_per_call, "weight_copies": sg.copies}
            for label, arm in arms.items():
                arm.step()
                stream.synchronize()
                if label != "ours":
                    # the comparison arm computes the same linear: its last call (copy n-1) against ours on the same copy
                    sg.call(sg.copies - 1)
                    stream.synchronize()
                    a, b = sg.y.view(torch.bfloat16).float(), y_ref.view(torch.bfloat16).float()
                    entry[label + "_rel_l2_vs_ours"] = float(torch.sqrt(((a - b) ** 2).sum() / (a ** 2).sum()))
                ms, mode, run, _ = time_graph(torch, stream, arm, 12, 3)
                us = ms * 1e3 / (12 * sg.copies)
                entry[label + "_us"] = us
                entry[label + "_GBps"] = sg.bytes_per_call / (us * 1e-6) / 1e9
                del run
            others = [v for k, v in entry.items() if k.endswith("_us") and not k.startswith("ours")]
            entry["ours_vs_best_other"] = min(others) / entry["ours_us"] if others else None   # > 1: this library is faster
            rows.append(entry)
            del sg, arms
            torch.cuda.empty_cache()
    print(json.dumps({"impl": "ref_gpu", "metric": "us per call, same GPU, same rotation and graph replay", "peak_GBps": peak,
                      "arms": {"ours": "this library", "ref_simt_sm100a": "reference gemv.cu / gemv_fp8.cu compiled unmodified for sm_100a",
                               "cublaslt": "cuBLASLt bf16 GEMM as native/runtime/gemm.cpp:67-128 sets it up (16 MB workspace, first heuristic)"},
                      "rows": rows}), flush=True)


def _ck(rc, what):
    if rc != 0:
        raise SystemExit(f"bench: comparison arm call failed ({rc}): {what}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ref_gpu"])
    ap.add_argument("--workload", default="stream", choices=["stream", "qkv", "o", "gate_up", "down", "lm_head"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--m", "--batch", dest="m", type=int, default=1, help="batch rows M (use --batch under torchrun, which claims --m)")
    ap.add_argument("--graph", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline leg")
    ap.add_argument("--configs", type=int, default=1, help="after the stream, measure the single-linear configurations (one GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "ref_gpu":
        run_ref_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
