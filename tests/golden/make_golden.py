"""Generates the golden fixtures in this directory from the reference's own
Python implementation.

Run where the reference tree is available (by default a directory `reference`
beside this repository; override with REF_ROOT):

    python tests/golden/make_golden.py

It imports `tools/minicpm_common.py` and `tools/reference_forward.py` from the
reference where they lie (nothing is copied), feeds them seeded synthetic
inputs, and stores inputs (small cases) or input digests (full-size cases)
together with the reference's outputs.  The fixtures are what pins the CPU
oracle (`oracle/`) to the reference; the GPU tests compare against them too.
"""
from __future__ import annotations

import hashlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("REF_ROOT", os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference")))
sys.path.insert(0, os.path.join(REF_ROOT, "tools"))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))

# reference_forward imports `tokenizers` at module top; it is not needed for
# the numeric functions, so a stub stands in when the package is missing.
try:
    import tokenizers  # noqa: F401
except Exception:  # pragma: no cover
    sys.modules["tokenizers"] = types.SimpleNamespace(Tokenizer=object)

import minicpm_common as rc      # noqa: E402  (reference)
import reference_forward as rf   # noqa: E402  (reference)
import oracle_np as onp          # noqa: E402  (seeding helpers only)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def seed_of(config: int, layer: int, tensor: int) -> int:
    return onp.SEED_BASE + 1000 * config + 10 * layer + tensor


def bf16_normal(seed, shape, std):
    rng = np.random.default_rng(seed)
    return rc.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def codec_fixture():
    rng = np.random.default_rng(7)
    f = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s
                        for s in (1e-3, 0.02, 1.0, 60.0, 500.0)])
    codes = np.arange(256, dtype=np.uint8)
    dec = rc.e4m3_to_f32(codes)
    pos = np.sort(dec[(codes & 0x80) == 0][:-1])
    ties = ((pos[:-1].astype(np.float64) + pos[1:].astype(np.float64)) / 2).astype(np.float32)
    edge = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 448, 449, 464, 465, 480, 1e-9,
                     2.0 ** -6, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10], dtype=np.float32)
    f = np.concatenate([f, ties, -ties, np.nextafter(ties, np.float32(0)),
                        np.nextafter(ties, np.float32(1e9)), edge])
    g = rng.standard_normal(8192).astype(np.float32) * np.float32(3.0)
    w = rng.standard_normal((16, 64)).astype(np.float32) * np.float32(0.02)
    w[3] = 0.0                                     # all-zero row: scale floor
    sc = rc.fp8_row_scales(w)
    np.savez_compressed(
        os.path.join(HERE, "codec.npz"),
        enc_in=f, enc_out=rc.f32_to_e4m3(f), dec_table=dec,
        bf16_in=g, bf16_out=rc.f32_to_bf16(g),
        rows_w=w, rows_scale=sc, rows_q=rc.quantize_fp8_rows(w, sc),
        fnv_foobar=np.uint64(rc.fnv1a64(b"foobar")))


def small_fixture():
    """Small shapes with the inputs stored, so the fixture is self-contained."""
    out = {}
    cases = [("a", 1, 64, 256), ("b", 3, 40, 272), ("c", 1, 17, 100), ("d", 8, 33, 512)]
    for tag, M, N, K in cases:
        w = bf16_normal(100 + len(out), (N, K), 0.02)
        x = bf16_normal(200 + len(out), (M, K), 1.0)
        q, sc = (lambda w32: (rc.quantize_fp8_rows(w32, rc.fp8_row_scales(w32)),
                              rc.fp8_row_scales(w32)))(rc.bf16_to_f32(w))
        xin = x[0] if M == 1 else x
        out[f"{tag}_w"], out[f"{tag}_x"], out[f"{tag}_q"], out[f"{tag}_scale"] = w, x, q, sc
        out[f"{tag}_y_bf16"] = rf.linear_bf16(w, xin).reshape(M, N)
        out[f"{tag}_y_fp8"] = rf.linear_fp8(q, sc, xin).reshape(M, N)
    # elementwise pieces
    g = bf16_normal(301, (2, 96), 2.0)
    u = bf16_normal(302, (2, 96), 1.0)
    out["sw_g"], out["sw_u"], out["sw_out"] = g, u, rf.swiglu_bf16(g, u)
    xr = bf16_normal(303, (2048,), 1.5)
    ad = bf16_normal(304, (2048,), 0.5)
    nw = bf16_normal(305, (2048,), 1.0)
    res = rf.add_bf16(xr, ad)
    out["rn_x"], out["rn_add"], out["rn_w"] = xr, ad, nw
    out["rn_res"], out["rn_out"] = res, rf.rmsnorm_bf16(nw, res)
    lg = bf16_normal(306, (1000,), 4.0)
    lg[[17, 400, 999]] = lg.max()                 # exact three-way tie at the top
    lg[[17, 400, 999]] = rc.f32_to_bf16(np.array([50.0], np.float32))[0]
    out["am_logits"], out["am_idx"] = lg, np.int64(rf.MiniCPM5Ref.greedy(lg))
    np.savez_compressed(os.path.join(HERE, "small.npz"), **out)


def baseline_fixture():
    """Full-size BASELINE shapes: inputs are regenerated from the seeds by the
    tests; the fixture stores digests of the inputs and the reference outputs."""
    K, QKV, I, V = 2304, 3456, 5760, 122753
    out = {}
    # config 1: bf16 fused-qkv GEMV
    w = bf16_normal(seed_of(1, 0, 0), (QKV, K), 0.02)
    x = bf16_normal(seed_of(1, 0, 1), (K,), 1.0)
    out["c1_w_sha"], out["c1_x_sha"] = sha(w), sha(x)
    out["c1_y"] = rf.linear_bf16(w, x)
    # config 2: fp8 gate_up + SwiGLU
    w = bf16_normal(seed_of(2, 0, 0), (2 * I, K), 0.02)
    x = bf16_normal(seed_of(2, 0, 1), (K,), 1.0)
    w32 = rc.bf16_to_f32(w)
    sc = rc.fp8_row_scales(w32)
    q = rc.quantize_fp8_rows(w32, sc)
    y = rf.linear_fp8(q, sc, x)
    out["c2_q_sha"], out["c2_scale_sha"], out["c2_x_sha"] = sha(q), sha(sc), sha(x)
    out["c2_gate_up"] = y
    out["c2_y"] = rf.swiglu_bf16(y[:I], y[I:])
    out["c2_y_bf16w"] = (lambda yy: rf.swiglu_bf16(yy[:I], yy[I:]))(rf.linear_bf16(w, x))
    # config 3: down projection, batched
    w = bf16_normal(seed_of(3, 0, 0), (K, I), 0.02)
    rng = np.random.default_rng(seed_of(3, 0, 1))
    X = rc.f32_to_bf16(rng.standard_normal((64, I), dtype=np.float32) * np.float32(0.5))
    w32 = rc.bf16_to_f32(w)
    sc = rc.fp8_row_scales(w32)
    q = rc.quantize_fp8_rows(w32, sc)
    out["c3_w_sha"], out["c3_q_sha"], out["c3_x_sha"] = sha(w), sha(q), sha(X)
    for M in (1, 2, 4, 8, 16, 32, 64):
        xin = X[0] if M == 1 else X[:M]
        out[f"c3_y_bf16_m{M}"] = rf.linear_bf16(w, xin).reshape(M, K)
        out[f"c3_y_fp8_m{M}"] = rf.linear_fp8(q, sc, xin).reshape(M, K)
    # config 4: lm_head, chunked like the reference's lm_head()
    w = bf16_normal(seed_of(4, 0, 0), (V, K), 0.02)
    X = bf16_normal(seed_of(4, 0, 1), (8, K), 1.0)
    out["c4_w_sha"], out["c4_x_sha"] = sha(w), sha(X)
    logits = np.empty((8, V), np.uint16)
    for m in range(8):
        h32 = rc.bf16_to_f32(X[m])
        for s in range(0, V, 8192):
            logits[m, s:s + 8192] = rc.f32_to_bf16(rc.bf16_to_f32(w[s:s + 8192]) @ h32)
    out["c4_logits_m0"] = logits[0]
    out["c4_argmax"] = np.array([rf.MiniCPM5Ref.greedy(logits[m]) for m in range(8)], np.int64)
    out["c4_top2_gap"] = np.array(
        [np.diff(np.sort(rc.bf16_to_f32(logits[m]))[-2:])[0] for m in range(8)], np.float32)
    np.savez_compressed(os.path.join(HERE, "baseline.npz"), **out)


if __name__ == "__main__":
    codec_fixture()
    small_fixture()
    baseline_fixture()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
