"""CPU: the oracle's linear layers against fixtures made by the reference's
Python code, the C restatement against the numpy one, and the reference's own
native CPU cross-check (compiled in place) against both."""
import ctypes
import hashlib
import os

import numpy as np
import pytest

import oracle_np as onp
from parity import check_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def c_linear_bf16(lib, w, x, use_double=0, threads=4):
    M = 1 if x.ndim == 1 else x.shape[0]
    N, K = w.shape
    y = np.empty((M, N), np.uint16)
    lib.oracle_linear_bf16(_ptr(w), _ptr(np.ascontiguousarray(x)), _ptr(y), None, M, N, K, use_double, threads)
    return y


def c_linear_fp8(lib, q, sc, x, use_double=0, threads=4):
    M = 1 if x.ndim == 1 else x.shape[0]
    N, K = q.shape
    y = np.empty((M, N), np.uint16)
    lib.oracle_linear_fp8(_ptr(q), _ptr(sc), _ptr(np.ascontiguousarray(x)), _ptr(y), None, M, N, K, use_double, threads)
    return y


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_small_linear_vs_reference_fixture(golden, cpu_ref_lib, tag):
    g = golden["small"]
    w, x, q, sc = g[f"{tag}_w"], g[f"{tag}_x"], g[f"{tag}_q"], g[f"{tag}_scale"]
    # quantiser: bit-exact with the reference packer
    q2, sc2 = onp.make_fp8_weight(w)
    assert np.array_equal(q2, q) and np.array_equal(sc2.view(np.uint32), sc.view(np.uint32))
    # matmuls: same statement, BLAS summation order may differ between hosts
    check_close(onp.linear_bf16(w, x), g[f"{tag}_y_bf16"], what=f"np bf16 {tag}")
    check_close(onp.linear_fp8(q, sc, x), g[f"{tag}_y_fp8"], abs_floor=1e-4, what=f"np fp8 {tag}")
    for dbl in (0, 1):
        check_close(c_linear_bf16(cpu_ref_lib, w, x, dbl), g[f"{tag}_y_bf16"], what=f"C bf16 {tag}")
        check_close(c_linear_fp8(cpu_ref_lib, q, sc, x, dbl), g[f"{tag}_y_fp8"], abs_floor=1e-4, what=f"C fp8 {tag}")


def test_elementwise_vs_reference_fixture(golden, cpu_ref_lib):
    g = golden["small"]
    assert np.array_equal(onp.swiglu_bf16(g["sw_g"], g["sw_u"]), g["sw_out"])
    res = onp.add_bf16(g["rn_x"], g["rn_add"])
    assert np.array_equal(res, g["rn_res"])
    # mean() is a pairwise sum in numpy: allow the last bf16 bit
    check_close(onp.rmsnorm_bf16(g["rn_w"], res), g["rn_out"], what="rmsnorm np")
    assert onp.greedy(g["am_logits"]) == int(g["am_idx"]) == 17
    # C restatement
    src = np.concatenate([g["sw_g"], g["sw_u"]], axis=1).copy()
    out = np.empty_like(g["sw_g"])
    cpu_ref_lib.oracle_swiglu_gated(_ptr(src), _ptr(out), 2, g["sw_g"].shape[1])
    d = np.abs(onp.bf16_to_f32(out) - onp.bf16_to_f32(g["sw_out"]))
    assert (d <= onp.bf16_ulp(onp.bf16_to_f32(g["sw_out"]))).all()       # expf vs np.exp: <= 1 ulp
    r = g["rn_x"].copy()
    o = np.empty_like(r)
    cpu_ref_lib.oracle_residual_rmsnorm(_ptr(r), _ptr(g["rn_add"]), _ptr(g["rn_w"]), _ptr(o), r.size,
                                        ctypes.c_float(1e-6))
    assert np.array_equal(r, g["rn_res"])
    check_close(o, g["rn_out"], what="rmsnorm C")
    cpu_ref_lib.oracle_argmax_bf16.restype = ctypes.c_int32
    assert cpu_ref_lib.oracle_argmax_bf16(_ptr(g["am_logits"]), g["am_logits"].size) == 17


def test_argmax_edge_cases(cpu_ref_lib):
    cpu_ref_lib.oracle_argmax_bf16.restype = ctypes.c_int32
    neg_inf = np.full(8, 0xFF80, np.uint16)          # all -inf: equal to the start value, index 0 wins
    assert cpu_ref_lib.oracle_argmax_bf16(_ptr(neg_inf), 8) == 0
    nan = np.full(8, 0x7FC0, np.uint16)              # NaN never compares: sentinel index
    assert cpu_ref_lib.oracle_argmax_bf16(_ptr(nan), 8) == 2 ** 31 - 1
    one = onp.f32_to_bf16(np.array([3.0], np.float32))
    assert cpu_ref_lib.oracle_argmax_bf16(_ptr(one), 1) == 0 == onp.greedy(one)


def test_baseline_config1_and_2_vs_reference_fixture(golden):
    """Full-size configs 1 and 2: inputs regenerated from the seeds must hash
    to what the reference saw; the oracle's outputs must match its outputs."""
    g = golden["baseline"]
    K, QKV, I = 2304, 3456, 5760
    w = onp.seeded_bf16(onp.SEED_BASE + 1000, (QKV, K), 0.02)
    x = onp.seeded_bf16(onp.SEED_BASE + 1001, (K,), 1.0)
    assert _sha(w) == str(g["c1_w_sha"]) and _sha(x) == str(g["c1_x_sha"])
    check_close(onp.linear_bf16(w, x), g["c1_y"], what="config1")
    w = onp.seeded_bf16(onp.SEED_BASE + 2000, (2 * I, K), 0.02)
    x = onp.seeded_bf16(onp.SEED_BASE + 2001, (K,), 1.0)
    q, sc = onp.make_fp8_weight(w)
    assert _sha(q) == str(g["c2_q_sha"]) and _sha(sc) == str(g["c2_scale_sha"])
    check_close(onp.linear_fp8(q, sc, x), g["c2_gate_up"], abs_floor=1e-4, what="config2 gate_up")
    # after the SwiGLU a 1-ulp flip of gate or up moves the product by ~1 ulp too
    check_close(onp.gate_up_swiglu_fp8(q, sc, x), g["c2_y"], abs_floor=4e-3, what="config2 swiglu")


def test_reference_native_cross_check(cpu_ref_lib):
    """The reference's own C++ gemv()/rmsnorm()/e4m3 decoder, compiled from its
    sources in place, against the C restatement: bit-exact (same sequential
    fp32 order)."""
    so = os.path.join(ROOT, "oracle", "_ref", "libref_native.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref not built (reference tree not mounted)")
    ref = ctypes.CDLL(so)
    ref.ref_native_e4m3_to_f32.restype = ctypes.c_float
    dec = np.array([ref.ref_native_e4m3_to_f32(ctypes.c_uint8(c)) for c in range(256)], np.float32)
    assert np.array_equal(dec.view(np.uint32), onp.e4m3_to_f32(np.arange(256, dtype=np.uint8)).view(np.uint32))
    w = onp.seeded_bf16(11, (300, 2304), 0.02)
    x = onp.seeded_bf16(12, (2304,), 1.0)
    y = np.empty(300, np.uint16)
    ref.ref_native_gemv(_ptr(x), _ptr(w), 300, 2304, _ptr(y))
    assert np.array_equal(y, c_linear_bf16(cpu_ref_lib, w, x, 0)[0])
    check_close(y, onp.linear_bf16(w, x), what="native ref vs numpy")
    xr = onp.seeded_bf16(13, (2048,), 1.3)
    nw = onp.seeded_bf16(14, (2048,), 1.0)
    o1 = np.empty(2048, np.uint16)
    ref.ref_native_rmsnorm2048(_ptr(xr), _ptr(nw), _ptr(o1))
    r = xr.copy()
    o2 = np.empty(2048, np.uint16)
    cpu_ref_lib.oracle_residual_rmsnorm(_ptr(r), None, _ptr(nw), _ptr(o2), 2048, ctypes.c_float(1e-6))
    assert np.array_equal(o1, o2)
