"""CPU oracle (numpy) for the decode linear-layer path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy, the arithmetic the reference defines for
the decode-time linear layers.  It is the checker for the CUDA library and the
`port`-kind CPU baseline of the benchmark; it is never imported by the product
package and is never a fallback.

Parity pin: every function here is compared bit-for-bit against the reference's
own Python implementation (imported where it lies, in the build container) by
`tests/golden/make_golden.py`; the resulting input/output vectors are committed
under `tests/golden/` and re-checked by the CPU test-suite.  The e4m3 / bf16 /
FNV-1a known-answer vectors of the reference's tests are checked as well.

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import numpy as np

FP8_MAX = np.float32(448.0)           # tools/minicpm_common.py:126
FP8_SCALE_FLOOR = np.float32(1e-12)   # tools/minicpm_common.py:127
RMS_EPS = np.float32(1e-6)            # native/runtime/generated_model_config.h:23


# --------------------------------------------------------------------------
# bf16 <-> f32   (tools/minicpm_common.py:102-113)
# --------------------------------------------------------------------------
def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    """Widen bf16 bit patterns (uint16) to float32: bits << 16, exact."""
    wide = np.ascontiguousarray(u16).astype(np.uint32)
    return (wide << np.uint32(16)).view(np.float32)


def f32_to_bf16(f32: np.ndarray) -> np.ndarray:
    """Narrow float32 to bf16 bits with round-to-nearest-even on bit 16.

    Same integer formula as the reference: (u + 0x7FFF + lsb) >> 16, so NaN/inf
    behave exactly like it does (no special-casing).
    """
    bits = np.ascontiguousarray(f32, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


# --------------------------------------------------------------------------
# e4m3 codec   (decode: native/kernels/sm120/kernels.h:131-148 and
#               tools/minicpm_common.py:174-201; encode: minicpm_common.py:130-171)
# --------------------------------------------------------------------------
def _decode_table() -> np.ndarray:
    tab = np.empty(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 0x7
        if e == 0:
            mag = (m / 8.0) * 2.0 ** -6            # subnormal grid k * 2^-9
        else:
            mag = (1.0 + m / 8.0) * 2.0 ** (e - 7)  # 0x7F/0xFF come out as 480
        tab[code] = np.float32(sign * mag)
    # keep the sign of zero (0x80 -> -0.0), as the reference's bit construction does
    tab[0x80] = np.float32(-0.0)
    return tab


E4M3_TABLE = _decode_table()


def e4m3_to_f32(q: np.ndarray) -> np.ndarray:
    """uint8 e4m3 codes -> float32 (exact; codes 0x7F/0xFF decode to +/-480)."""
    return E4M3_TABLE[np.asarray(q, dtype=np.uint8)]


def f32_to_e4m3(f32: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 code, RNE on the 3-bit mantissa, magnitudes beyond 448
    (inf and NaN included) saturate to +/-448; never emits 0x7F/0xFF.

    Restated with exact float64 arithmetic instead of the reference's bit
    surgery: scale the magnitude onto the integer grid of its binade
    (2^(e-10) for normals, 2^-9 for subnormals), round half to even, rebuild
    the code.  Bit-equality with the reference encoder over random and
    boundary inputs is part of the golden pin.
    """
    f = np.ascontiguousarray(f32, dtype=np.float32)
    sign = (f.view(np.uint32) >> np.uint32(31)).astype(np.uint8) << np.uint8(7)
    mag = np.abs(f).astype(np.float64)
    mag = np.where(np.isfinite(mag), mag, 1e9)          # inf/NaN saturate
    # exponent of the binade (frexp is exact), clamped to the subnormal grid
    e = np.frexp(mag)[1].astype(np.int64) - 1
    e = np.maximum(e, -6)
    step = np.exp2((e - 3).astype(np.float64))           # spacing inside binade
    k = np.rint(mag / step)                              # rint = half to even
    val = k * step                                       # rounded magnitude
    val = np.minimum(val, 448.0)
    # rebuild code from the rounded value
    e2 = np.frexp(val)[1].astype(np.int64) - 1
    normal = val >= 2.0 ** -6
    e2 = np.where(normal, e2, -6)
    man = np.where(normal, val / np.exp2(e2.astype(np.float64)) * 8.0 - 8.0,
                   val * 512.0)
    expf = np.where(normal, e2 + 7, 0)
    code = (expf.astype(np.int64) << 3) + man.astype(np.int64)
    code = np.minimum(code, 0x7E).astype(np.uint8)
    return sign | code


def fp8_row_scales(w32: np.ndarray) -> np.ndarray:
    """Per-output-row scale max|row|/448, floored at 1e-12 (minicpm_common.py:204-207)."""
    amax = np.max(np.abs(w32.astype(np.float32)), axis=-1)
    return np.maximum(amax / FP8_MAX, FP8_SCALE_FLOOR).astype(np.float32)


def quantize_fp8_rows(w32: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """q = e4m3(w / scale) row-wise, fp32 division (minicpm_common.py:210-212)."""
    return f32_to_e4m3(w32.astype(np.float32) / scales[..., np.newaxis])


# --------------------------------------------------------------------------
# linear layers   (tools/reference_forward.py:158-172)
# --------------------------------------------------------------------------
def linear_bf16(w_u16: np.ndarray, x_u16: np.ndarray) -> np.ndarray:
    """y = bf16(x @ W^T), fp32 accumulate.  W [N,K], x [K] or [M,K]."""
    return f32_to_bf16(bf16_to_f32(x_u16) @ bf16_to_f32(w_u16).T)


def linear_fp8(q_u8: np.ndarray, scales: np.ndarray, x_u16: np.ndarray) -> np.ndarray:
    """y = bf16(scale[n] * sum_k e4m3(q[n,k]) * x[k]); the row scale multiplies
    the finished fp32 sum once (reference_forward.py:165-172; gemv_fp8.cu:166-172)."""
    acc = bf16_to_f32(x_u16) @ e4m3_to_f32(q_u8).T
    return f32_to_bf16(acc.astype(np.float32) * scales.astype(np.float32))


def linear_f64(w32: np.ndarray, x_u16: np.ndarray, scales: np.ndarray | None = None) -> np.ndarray:
    """Double-accumulate statement used by the reference's kernel tests
    (native/tests/gemv_bench.cpp:122-162, kernel_ops.cpp:842-850): returns the
    fp32-rounded exact result, before the bf16 rounding.  w32 is the already
    decoded weight (bf16 or e4m3 widened to f32)."""
    acc = bf16_to_f32(x_u16).astype(np.float64) @ w32.astype(np.float64).T
    if scales is not None:
        acc = acc * scales.astype(np.float64)
    return acc.astype(np.float32)


# --------------------------------------------------------------------------
# elementwise pieces of the layer   (reference_forward.py:175-183, 235-237;
#                                    swiglu.cu:57-70; rmsnorm.cu:130-166)
# --------------------------------------------------------------------------
def swiglu_bf16(g_u16: np.ndarray, u_u16: np.ndarray) -> np.ndarray:
    """bf16( silu(f32 g) * f32 u ) on bf16-rounded gate/up."""
    g = bf16_to_f32(g_u16)
    silu = g * (np.float32(1.0) / (np.float32(1.0) + np.exp(-g)))
    return f32_to_bf16(silu * bf16_to_f32(u_u16))


def rmsnorm_bf16(w_u16: np.ndarray, x_u16: np.ndarray, eps: np.float32 = RMS_EPS) -> np.ndarray:
    """bf16( x * rsqrt(mean(x^2)+eps) * w ), one rounding."""
    x = bf16_to_f32(x_u16)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps)
    return f32_to_bf16(x * (np.float32(1.0) / np.sqrt(ms)) * bf16_to_f32(w_u16))


def add_bf16(a_u16: np.ndarray, b_u16: np.ndarray) -> np.ndarray:
    """bf16( f32 a + f32 b ): the residual is stored rounded."""
    return f32_to_bf16(bf16_to_f32(a_u16) + bf16_to_f32(b_u16))


def greedy(logits_u16: np.ndarray) -> int:
    """argmax over bf16 logits compared as f32; ties -> lowest index
    (reference_forward.py:327-331; sampling.cu:77-83)."""
    return int(np.argmax(bf16_to_f32(logits_u16)))


def gate_up_swiglu_bf16(w_u16: np.ndarray, x_u16: np.ndarray) -> np.ndarray:
    """Fused gate_up projection + SwiGLU on the WPK row order gate|up
    (reference_forward.py:293-294): both halves are rounded to bf16 first."""
    y = linear_bf16(w_u16, x_u16)
    inter = w_u16.shape[0] // 2
    return swiglu_bf16(y[..., :inter], y[..., inter:])


def gate_up_swiglu_fp8(q_u8: np.ndarray, scales: np.ndarray, x_u16: np.ndarray) -> np.ndarray:
    y = linear_fp8(q_u8, scales, x_u16)
    inter = q_u8.shape[0] // 2
    return swiglu_bf16(y[..., :inter], y[..., inter:])


# --------------------------------------------------------------------------
# activation quantiser of the W8A8 variant   (native/kernels/sm120/quant.cu:34-77)
# --------------------------------------------------------------------------
def quant_rows_e4m3(x_u16: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-row dynamic quantisation of bf16 activations: scale = amax/448
    (all-zero row -> 1.0), q = e4m3_rne_satfinite(x * (448/amax))."""
    x = bf16_to_f32(x_u16)
    amax = np.max(np.abs(x), axis=-1)
    scale = np.where(amax > 0, amax / FP8_MAX, np.float32(1.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(amax > 0, FP8_MAX / amax, np.float32(0.0)).astype(np.float32)
    return f32_to_e4m3(x * inv[..., np.newaxis]), scale


# --------------------------------------------------------------------------
# FNV-1a 64 (section-name hash of the packed weight file; minicpm_common.py:80-95)
# --------------------------------------------------------------------------
def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


# --------------------------------------------------------------------------
# seeded synthetic inputs shared by tests, bench and the C side
# --------------------------------------------------------------------------
SEED_BASE = 20260908


def seeded_bf16(seed: int, shape, std: float) -> np.ndarray:
    """Normal(0, std) drawn in fp32 from numpy's PCG64, rounded to bf16 bits."""
    rng = np.random.default_rng(seed)
    return f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def make_fp8_weight(w_u16: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """bf16 weight -> (e4m3 codes, fp32 row scales) with the packer's rule."""
    w32 = bf16_to_f32(w_u16)
    sc = fp8_row_scales(w32)
    return quantize_fp8_rows(w32, sc), sc


def bf16_ulp(ref_f32: np.ndarray) -> np.ndarray:
    """Size of one bf16 unit in the last place at the magnitude of ref."""
    a = np.abs(ref_f32.astype(np.float32))
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -126))))
    return np.exp2(e - 7).astype(np.float32)


# ---- sampling tail (native/kernels/sm120/sampling.cu:276-283, 489-531; kernels.h:108-113) -------------
_M64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    """Seed -> generator state, as the host does (native/kernels/sm120/kernels.h:108-113)."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def rng_next(state: int) -> tuple[int, int]:
    """xorshift64*: (32-bit draw, new state) (sampling.cu:276-283)."""
    x = state
    x ^= x >> 12
    x = (x ^ (x << 25)) & _M64
    x ^= x >> 27
    return ((x * 2685821657736338717) & _M64) >> 32, x


def sample_topk_topp(logits_u16: np.ndarray, temperature: float, top_p: float, top_k: int, rng_state: int, index_base: int = 0):
    """One row: the k strongest logits (value descending, index ascending), temperature softmax, top-p cut,
    renormalisation and the draw, every sum sequential in fp32 as sampling.cu:489-531 does it.  Returns
    (token, new generator state, margin) where margin is the distance of the uniform draw from the nearest
    decision boundary (a device exp that differs in the last bit can only change the token when it is tiny)."""
    v = bf16_to_f32(np.asarray(logits_u16).reshape(-1))
    k = max(1, min(int(top_k), 128))
    order = np.lexsort((np.arange(v.size), -v.astype(np.float64)))[:k]        # value desc, index asc
    sv = v[order].astype(np.float32)
    hsize = min(k, v.size)
    if not (temperature > 0) or hsize == 1:
        return int(order[0]) + index_base, rng_state, 1.0
    f32 = np.float32
    mx = sv[0]
    sum_ = f32(0)
    e = np.empty(hsize, dtype=np.float32)
    for i in range(hsize):
        e[i] = np.exp(f32((sv[i] - mx) / f32(temperature)), dtype=np.float32)
        sum_ = f32(sum_ + e[i])
    e = (e / sum_).astype(np.float32)
    cut = hsize
    if top_p < 1.0:
        cum = f32(0)
        for i in range(hsize):
            cum = f32(cum + e[i])
            if cum >= f32(top_p):
                cut = i + 1
                break
    kept = f32(0)
    for i in range(cut):
        kept = f32(kept + e[i])
    r, state = rng_next(rng_state)
    u = f32(r >> 8) * f32(1.0 / 16777216.0)
    acc, pick, margin = f32(0), cut - 1, 1.0
    for i in range(cut):
        acc = f32(acc + f32(e[i] / kept))
        margin = min(margin, abs(float(u) - float(acc)))
        if u < acc:
            pick = i
            break
    return int(order[pick]) + index_base, state, margin
