"""CPU: the oracle's codecs against the known answers the reference's tests hold
and against fixtures produced by the reference's own Python code."""
import ctypes

import numpy as np

import oracle_np as onp


def _f32(bits):
    return np.array([bits], dtype=np.uint32).view(np.float32)[0]


def test_e4m3_decode_known_answers(cpu_ref_lib):
    # format facts of e4m3 checked by native/tests/kernel_ops.cpp:1238-1249 and tools/test_fp8.py:57-66
    ka = {0x00: 0.0, 0x66: 56.0, 0xE6: -56.0, 0x7E: 448.0, 0xFE: -448.0, 0x01: 2.0 ** -9, 0x02: 2.0 ** -8,
          0x07: 7 * 2.0 ** -9, 0x08: 2.0 ** -6, 0x40: 2.0, 0x50: 8.0, 0x38: 1.0, 0xB8: -1.0, 0x77: 240.0,
          0x7F: 480.0, 0xFF: -480.0}
    cpu_ref_lib.oracle_e4m3_to_f32.restype = ctypes.c_float
    for code, want in ka.items():
        assert onp.e4m3_to_f32(np.uint8(code)) == np.float32(want)
        assert cpu_ref_lib.oracle_e4m3_to_f32(ctypes.c_uint8(code)) == want
    assert np.signbit(onp.e4m3_to_f32(np.uint8(0x80)))


def test_e4m3_encode_known_answers():
    # tools/test_fp8.py:33-54
    enc = [(0.0, 0x00), (1.0, 0x38), (-1.0, 0xB8), (0.5, 0x30), (2.0, 0x40), (1.5, 0x3C), (6.0, 0x4C),
           (240.0, 0x77), (448.0, 0x7E), (449.0, 0x7E), (1000.0, 0x7E), (-1000.0, 0xFE),
           (float("inf"), 0x7E), (float("nan"), 0x7E), (2.0 ** -6, 0x08), (0.001, 0x01), (2.0 ** -10, 0x00),
           (3 * 2.0 ** -10, 0x02), (1.0625, 0x38), (1.1875, 0x3A)]
    v = np.array([a for a, _ in enc], np.float32)
    assert onp.f32_to_e4m3(v).tolist() == [b for _, b in enc]


def test_bf16_rne_known_answers(cpu_ref_lib):
    # native/tests/kernel_ops.cpp:513-531
    tab = [(0x3F800000, 0x3F80), (0x3F000000, 0x3F00), (0xBF800000, 0xBF80), (0x3F808000, 0x3F80),
           (0x3F808001, 0x3F81), (0x3F807FFF, 0x3F80), (0x3F818000, 0x3F82), (0x3F008000, 0x3F00),
           (0x3F018000, 0x3F02), (0x80000000, 0x8000), (0x00000000, 0x0000), (0x00800000, 0x0080),
           (0x00400000, 0x0040), (0x00000001, 0x0000), (0x00008000, 0x0000), (0x00008001, 0x0001),
           (0x7F7FFFFF, 0x7F80)]
    cpu_ref_lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
    for f, b in tab:
        assert int(onp.f32_to_bf16(np.array([_f32(f)]))[0]) == b
        assert cpu_ref_lib.oracle_f32_to_bf16(ctypes.c_float(float(_f32(f)))) == b


def test_fnv1a64_known_answers():
    # tools/minicpm_common.py:94-95; native/tests/kernel_ops.cpp:4232-4234
    assert onp.fnv1a64(b"") == 0xCBF29CE484222325
    assert onp.fnv1a64(b"a") == 0xAF63DC4C8601EC8C
    assert onp.fnv1a64(b"foobar") == 0x85944171F73967E8


def test_codec_fixture_from_reference(golden):
    g = golden["codec"]
    assert np.array_equal(onp.f32_to_e4m3(g["enc_in"]), g["enc_out"])
    assert np.array_equal(onp.e4m3_to_f32(np.arange(256, dtype=np.uint8)).view(np.uint32),
                          g["dec_table"].view(np.uint32))
    assert np.array_equal(onp.f32_to_bf16(g["bf16_in"]), g["bf16_out"])
    sc = onp.fp8_row_scales(g["rows_w"])
    assert np.array_equal(sc.view(np.uint32), g["rows_scale"].view(np.uint32))
    assert sc[3] == np.float32(1e-12)                     # all-zero row: floor, not 1.0
    assert np.array_equal(onp.quantize_fp8_rows(g["rows_w"], sc), g["rows_q"])
    assert int(g["fnv_foobar"]) == onp.fnv1a64(b"foobar")


def test_encode_decode_round_trip_and_half_ulp():
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    assert np.array_equal(onp.f32_to_e4m3(onp.e4m3_to_f32(codes)) & 0x7F, codes & 0x7F)
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(20000) * 50).astype(np.float32)
    x = x[np.abs(x) <= 448]
    q = onp.e4m3_to_f32(onp.f32_to_e4m3(x)).astype(np.float64)
    e = np.floor(np.log2(np.maximum(np.abs(x.astype(np.float64)), 2.0 ** -6)))
    assert np.all(np.abs(q - x) <= 0.5 * 2.0 ** (e - 3) + 1e-12)
    assert not np.any((onp.f32_to_e4m3(x) & 0x7F) == 0x7F)


def test_quant_rows_statement():
    x = onp.seeded_bf16(5, (3, 64), 1.0)
    x[1] = 0
    q, s = onp.quant_rows_e4m3(x)
    assert s[1] == 1.0 and not q[1].any()
    amax = np.abs(onp.bf16_to_f32(x[0])).max()
    assert s[0] == np.float32(amax / np.float32(448.0))
    assert (q[0] & 0x7F).max() == 0x7E
