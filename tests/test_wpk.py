"""The packed-weight reader: header/TOC validation on CPU (no GPU calls), shard and
interleave uploads on GPU."""
import os
import struct

import numpy as np
import pytest

import oracle_np as onp
import wpk_np


def _sections():
    w = onp.seeded_bf16(1, (24, 64), 0.02)
    gu = onp.seeded_bf16(2, (32, 64), 0.02)
    q, sc = onp.make_fp8_weight(gu)
    return w, gu, q, sc, [("final_norm", onp.seeded_bf16(3, (64,), 1.0)), ("layer0.qkv", w), ("layer0.gate_up", q, sc),
                          ("layer1.gate_up", gu)]


def test_name_hash_matches_fnv_vectors(pkg):
    lib = pkg.lib()
    assert lib.mc_sm100_wpk_name_hash(b"") == 0xCBF29CE484222325
    assert lib.mc_sm100_wpk_name_hash(b"a") == 0xAF63DC4C8601EC8C
    assert lib.mc_sm100_wpk_name_hash(b"foobar") == 0x85944171F73967E8


def test_open_find_and_layout(pkg, tmp_path):
    w, gu, q, sc, secs = _sections()
    p = str(tmp_path / "m.wpk")
    wpk_np.write_wpk(p, secs)
    raw = open(p, "rb").read()
    assert struct.unpack_from("<I", raw, 0)[0] == 0x31504B4D and struct.unpack_from("<Q", raw, 56)[0] == 768   # align256(64+132*4)
    h = pkg.wpk_open(p)
    try:
        assert pkg.lib().mc_sm100_wpk_section_count(h) == 4
        s = pkg.wpk_find(h, "layer0.qkv")
        assert (s.dtype, s.rank, s.dims[0], s.dims[1], s.data_bytes) == (0, 2, 24, 64, 24 * 64 * 2) and s.data_offset % 256 == 0
        assert raw[s.data_offset:s.data_offset + s.data_bytes] == w.tobytes()
        s = pkg.wpk_find(h, "layer0.gate_up")
        assert s.dtype == 2 and s.scale_bytes == 32 * 4 and s.scale_offset == s.data_offset + s.data_bytes
        assert raw[s.scale_offset:s.scale_offset + s.scale_bytes] == sc.tobytes()
        with pytest.raises(pkg.McError) as e:
            pkg.wpk_find(h, "layer9.qkv")
        assert e.value.status == 4 and "missing section" in e.value.message
    finally:
        pkg.wpk_close(h)


@pytest.mark.parametrize("what", ["magic", "abi", "sm", "toc_offset", "reserved", "truncated", "duplicate", "misaligned", "size"])
def test_corrupt_files_are_rejected(pkg, tmp_path, what):
    _, _, _, _, secs = _sections()
    p = str(tmp_path / "m.wpk")
    wpk_np.write_wpk(p, secs)
    raw = bytearray(open(p, "rb").read())
    if what == "magic": raw[0] ^= 0xFF
    elif what == "abi": struct.pack_into("<H", raw, 4, 3)
    elif what == "sm": struct.pack_into("<H", raw, 6, 90)
    elif what == "toc_offset": struct.pack_into("<Q", raw, 48, 128)
    elif what == "reserved": struct.pack_into("<I", raw, 44, 1)
    elif what == "truncated": raw = raw[:len(raw) - 600]
    elif what == "duplicate": raw[64 + 132:64 + 132 + 8] = raw[64:72]
    elif what == "misaligned": struct.pack_into("<Q", raw, 64 + 132 + 52, struct.unpack_from("<Q", raw, 64 + 132 + 52)[0] + 16)
    elif what == "size": struct.pack_into("<Q", raw, 64 + 132 + 60, 100)
    open(p, "wb").write(bytes(raw))
    with pytest.raises(pkg.McError) as e:
        pkg.wpk_open(p)
    assert e.value.status in (2, 4) and e.value.message
    with pytest.raises(pkg.McError) as e:
        pkg.wpk_open(str(tmp_path / "nope.wpk"))
    assert e.value.status == 2


@pytest.mark.gpu
def test_upload_shards_and_interleave(pkg, tmp_path):
    torch = pytest.importorskip("torch")
    w, gu, q, sc, secs = _sections()
    p = str(tmp_path / "m.wpk")
    wpk_np.write_wpk(p, secs, target_sm=100)
    h = pkg.wpk_open(p)
    try:
        d = torch.zeros((8, 64), dtype=torch.int16, device="cuda")
        pkg.wpk_upload(h, "layer0.qkv", 8, 16, False, d)                       # an N-shard: rows 8..15
        assert np.array_equal(d.cpu().numpy().view(np.uint16), w[8:16])
        d = torch.zeros((12, 64), dtype=torch.uint8, device="cuda")            # pairs 2..7 of the fused e4m3 tensor
        ds = torch.zeros(12, dtype=torch.float32, device="cuda")
        pkg.wpk_upload(h, "layer0.gate_up", 2, 8, True, d, ds)
        want = np.empty((12, 64), np.uint8); want[0::2], want[1::2] = q[2:8], q[18:24]
        wsc = np.empty(12, np.float32); wsc[0::2], wsc[1::2] = sc[2:8], sc[18:24]
        assert np.array_equal(d.cpu().numpy(), want) and np.array_equal(ds.cpu().numpy(), wsc)
        d = torch.zeros((32, 64), dtype=torch.int16, device="cuda")
        pkg.wpk_upload(h, "layer1.gate_up", 0, 16, True, d)
        want = np.empty_like(gu); want[0::2], want[1::2] = gu[:16], gu[16:]
        assert np.array_equal(d.cpu().numpy().view(np.uint16), want)
        with pytest.raises(pkg.McError):
            pkg.wpk_upload(h, "layer0.qkv", 0, 25, False, d)                   # beyond the section
        small = torch.zeros(8, dtype=torch.int16, device="cuda")
        with pytest.raises(pkg.McError):
            pkg.wpk_upload(h, "layer0.qkv", 0, 24, False, small)               # destination too small
    finally:
        pkg.wpk_close(h)


def test_writer_is_byte_identical_to_the_packer_layout(pkg, tmp_path):
    """The C writer against the restated packer (oracle/wpk_np.py): same bytes, and readable back."""
    w, gu, q, sc, secs = _sections()
    a, b = str(tmp_path / "oracle.wpk"), str(tmp_path / "lib.wpk")
    wpk_np.write_wpk(a, secs)
    pkg.wpk_write(b, secs)
    assert open(a, "rb").read() == open(b, "rb").read()
    h = pkg.wpk_open(b)
    try:
        s = pkg.wpk_find(h, "layer0.gate_up")
        assert (s.dtype, s.dims[0], s.scale_bytes, s.scale_offset) == (2, 32, 32 * 4, s.data_offset + s.data_bytes)
    finally:
        pkg.wpk_close(h)
    with pytest.raises(pkg.McError):                        # a section name twice
        pkg.wpk_write(str(tmp_path / "dup.wpk"), [("a", w), ("a", w)])
    assert not os.path.exists(str(tmp_path / "dup.wpk"))    # aborted writers leave no file behind


def test_host_quantiser_matches_reference_fixture(pkg, golden):
    """mc_sm100_quantize_rows_host against the reference packer's outputs (golden fixture) and the oracle."""
    g = golden["codec"]
    assert np.array_equal(pkg.e4m3_from_f32_host(g["enc_in"]), g["enc_out"])        # all 20999 reference encoder outputs
    # through the row quantiser: every fixture input that is exact in bf16 and within +-448
    # goes into a row whose maximum is 448, so that the row scale is exactly 1 and q = e4m3(v)
    v = g["enc_in"]
    exact = (onp.bf16_to_f32(onp.f32_to_bf16(v)) == v) & (np.abs(v) <= 448.0)
    vin, want = v[exact], g["enc_out"][exact]
    assert vin.size > 200           # code points, midpoints and boundaries of the fixture survive the bf16 filter
    row = np.concatenate(([np.float32(448.0)], vin)).astype(np.float32)
    pad = (-row.size) % 16
    row = np.concatenate((row, np.zeros(pad, dtype=np.float32)))
    q, sc = pkg.quantize_rows_host(onp.f32_to_bf16(row).reshape(1, -1))
    assert sc[0] == np.float32(1.0) and np.array_equal(q[0, 1:1 + vin.size], want)
    # the packer's row fixture (fp32 rows): rows that are exact in bf16 must reproduce codes and scales
    rw = g["rows_w"]
    rows_exact = np.all(onp.bf16_to_f32(onp.f32_to_bf16(rw)) == rw, axis=1)
    if rows_exact.any():
        q, sc = pkg.quantize_rows_host(onp.f32_to_bf16(rw[rows_exact]))
        assert np.array_equal(q, g["rows_q"][rows_exact]) and np.array_equal(sc.view(np.uint32), g["rows_scale"][rows_exact].view(np.uint32))
    rng = np.random.default_rng(77)
    w = onp.f32_to_bf16((rng.standard_normal((64, 256)) * 0.02).astype(np.float32))
    w[3, :] = 0                                             # all-zero row: scale floor 1e-12, codes 0
    w[5, 7] = 0x7F80                                        # +inf saturates to 448
    w[6, 9] = 0x7FC0                                        # NaN saturates too, never 0x7F
    q, sc = pkg.quantize_rows_host(w)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        rq, rsc = onp.make_fp8_weight(w)
    rows = [r for r in range(64) if r not in (5, 6)]        # rows with inf/NaN: the row maximum itself is not finite
    assert np.array_equal(q[rows], rq[rows]) and np.array_equal(sc[rows].view(np.uint32), rsc[rows].view(np.uint32))
    assert sc[3] == np.float32(1e-12) and not q[3].any()
    assert not np.any((q & 0x7F) == 0x7F)
