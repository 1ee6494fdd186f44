"""Writer of the packed weight file (WPK v1).  TEST INFRASTRUCTURE ONLY.

Restates the on-disk layout the reference's packer produces
(tools/minicpm_common.py:47-75 header/TOC records, :318-348 writer,
tools/quantize.py:85-113 placement of the fp32 row scales right after the e4m3
data): 64-byte header, 132-byte packed TOC entries, 256-byte aligned data.
Used by the tests to feed the library's reader; pinned by the byte offsets that
native/tests/kernel_ops.cpp:4245-4300 parses literally and by the FNV-1a vectors.
"""
from __future__ import annotations

import struct

import numpy as np

from oracle_np import fnv1a64

MAGIC = 0x31504B4D
HEADER = struct.Struct("<IHH32sIIQQ")          # 64 bytes
TOC = struct.Struct("<QIII8IQQQQ6Q")           # 132 bytes
assert HEADER.size == 64 and TOC.size == 132


def align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


def write_wpk(path: str, sections, target_sm: int = 120, model_hash: bytes = b"\0" * 32) -> None:
    """sections: list of (name, bf16_u16_array) or (name, e4m3_u8_array, fp32_scales)."""
    count = len(sections)
    data_start = align(64 + TOC.size * count)
    off = data_start
    toc, blobs = [], []
    for sec in sections:
        name, arr = sec[0], np.ascontiguousarray(sec[1])
        dims = list(arr.shape) + [0] * (8 - arr.ndim)
        if len(sec) == 3:                       # dtype 2: e4m3 codes, scales directly behind the data
            sc = np.ascontiguousarray(sec[2], dtype=np.float32)
            d_off, d_n = off, arr.size
            s_off, s_n = d_off + d_n, sc.size * 4
            blobs.append((d_off, arr.tobytes() + sc.tobytes()))
            toc.append(TOC.pack(fnv1a64(name.encode()), 2, 0, arr.ndim, *dims, d_off, d_n, s_off, s_n, *([0] * 6)))
            off = align(s_off + s_n)
        else:
            d_off, d_n = off, arr.size * 2
            blobs.append((d_off, arr.astype(np.uint16).tobytes()))
            toc.append(TOC.pack(fnv1a64(name.encode()), 0, 0, arr.ndim, *dims, d_off, d_n, 0, 0, *([0] * 6)))
            off = align(d_off + d_n)
    with open(path, "wb") as f:
        f.write(HEADER.pack(MAGIC, 2, target_sm, model_hash, count, 0, 64, data_start))
        for t in toc:
            f.write(t)
        for at, blob in blobs:
            f.seek(at)
            f.write(blob)
        f.truncate(max(off, f.tell()))
