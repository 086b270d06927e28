"""Writer for the weight "message" files a compiled program reads through
Pt_from_msg (layout: fhe-cmplr/include/fhe/core/rt_data_def.h:91-112).

The compiler normally writes these next to the generated C file.  Synthetic
ones stand in for them in tests and benchmarks: a 4 KiB header page, float32
entries each aligned to 32 bytes, then the lookup table.
"""
import struct

import numpy as np

PAGE = 4096
ALIGN_LOG2 = 5
DE_MSG_F32 = 0
DE_PLAINTEXT = 2


def write_msg_file(path, entries, model=b"synthetic", uuid=b"0" * 36):
    """entries: list of (name, float32 array, scale_degree, level)."""
    payload = bytearray()
    lut = bytearray()
    for index, (name, values, scale, level) in enumerate(entries):
        data = np.ascontiguousarray(values, dtype=np.float32).tobytes()
        pad = (-len(payload)) % (1 << ALIGN_LOG2)
        payload += b"\0" * pad
        offset = PAGE + len(payload)
        payload += data
        packed = (scale & 0xFF) | ((level & 0xFF) << 8) | (offset << 16)
        lut += struct.pack("<16sIIQ", name.encode()[:15], index, len(data), packed)
    pad = (-len(payload)) % (1 << ALIGN_LOG2)
    payload += b"\0" * pad
    lut_ofst = PAGE + len(payload)
    # magic, version, flag, entry type, entry alignment, count, table offset,
    # creation time (two 64-bit words), model name, uuid
    header = struct.pack("<8sIHBBQQqq48s40s", b"!ANTFHE\0", 0, 0, DE_MSG_F32, ALIGN_LOG2,
                         len(entries), lut_ofst, 0, 0, model, uuid)
    assert len(header) == 136
    with open(path, "wb") as f:
        f.write(header + b"\0" * (PAGE - len(header)))
        f.write(payload)
        f.write(lut)
    return lut_ofst


def write_plaintext_file(path, buffers, model=b"synthetic", uuid=b"0" * 36):
    """A data file of pre-encoded plaintexts (entry type DE_PLAINTEXT): buffers is
    a list of (name, bytes, scale_degree, level) where bytes is one
    PLAINTEXT_BUFFER as the reference's Encode_plain_buffer returns it
    (fhe-cmplr/include/fhe/core/rt_encode_api.h:22-27)."""
    payload = bytearray()
    lut = bytearray()
    for index, (name, data, scale, level) in enumerate(buffers):
        pad = (-len(payload)) % (1 << ALIGN_LOG2)
        payload += b"\0" * pad
        offset = PAGE + len(payload)
        payload += data
        packed = (scale & 0xFF) | ((level & 0xFF) << 8) | (offset << 16)
        lut += struct.pack("<16sIIQ", name.encode()[:15], index, len(data), packed)
    pad = (-len(payload)) % (1 << ALIGN_LOG2)
    payload += b"\0" * pad
    lut_ofst = PAGE + len(payload)
    header = struct.pack("<8sIHBBQQqq48s40s", b"!ANTFHE\0", 0, 0, DE_PLAINTEXT, ALIGN_LOG2,
                         len(buffers), lut_ofst, 0, 0, model, uuid)
    with open(path, "wb") as f:
        f.write(header + b"\0" * (PAGE - len(header)))
        f.write(payload)
        f.write(lut)
    return lut_ofst


def write_synthetic_msg_file(path, entry_count, entry_floats=32768, distinct=64, sigma=0.05, seed=7):
    """A stand-in for a compiled model's weight file: entry_count entries of
    entry_floats seeded N(0, sigma) floats each.  Only `distinct` different
    payload rows are stored; the lookup table points every entry at one of
    them, which keeps the file small while each entry keeps its own index
    (and so its own slot in the plaintext cache)."""
    rng = np.random.default_rng(seed)
    rows = rng.normal(0.0, sigma, (distinct, entry_floats)).astype(np.float32)
    payload = rows.tobytes()
    row_bytes = entry_floats * 4
    assert row_bytes % (1 << ALIGN_LOG2) == 0
    lut = bytearray()
    for index in range(entry_count):
        offset = PAGE + (index % distinct) * row_bytes
        packed = 1 | (0 << 8) | (offset << 16)
        lut += struct.pack("<16sIIQ", b"w%d" % index, index, row_bytes, packed)
    lut_ofst = PAGE + len(payload)
    header = struct.pack("<8sIHBBQQqq48s40s", b"!ANTFHE\0", 0, 0, DE_MSG_F32, ALIGN_LOG2,
                         entry_count, lut_ofst, 0, 0, b"synthetic", b"0" * 36)
    with open(path, "wb") as f:
        f.write(header + b"\0" * (PAGE - len(header)))
        f.write(payload)
        f.write(lut)
    return lut_ofst
