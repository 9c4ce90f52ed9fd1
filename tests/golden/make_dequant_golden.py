#!/usr/bin/env python3
"""Extract the dequantisation golden vectors this repository pins its oracle to.

Source: ``crates/denno-engine/tests/data/dequant_ref.bin`` of a denno-beta
checkout -- raw GGUF blocks and the f32 rows llama.cpp's ``dequantize_row_*``
produced for them (the reference's own bit-exactness fixture, read by its
``tests/dequant_ref.rs``).  The sections of the block types handled here are
copied unchanged, in the same container format:

    u32 n_sections; { u32 len, name; u32 nbytes, raw; u32 nf32, f32[nf32] } ...

    python make_dequant_golden.py <denno-beta checkout>
"""
import os
import struct
import sys

KEEP = ["Q8_0", "Q4_0", "Q4_0_EDGE", "Q5_1", "Q4_K", "Q5_K", "Q6_K", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ4_NL",
        "IQ4_XS", "Q2_0"]


def sections(data):
    p = 0
    (n,) = struct.unpack_from("<I", data, p)
    p += 4
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", data, p)
        name = data[p + 4:p + 4 + nl].decode()
        p += 4 + nl
        (nb,) = struct.unpack_from("<I", data, p)
        raw = data[p + 4:p + 4 + nb]
        p += 4 + nb
        (nf,) = struct.unpack_from("<I", data, p)
        f32 = data[p + 4:p + 4 + 4 * nf]
        p += 4 + 4 * nf
        yield name, raw, f32
    assert p == len(data)


def main(argv):
    src = os.path.join(argv[1], "crates", "denno-engine", "tests", "data", "dequant_ref.bin")
    data = open(src, "rb").read()
    out = bytearray()
    kept = [(n, r, f) for n, r, f in sections(data) if n in KEEP]
    assert sorted(n for n, _, _ in kept) == sorted(KEEP), "fixture lacks a section"
    out += struct.pack("<I", len(kept))
    for name, raw, f32 in kept:
        out += struct.pack("<I", len(name)) + name.encode()
        out += struct.pack("<I", len(raw)) + raw
        out += struct.pack("<I", len(f32) // 4) + f32
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dequant_golden.bin")
    open(dst, "wb").write(bytes(out))
    print("wrote %s: %d sections, %d bytes" % (dst, len(kept), len(out)))


if __name__ == "__main__":
    main(sys.argv)
