"""The oracle's dequantisers against the reference's llama.cpp golden vectors.

Mirrors crates/denno-engine/tests/dequant_ref.rs (kquant_dequant_bitexact_vs_llama_cpp):
same fixture sections, same bit-for-bit requirement.
"""
import os
import struct

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dequant_golden.bin")


def _sections():
    data = open(GOLDEN, "rb").read()
    p = 0
    (n,) = struct.unpack_from("<I", data, p)
    p += 4
    out = []
    for _ in range(n):
        (nl,) = struct.unpack_from("<I", data, p)
        name = data[p + 4:p + 4 + nl].decode()
        p += 4 + nl
        (nb,) = struct.unpack_from("<I", data, p)
        raw = np.frombuffer(data, np.uint8, nb, p + 4)
        p += 4 + nb
        (nf,) = struct.unpack_from("<I", data, p)
        want = np.frombuffer(data, np.float32, nf, p + 4)
        p += 4 + 4 * nf
        out.append((name, raw, want))
    assert p == len(data)
    return out


SECTIONS = _sections()


def test_fixture_has_the_path_types():
    names = {s[0] for s in SECTIONS}
    assert {"Q4_K", "IQ3_XXS", "Q6_K", "Q8_0", "Q5_K", "Q5_1"} <= names


@pytest.mark.parametrize("name,raw,want", SECTIONS, ids=[s[0] for s in SECTIONS])
def test_dequant_bit_exact(orc, name, raw, want):
    ty = orc.TYPE_BY_NAME[name]
    got = orc.dequant_row(ty, raw, want.size)
    assert raw.size == want.size // orc.blck_size(ty) * orc.type_size(ty)
    bad = np.nonzero(got.view(np.uint32) != want.view(np.uint32))[0]
    assert bad.size == 0, "%s: first mismatch at %d: got %r want %r" % (name, bad[0], got[bad[0]], want[bad[0]])


def test_row_bytes_rejects_partial_blocks(orc):
    # moe_expert.rs:84-100: n_in must be a whole number of blocks
    assert orc.row_bytes(orc.Q4_K, 2048) == 8 * 144
    assert orc.row_bytes(orc.IQ3_XXS, 512) == 2 * 98
    assert orc.row_bytes(orc.Q8_0, 64) == 68
    with pytest.raises(ValueError):
        orc.row_bytes(orc.Q4_K, 100)
    with pytest.raises(ValueError):
        orc.row_bytes(99, 256)


def test_gemv_scalar_is_dequant_then_sequential_dot(orc):
    # moe_expert.rs:698-713: out[r] = dot_seq(dequant(row r), x)
    rng = np.random.default_rng(1)
    for ty in (orc.Q4_K, orc.IQ3_XXS, orc.Q6_K, orc.Q8_0):
        n_in, n_out = 512, 5
        w = orc.synth_blocks(ty, 7, ty, n_out * n_in // orc.blck_size(ty))
        x = rng.standard_normal(n_in).astype(np.float32)
        got = orc.gemv_scalar(ty, w, n_in, n_out, x)
        rb = orc.row_bytes(ty, n_in)
        for r in range(n_out):
            row = orc.dequant_row(ty, w[r * rb:(r + 1) * rb], n_in)
            acc = np.float32(0)
            for i in range(n_in):
                acc = np.float32(acc + np.float32(row[i] * x[i]))
            assert got[r].view(np.uint32) == acc.view(np.uint32)
        # the multi-threaded lane-split variant stays within the reference's own bound
        # between its fused and scalar kernels (moe_expert.rs:8755-8758)
        fast = orc.gemv_mt(ty, w, n_in, n_out, x)
        assert np.all(np.abs(fast - got) <= 1e-4 + 1e-5 * np.abs(got) * 50)
