"""The arithmetic identities the tensor-core kernels rest on, checked on the CPU against the oracle's block decode
(no GPU, no product code): what must hold for the kernels' operand formats to be EXACT.

* Q4_K with integer weights (csrc/grouped_q4k_int.cu): w = d * sc * q - dmin * m (kquant.rs:505-526), so
  W . x = sum_blocks d * [sum (sc * q) * x] - sum_subblocks (dmin * m) * X with X the sub-block sums of x;
  sc * q <= 945 is exact in fp16 and one fp16 fma (1024 + q) * sc - 1024 * sc produces it; -(dmin * m) is exact as
  fp16 hi + lo.
* IQ3_XXS with exact weights (csrc/grouped_exact.cu): w = db * (grid magnitude) * sign, magnitudes exact in bf16.
* Router operands (csrc/router_tc.cu): an fp32 value is the exact sum of three bf16 numbers (round, round, round).
"""
import numpy as np

SEED = 0xD3770B200


def _bf16_rn(x):
    """float32 array -> the nearest bf16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def _q4k_fields(blocks, n_blocks):
    """d, dmin [nb] float32; sc, m [nb, 8] integers; q [nb, 256] integers, element order of kquant.rs:505-526."""
    b = np.frombuffer(blocks, np.uint8).reshape(n_blocks, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(n_blocks)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32).reshape(n_blocks)
    s = b[:, 4:16].astype(np.int64)
    sc = np.empty((n_blocks, 8), np.int64)
    m = np.empty((n_blocks, 8), np.int64)
    for j in range(8):
        if j < 4:
            sc[:, j] = s[:, j] & 63
            m[:, j] = s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            m[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    qs = b[:, 16:144].astype(np.int64).reshape(n_blocks, 4, 32)
    q = np.empty((n_blocks, 4, 64), np.int64)
    q[:, :, :32] = qs & 0xF   # low nibbles first, then the high nibbles of the same 32 bytes
    q[:, :, 32:] = qs >> 4
    return d, dmin, sc, m, q.reshape(n_blocks, 256)


def test_q4k_integer_weight_decomposition(orc):
    k, n = 1024, 24
    nb = k // 256
    w = orc.synth_blocks(orc.Q4_K, SEED, 901, n * nb)
    x = orc.synth_normal(SEED, 902, 1.0, k)
    want = orc.gemv_scalar(orc.Q4_K, w, k, n, x).astype(np.float64)
    d, dmin, sc, m, q = _q4k_fields(w, n * nb)
    # the field extraction is the format's: rebuilding the weights gives the oracle's dequantised row
    wq = (d[:, None, None] * sc[:, :, None]) * q.reshape(-1, 8, 32) - (dmin[:, None] * m)[:, :, None]
    deq = np.stack([orc.dequant_row(orc.Q4_K, w[r * nb * 144:(r + 1) * nb * 144], k) for r in range(n)])
    assert np.allclose(wq.reshape(n, k), deq, rtol=1e-6, atol=1e-7)
    # (1) sc * q is an integer <= 945: exact in fp16, and one fp16 fma (1024 + q) * sc - 1024 * sc gives it
    iw = sc[:, :, None] * q.reshape(-1, 8, 32)
    assert iw.max() <= 945 and np.array_equal(iw.astype(np.float16).astype(np.int64), iw)
    big = (1024 + q.reshape(-1, 8, 32)).astype(np.float16)      # 0x6400 | q
    assert np.array_equal(big.astype(np.int64), 1024 + q.reshape(-1, 8, 32))
    c = (-1024.0 * sc).astype(np.float16)
    assert np.array_equal(c.astype(np.float64), -1024.0 * sc)   # six bits times 2^10: exact
    fma = (big.astype(np.float64) * sc[:, :, None] + c.astype(np.float64)[:, :, None]).astype(np.float16)  # rounds once
    assert np.array_equal(fma.astype(np.int64), iw)
    # (2) -(dmin * m) as fp16 hi + lo is exact
    v = -(dmin[:, None].astype(np.float64) * m)
    hi = v.astype(np.float16)
    lo = (v - hi.astype(np.float64)).astype(np.float16)
    assert np.array_equal(hi.astype(np.float64) + lo.astype(np.float64), v)
    # (3) the decomposition: block sums scaled by d, minus the offsets against the sub-block sums of x
    xs = x.astype(np.float64).reshape(nb, 8, 32)
    main = np.einsum("rbsi,bsi->rb", iw.reshape(n, nb, 8, 32).astype(np.float64), xs) * d.reshape(n, nb)
    corr = np.einsum("rbs,bs->r", v.reshape(n, nb, 8), xs.sum(axis=2))
    got = main.sum(axis=1) + corr
    rms = np.sqrt(np.mean(want * want))
    assert np.max(np.abs(got - want)) <= 2e-6 * rms   # the oracle's own fp32 rounding


def test_activation_rows_as_scaled_fp16_pairs(orc):
    """Rows scaled by a power of two so that the largest element is in [256, 512): hi + lo fp16 carry 22 bits of every
    element that matters and the sub-block sums (<= 32 * 512) stay inside fp16's range."""
    x = orc.synth_normal(SEED, 903, 37.5, 4096).astype(np.float32)
    x[7] = 3.1e4      # an outlier, as SwiGLU outputs have
    x[11] = 1e-7
    mx = float(np.max(np.abs(x)))
    e = int(np.frexp(mx)[1])
    up = np.float32(2.0 ** (9 - e))
    xs = x * up
    assert 256 <= np.max(np.abs(xs)) < 512
    hi = xs.astype(np.float16)
    lo = (xs - hi.astype(np.float32)).astype(np.float16)
    err = np.abs(hi.astype(np.float64) + lo.astype(np.float64) - xs.astype(np.float64))
    assert np.max(err) <= 2.0 ** -13 * 2.0 ** -11 * 512 + 2.0 ** -25   # 2^-22 of the row's scale (+ the subnormal floor)
    sums = xs.reshape(-1, 32).astype(np.float64).sum(axis=1)
    assert np.max(np.abs(sums)) < 65504


def test_iq3xxs_magnitudes_are_exact_in_bf16(orc):
    k = 512
    w = orc.synth_blocks(orc.IQ3_XXS, SEED, 904, k // 256)
    row = orc.dequant_row(orc.IQ3_XXS, w, k).astype(np.float64)
    b = np.frombuffer(w, np.uint8).reshape(-1, 98)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float64).reshape(-1)
    aux = b[:, 66:98].copy().view(np.uint32).reshape(-1, 8)          # one 32-bit word per 32-element sub-block
    db = d[:, None] * (0.5 + (aux >> 28)) * 0.5
    mag = row.reshape(-1, 8, 32) / db[:, :, None]                     # grid magnitude x sign
    assert np.allclose(mag, np.round(mag), atol=1e-3)
    mag = np.round(mag).astype(np.float32)
    assert np.max(np.abs(mag)) <= 62
    assert np.array_equal(_bf16_rn(mag), mag)


def test_three_bf16_parts_carry_an_fp32_exactly(orc):
    x = np.concatenate([orc.synth_normal(SEED, 905, 1.0, 20000), orc.synth_normal(SEED, 906, 0.02, 20000),
                        np.array([0.0, 1.0, -1.0, 3.0e38, 1.17549435e-38, 16777215.0, 1.0 + 2.0 ** -23], np.float32)])
    hi = _bf16_rn(x)
    r1 = (x - hi).astype(np.float32)
    assert np.array_equal(r1.astype(np.float64), x.astype(np.float64) - hi.astype(np.float64))   # exact remainder
    mid = _bf16_rn(r1)
    r2 = (r1 - mid).astype(np.float32)
    assert np.array_equal(r2.astype(np.float64), r1.astype(np.float64) - mid.astype(np.float64))
    lo = _bf16_rn(r2)
    assert np.array_equal(hi.astype(np.float64) + mid.astype(np.float64) + lo.astype(np.float64), x.astype(np.float64))
