"""The timed CPU baseline (oracle/dnb_cpu_fast.c: AVX2+FMA kernels in the form the reference runs in
production) against the sequential-order oracle.  The reference bounds its own fused kernels by
|fused - scalar| <= 1e-4 + 1e-5 * |scalar| per element (model/moe_expert.rs:8755-8758); the same
bound is applied here to the GEMVs, and the path's parity metric (max|d| / rms) to whole blocks."""
import numpy as np
import pytest

SEED = 0xD3770B200


@pytest.mark.parametrize("name", ["Q4_K", "IQ3_XXS", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("k,n", [(2048, 96), (512, 200)])
def test_fast_gemv_within_the_references_bound(orc, name, k, n):
    ty = orc.TYPE_BY_NAME[name]
    w = orc.synth_blocks(ty, SEED, 300 + ty, n * k // orc.blck_size(ty))
    x = orc.synth_normal(SEED, 301 + ty, 1.0, k)
    want = orc.gemv_scalar(ty, w, k, n, x)
    for threads in (1, 3):
        orc.set_threads(threads)
        got = orc.fast_gemv(ty, w, k, n, x)
        scale = max(1.0, float(np.sqrt(np.mean(want.astype(np.float64) ** 2))))  # the bound is stated for O(1) outputs
        assert np.all(np.abs(got - want) <= (1e-4 + 1e-5 * np.abs(want)) * scale), name
    orc.set_threads(0)


def _layer(orc, ty, e, ff, ne, k, bias):
    nb = lambda rows, cols: rows * cols // orc.blck_size(ty)
    gate = orc.synth_blocks(ty, SEED, 0, ne * nb(ff, e))
    up = orc.synth_blocks(ty, SEED, 1, ne * nb(ff, e))
    down = orc.synth_blocks(ty, SEED, 2, ne * nb(e, ff))
    sh = (orc.synth_blocks(ty, SEED, 3, nb(ff, e)), orc.synth_blocks(ty, SEED, 4, nb(ff, e)), orc.synth_blocks(ty, SEED, 5, nb(e, ff)))
    rw = orc.synth_normal(SEED, 6, 0.02, ne * e).reshape(ne, e)
    rb = orc.synth_zipf_bias(SEED, 7, 1.1, ne) if bias else None
    return orc.Layer(e, ff, ne, k, ty, ty, ty, gate, up, down, rw, router_bias=rb, norm_w=np.ones(e, np.float32), shared=sh)


@pytest.mark.parametrize("name", ["Q4_K", "IQ3_XXS", "Q6_K"])
def test_fast_block_matches_the_oracle(orc, name):
    ty = orc.TYPE_BY_NAME[name]
    e, ff, ne, k = 512, 256, 16, 3
    L = _layer(orc, ty, e, ff, ne, k, bias=(name == "Q4_K"))
    h = orc.synth_normal(SEED, 310, 1.0, 37 * e).reshape(37, e)
    want, _, _ = orc.moe_block(L, h)
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    orc.set_threads(4)
    try:
        one = orc.fast_moe_block(L, h[:5])
        assert np.max(np.abs(one - want[:5])) / rms <= 2e-5
        grouped = orc.fast_moe_block(L, h, grouped=True)
        assert np.max(np.abs(grouped - want)) / rms <= 2e-5
    finally:
        orc.set_threads(0)


def test_placed_zipf_bias_keeps_the_values_and_balances_contiguous_shards(orc):
    """bench.py's expert placement for the expert-parallel prefill lines: the same bias values on other expert
    indices, such that contiguous shards of 64 / 128 / 256 experts see about equal numbers of routed rows."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench

    rb = orc.synth_zipf_bias(bench.SEED, 7, 1.1, bench.NE)
    pb = bench.placed_zipf_bias(rb)
    assert sorted(pb.tolist()) == sorted(rb.tolist())
    assert np.array_equal(pb, bench.placed_zipf_bias(rb)), "placement is deterministic"
    nt = 256
    h = orc.synth_normal(bench.SEED, 8000, 1.0, nt * bench.E).reshape(nt, bench.E)
    rw = orc.synth_normal(bench.SEED, 6, 0.02, bench.NE * bench.E).reshape(bench.NE, bench.E)
    x = orc.rmsnorm(h, np.ones(bench.E, np.float32))
    worst = {}
    for name, b in (("seeded", rb), ("placed", pb)):
        counts = np.bincount(orc.router(x, rw, b, bench.K)[0].ravel(), minlength=bench.NE)
        worst[name] = {g: float(counts.reshape(g, -1).sum(1).max() / counts.reshape(g, -1).sum(1).mean()) for g in (2, 4, 8)}
    assert worst["placed"][8] <= 1.2 and worst["placed"][4] <= 1.12 and worst["placed"][2] <= 1.06, worst
    assert worst["seeded"][8] >= 1.5, worst
