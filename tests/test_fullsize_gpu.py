"""Parity at the benchmark configurations' full sizes.

config 0  one 4096 x 4096 GEMV in each block format of the path
config 2  one 512-token prefill chunk, Q4_K experts, Zipf router bias: EVERY token of the tensor-core
          path against the fp32 kernels, and an oracle sample that holds the hottest expert's tokens
          on the seams of its 128-token tiles
config 3  the 48-layer decode stack (40 IQ3_XXS + 8 Q4_K layers) at batch 1 / 8 / 32 and config 4's
          194-token tail chunk: per-layer parity with each tested layer fed the same input on both
          sides, the stack entry point against the layer-by-layer sum, bit identity run to run

The 48-layer model (32 GB) is generated on the device; the oracle gets, for a tested layer, only the
experts its tokens select (copied back from the device into an otherwise untouched host array)."""
import numpy as np
import pytest

from helpers import SEED, check_block, make_layer, rel_err

pytestmark = pytest.mark.gpu

E, FF, NE, K = 2048, 512, 512, 10


@pytest.mark.parametrize("name", ["IQ3_XXS", "Q6_K", "Q8_0"])
def test_config0_other_formats_4096(orc, name):
    """Benchmark config 0's shape in the path's other formats (Q4_K is in test_gemv_gpu.py)."""
    from denno_beta_b200 import cuda as cu

    ty = orc.TYPE_BY_NAME[name]
    n = k = 4096
    w = orc.synth_blocks(ty, SEED, 40 + ty, n * k // orc.blck_size(ty))
    x = orc.synth_normal(SEED, 1040 + ty, 1.0, k)
    want = orc.gemv_scalar(ty, w, k, n, x)
    out = np.empty(n, np.float32)
    assert cu.maybe_gpu_gguf_gemv_into(0xC0F000 + ty, ty, w, k, n, x, out)
    assert rel_err(out, want) <= 2e-5
    again = np.empty(n, np.float32)
    assert cu.maybe_gpu_gguf_gemv_into(0xC0F000 + ty, ty, w, k, n, x, again)
    assert np.array_equal(out.view(np.uint32), again.view(np.uint32))


@pytest.mark.parametrize("ty_name,seam", [("Q4_K", 128), ("IQ3_XXS", 32)])
def test_config2_every_token(orc, ty_name, seam):
    """Config 2 (Q4_K: three-product tcgen05 kernel, 128-token tiles) and the same chunk with IQ3_XXS experts
    (exact-weight tcgen05 kernel, 32-token tiles): every token against the fp32 kernels, a sample that covers the
    hottest expert's tile seams against the oracle."""
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, E, FF, NE, K)
        L = make_layer(orc, c, 0, getattr(orc, ty_name), E, FF, NE, K, bias=True)
        nt = 512
        h = orc.synth_normal(SEED, 3000, 1.0, nt * E).reshape(nt, E)
        n0 = c.launch_count()
        out, sels, wts = c.moe_block(0, h, want_routing=True)
        assert c.launch_count() - n0 == 8, "prep (RMSNorm + the router operand), router GEMM on tcgen05, top-k (adds the K splits), tables, gather, 2 x tcgen05, combine"
        c.set_gemv_impl(2)
        try:
            fp, fsels, fwts = c.moe_block(0, h, want_routing=True)
        finally:
            c.set_gemv_impl(0)
        assert np.array_equal(sels, fsels) and np.array_equal(wts.view(np.uint32), fwts.view(np.uint32))
        rms = float(np.sqrt(np.mean(fp.astype(np.float64) ** 2)))
        per_token = np.max(np.abs(out.astype(np.float64) - fp), axis=1) / rms
        assert per_token.max() <= 5e-4, "token %d: %.3g" % (int(per_token.argmax()), per_token.max())
        # oracle sample: the hottest expert's tokens on its tile seams (packed rows 0, 127, 128, 129, 255,
        # 256, ..., last), more of its tokens, and tokens spread over the chunk
        counts = np.bincount(sels.ravel(), minlength=NE)
        hot = int(counts.argmax())
        assert counts[hot] > 256, "the Zipf bias should give one expert several 128-token tiles"
        hot_tokens = np.nonzero(np.any(sels == hot, axis=1))[0]  # ascending = packed order inside the expert
        seams = [i for i in (0, 1, seam - 1, seam, seam + 1, 2 * seam - 1, 2 * seam, 2 * seam + 1, 3 * seam - 1, 3 * seam,
                             3 * seam + 1, len(hot_tokens) - 1) if i < len(hot_tokens)]
        pick = set(hot_tokens[seams].tolist()) | set(hot_tokens[::37].tolist())
        cold = np.nonzero(~np.any(sels == hot, axis=1))[0]
        pick |= set(cold.tolist()[:8])
        pick |= set(range(0, nt, 11))
        idx = np.array(sorted(pick))
        assert idx.size >= 64 and np.sum(np.any(sels[idx] == hot, axis=1)) >= 8
        err, redo = check_block(orc, L, h[idx], out[idx], sels[idx], wts[idx])
        assert err <= 1e-3 and redo <= 1, (err, redo)
        assert np.array_equal(out.view(np.uint32), c.moe_block(0, h).view(np.uint32))
        assert c.device_status() == 0
    finally:
        c.close()


def _sparse_oracle_layer(orc, cu, c, l, ty, router_w, sels_needed):
    """The oracle's view of layer l with only the experts in `sels_needed` filled in."""
    gb = FF * orc.row_bytes(ty, E)
    db = E * orc.row_bytes(ty, FF)
    gate, up, down = (np.zeros(NE * gb, np.uint8), np.zeros(NE * gb, np.uint8), np.zeros(NE * db, np.uint8))
    for ex in sorted(set(int(v) for v in np.asarray(sels_needed).ravel())):
        gate[ex * gb:(ex + 1) * gb] = c.download_expert(l, cu.GATE, ex, gb)
        up[ex * gb:(ex + 1) * gb] = c.download_expert(l, cu.UP, ex, gb)
        down[ex * db:(ex + 1) * db] = c.download_expert(l, cu.DOWN, ex, db)
    sh = (c.download_expert(l, cu.SHARED_GATE, 0, gb), c.download_expert(l, cu.SHARED_UP, 0, gb),
          c.download_expert(l, cu.SHARED_DOWN, 0, db))
    return orc.Layer(E, FF, NE, K, ty, ty, ty, gate, up, down, router_w, norm_w=np.ones(E, np.float32), shared=sh)


@pytest.fixture(scope="module")
def stack48(orc):
    """Config 3's model: 48 layers, every sixth Q4_K, the others IQ3_XXS; expert tables generated on the device."""
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    assert c.moe_config(48, E, FF, NE, K)
    types, routers = [], []
    for l in range(48):
        ty = orc.Q4_K if l % 6 == 5 else orc.IQ3_XXS
        types.append(ty)
        for m, (ni, no, n) in ((cu.GATE, (E, FF, NE)), (cu.UP, (E, FF, NE)), (cu.DOWN, (FF, E, NE)),
                               (cu.SHARED_GATE, (E, FF, 1)), (cu.SHARED_UP, (E, FF, 1)), (cu.SHARED_DOWN, (FF, E, 1))):
            assert c.synth_experts(l, m, ty, ni, no, n, SEED)
        rw = orc.synth_normal(SEED, l * 16 + 6, 0.02, NE * E).reshape(NE, E)
        routers.append(rw)
        c.register_router(l, rw, None, np.ones(E, np.float32), None)
    assert c.sync()
    yield c, types, routers
    c.close()


@pytest.mark.parametrize("nt", [1, 8, 32, 194])
def test_stack48_per_layer_parity(orc, stack48, nt):
    """Per-layer parity inside the 48-layer stack: the residual stream is advanced layer by layer
    through the block entry point, and at the tested layers (two IQ3_XXS, two Q4_K, first and last
    included) the block's output is compared with the oracle's on the SAME input.  Then the stack
    entry point (device-resident, residual add fused) against that layer-by-layer sum, twice."""
    from denno_beta_b200 import cuda as cu

    c, types, routers = stack48
    tested = (0, 5, 24, 47)
    h0 = orc.synth_normal(SEED, 8100 + nt, 1.0, nt * E).reshape(nt, E)
    h = h0.copy()
    sample = list(range(nt)) if nt <= 8 else sorted({0, 1, nt // 3, nt // 2, nt - 2, nt - 1})
    for l in range(48):
        out, sels, wts = c.moe_block(l, h, want_routing=True)
        assert out is not None
        if l in tested:
            idx = np.array(sample)
            L = _sparse_oracle_layer(orc, cu, c, l, types[l], routers[l], sels[idx])
            want, osels, owts = orc.moe_block(L, h[idx])
            same = np.all(osels == sels[idx], axis=1)
            assert same.mean() >= 0.8, "layer %d: routing differs on most sampled tokens" % l
            for n_, t in enumerate(idx):
                if not same[n_]:  # a tie within rounding: re-evaluate under the GPU's selection (its experts were fetched)
                    x = orc.rmsnorm(h[t:t + 1], np.ones(E, np.float32))
                    want[n_] = orc.moe_experts_given(L, x, sels[t:t + 1], wts[t:t + 1])[0]
            err = rel_err(out[idx], want)
            print("nt %d layer %d (type %d): %.3g, %d re-evaluated" % (nt, l, types[l], err, int((~same).sum())))
            assert err <= 1e-3, "nt %d layer %d: %.3g" % (nt, l, err)
        h = (h + out).astype(np.float32)
    s1 = c.moe_stack(h0)
    s2 = c.moe_stack(h0)
    assert np.array_equal(s1.view(np.uint32), s2.view(np.uint32)), "stack not bit-identical run to run"
    assert rel_err(s1, h) <= 1e-5, "stack entry point vs layer-by-layer: %.3g" % rel_err(s1, h)
    assert c.device_status() == 0
