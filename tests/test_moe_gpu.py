"""GPU parity of the MoE block (decode and chunked prefill) against the CPU oracle."""
import numpy as np
import pytest

from helpers import SEED, check_block, make_layer, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(orc):
    """A small model with both headline formats: layer 0 IQ3_XXS, layer 1 Q4_K (Zipf bias,
    shared-expert gate row), layer 2 Q6_K experts with a Q8_0 down projection."""
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    e, ff, ne, k = 512, 256, 32, 4
    assert c.moe_config(3, e, ff, ne, k)
    layers = [
        make_layer(orc, c, 0, orc.IQ3_XXS, e, ff, ne, k),
        make_layer(orc, c, 1, orc.Q4_K, e, ff, ne, k, bias=True, gate_row=True),
        make_layer(orc, c, 2, orc.Q6_K, e, ff, ne, k, ty_down=orc.Q8_0, shared=False),
    ]
    yield c, layers
    c.close()


@pytest.mark.parametrize("layer", [0, 1, 2])
@pytest.mark.parametrize("nt", [1, 2, 3, 5, 8, 33])
def test_block_small(orc, small, layer, nt):
    c, layers = small
    L = layers[layer]
    h = orc.synth_normal(SEED, 900 + nt, 1.0, nt * L.e).reshape(nt, L.e)
    out, sels, wts = c.moe_block(layer, h, want_routing=True)
    err, redo = check_block(orc, L, h, out, sels, wts)
    assert err <= 1e-3, "layer %d nt %d: %.3g" % (layer, nt, err)
    assert redo == 0
    out2 = c.moe_block(layer, h)
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32)), "not bit-identical run to run"


def test_batch_equals_token_by_token(orc, small):
    """qwen4exp.rs:28259 (batch prefill == sequential).  A token's routing never depends
    on its neighbours; its values agree across chunk sizes and kernel families (one-token
    decode kernels, tiled fp32 kernels, tcgen05 grouped GEMM) to rounding, and are
    bit-identical when the same kernels run (fp32 tiled path, any chunk composition)."""
    c, layers = small
    nt = 21
    for layer in (0, 1):
        h = orc.synth_normal(SEED, 950 + layer, 1.0, nt * layers[layer].e).reshape(nt, -1)
        batch, bsel, bw = c.moe_block(layer, h, want_routing=True)
        for t in (0, 7, 20):
            pair = c.moe_block(layer, h[[t, (t + 1) % nt]])
            assert rel_err(pair[0], batch[t]) <= 5e-4
            one, osel, ow = c.moe_block(layer, h[t:t + 1], want_routing=True)
            assert np.array_equal(osel[0], bsel[t]) and np.array_equal(ow[0].view(np.uint32), bw[t].view(np.uint32))
            assert rel_err(one[0], batch[t]) <= 5e-4
    h = orc.synth_normal(SEED, 952, 1.0, nt * layers[0].e).reshape(nt, -1)
    batch = c.moe_block(0, h[:13])  # IQ3_XXS layer, 13 and 4 tokens: the decode kernels over one-row segments both times
    sub = c.moe_block(0, h[[5, 3, 12, 11]])
    assert np.array_equal(sub.view(np.uint32), batch[[5, 3, 12, 11]].view(np.uint32))
    big = c.moe_block(0, np.concatenate([h, h]))  # 42 and 21 tokens: the tiled fp32 kernels both times
    assert np.array_equal(big[:nt].view(np.uint32), c.moe_block(0, h).view(np.uint32))


@pytest.mark.parametrize("int_weights", [True, False])
def test_tcgen05_grouped_gemm_matches_fp32_kernels(orc, small, int_weights):
    """Q4_K prefill chunks on the tensor cores, both kernels: scales folded into bf16 hi / lo weights (three MMAs per
    product, the default), and integer fp16 weights sc * q with the block scales applied after the sum.
    The result must stay at fp32-kernel accuracy, far inside the 1e-3 bar, for ragged chunk sizes that
    exercise every N tile width, one and several token tiles per expert and tiles with one token."""
    c, layers = small
    L = layers[1]
    c.set_q4k_int(int_weights)
    try:
        for nt in (16, 17, 33, 40, 100, 130, 300):
            h = orc.synth_normal(SEED, 1300 + nt, 1.0, nt * L.e).reshape(nt, L.e)
            tc, tsel, tw = c.moe_block(1, h, want_routing=True)
            c.set_gemv_impl(2)
            try:
                fp = c.moe_block(1, h)
            finally:
                c.set_gemv_impl(0)
            print("nt=%d tcgen05 (%s) vs fp32 kernels: %.3g" % (nt, "integer" if int_weights else "bf16 x 3", rel_err(tc, fp)))
            assert rel_err(tc, fp) <= 5e-4, "nt=%d: tcgen05 vs fp32 kernels %.3g" % (nt, rel_err(tc, fp))
            idx = sorted({0, nt // 3, nt - 1})
            err, _ = check_block(orc, L, h[idx], tc[idx], tsel[idx], tw[idx])
            assert err <= 5e-4, "nt=%d: %.3g vs oracle" % (nt, err)
            again = c.moe_block(1, h)
            assert np.array_equal(tc.view(np.uint32), again.view(np.uint32)), "tcgen05 path not bit-identical run to run"
        assert c.device_status() == 0
    finally:
        c.set_q4k_int(False)


def test_exact_weight_tcgen05_kernel_matches_fp32_kernels(orc, small):
    """IQ3_XXS chunks and decode batches from the threshold up (lowered to 2 here): exact bf16 weights on the tensor cores, sub-block scales
    applied by the epilogue.  Ragged sizes cover one and several 32-token tiles per expert and tiles with one token;
    a batch's rows do not depend on their companions."""
    c, layers = small
    L = layers[0]
    c.set_tc_min_tokens(2)
    try:
        for nt in (2, 3, 4, 7, 31, 32, 33, 100, 300):
            h = orc.synth_normal(SEED, 1400 + nt, 1.0, nt * L.e).reshape(nt, L.e)
            tc, tsel, tw = c.moe_block(0, h, want_routing=True)
            c.set_gemv_impl(2)
            try:
                fp = c.moe_block(0, h)
            finally:
                c.set_gemv_impl(0)
            print("nt=%d exact-weight tcgen05 vs fp32 kernels: %.3g" % (nt, rel_err(tc, fp)))
            assert rel_err(tc, fp) <= 2e-4, "nt=%d: %.3g" % (nt, rel_err(tc, fp))
            idx = sorted({0, nt // 3, nt - 1})
            err, _ = check_block(orc, L, h[idx], tc[idx], tsel[idx], tw[idx])
            assert err <= 2e-4, "nt=%d: %.3g vs oracle" % (nt, err)
            again = c.moe_block(0, h)
            assert np.array_equal(tc.view(np.uint32), again.view(np.uint32)), "not bit-identical run to run"
            if nt >= 8:
                part = c.moe_block(0, h[nt // 2:])
                assert np.array_equal(part.view(np.uint32), tc[nt // 2:].view(np.uint32)), "a row depends on its companions"
    finally:
        c.set_tc_min_tokens(16)
    # the default threshold: 15 tokens stay on the one-token kernels, 16 take the tensor cores; both within the bar
    for nt in (15, 16):
        h = orc.synth_normal(SEED, 1450 + nt, 1.0, nt * L.e).reshape(nt, L.e)
        tc, tsel, tw = c.moe_block(0, h, want_routing=True)
        err, _ = check_block(orc, L, h[:4], tc[:4], tsel[:4], tw[:4])
        assert err <= 2e-4, "nt=%d: %.3g vs oracle" % (nt, err)
    assert c.device_status() == 0


def test_decode_kernels_agree_with_tiled_kernels(orc, small):
    """One-token calls take the bulk-copy GEMV + fused router kernels; the general
    tiled kernels (set_gemv_impl(2) forces them) must route identically and agree in
    value to rounding."""
    c, layers = small
    for layer in (0, 1, 2):
        h = orc.synth_normal(SEED, 960 + layer, 1.0, layers[layer].e)
        fast = c.moe_block(layer, h, want_routing=True)
        c.set_gemv_impl(2)
        try:
            tiled = c.moe_block(layer, h, want_routing=True)
        finally:
            c.set_gemv_impl(0)
        assert np.array_equal(fast[1], tiled[1])
        assert np.array_equal(fast[2].view(np.uint32), tiled[2].view(np.uint32))
        assert rel_err(fast[0], tiled[0]) <= 2e-5
    assert c.device_status() == 0


def test_graph_replay_gives_the_same_bits(orc, small):
    """The block and stack entry points replay a captured CUDA graph from their third
    call on; replays, direct launches and different inputs through the same graph must
    all give the bits of the first call."""
    c, layers = small
    e = layers[0].e
    for nt in (1, 6):
        h1 = orc.synth_normal(SEED, 1100 + nt, 1.0, nt * e).reshape(nt, e)
        h2 = orc.synth_normal(SEED, 1200 + nt, 1.0, nt * e).reshape(nt, e)
        first = [c.moe_block(0, h).copy() for h in (h1, h2)]
        for _ in range(3):
            for h, want in zip((h1, h2), first):
                assert np.array_equal(c.moe_block(0, h).view(np.uint32), want.view(np.uint32))
        c.use_graphs(False)
        try:
            assert np.array_equal(c.moe_block(0, h1).view(np.uint32), first[0].view(np.uint32))
        finally:
            c.use_graphs(True)
        s1 = c.moe_stack(h1)
        for _ in range(3):
            assert np.array_equal(c.moe_stack(h1).view(np.uint32), s1.view(np.uint32))
    assert c.device_status() == 0


def test_experts_with_given_selection(orc, small):
    """cuda.rs:8088 moe_seg_layer_sum: selection and weights supplied by the caller."""
    from denno_beta_b200 import _lib, cuda as cu

    c, layers = small
    L = layers[1]
    nt = 4
    x = orc.synth_normal(SEED, 970, 1.0, nt * L.e).reshape(nt, L.e)
    sels = np.array([[0, 1, 2, 3], [5, 9, 17, 31], [0, 10, 20, 30], [28, 29, 30, 31]], np.int32)
    wts = np.abs(orc.synth_normal(SEED, 971, 1.0, nt * L.k)).reshape(nt, L.k).astype(np.float32)
    got = cu.moe_seg_layer_sum(c, 1, sels, wts, x)
    want = orc.moe_experts_given(L, x, sels, wts)
    assert rel_err(got, want) <= 1e-3
    with pytest.raises(_lib.DnbError):  # not ascending: misuse (cuda.rs:8120-8126 returns Err)
        c.moe_experts(1, x, sels[:, ::-1], wts)


def test_router_topk(orc, small):
    from denno_beta_b200 import cuda as cu

    c, layers = small
    L = layers[1]
    nt = 64
    x = orc.synth_normal(SEED, 980, 1.0, nt * L.e).reshape(nt, L.e)
    sels, wts, rowsum = cu.pf_router_dev_topk(c, 1, x)
    osels, owts, probs = orc.router(x, L.keep["router_w"], L.keep["router_bias"], L.k)
    assert np.array_equal(sels, osels)
    assert np.all(np.diff(sels, axis=1) > 0)
    assert np.max(np.abs(wts - owts)) < 2e-6
    want_rowsum = np.take_along_axis(probs, osels, 1).sum(1)
    assert np.max(np.abs(rowsum - want_rowsum)) < 2e-6


def test_grouped_gemm(orc, small):
    from denno_beta_b200 import _lib, cuda as cu

    c, layers = small
    L = layers[1]
    segs = np.array([[3, 9, 0, 0], [0, 4, 9, 9], [31, 1, 13, 13], [7, 2, 14, 14]], np.uint32)
    m_total = 16
    xs = orc.synth_normal(SEED, 990, 1.0, m_total * L.e).reshape(m_total, L.e)
    got = cu.moe_grouped_gemm_layer(c, 1, cu.GATE, segs, xs, L.ff)
    want = orc.grouped_gemm(orc.Q4_K, L.keep["gate"], L.e, L.ff, segs, xs)
    assert rel_err(got, want) <= 2e-5
    bad = segs.copy()
    bad[2, 2] = 12  # gap in x_off: moe_expert.rs:8399-8440 check_segments rejects it
    with pytest.raises(_lib.DnbError):
        c.grouped_gemm(1, cu.GATE, bad, xs, L.ff)


@pytest.fixture(scope="module")
def config1(orc):
    """Benchmark config 1 at full size: e 2048, ff 512, 512 experts, top-10 + shared, IQ3_XXS."""
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    assert c.moe_config(1, 2048, 512, 512, 10)
    L = make_layer(orc, c, 0, orc.IQ3_XXS, 2048, 512, 512, 10)
    yield c, L
    c.close()


@pytest.mark.parametrize("impl", [0, 5, 4, 3])
def test_config1_decode(orc, config1, impl):
    """One token of config 1 through each family of one-token kernels: 0 = the whole block (router,
    gate/up, down, two grid barriers) as one mma.sync kernel; 5 = the router as a kernel of its own
    in front of the fused gate/up + down kernel; 4 = the mma.sync gate/up kernel and the down kernel
    as two launches; 3 = the register-decode kernels.  Each against the oracle, bit-identical
    run to run, with and without the residual of the stack entry point."""
    c, L = config1
    c.set_gemv_impl(impl)
    try:
        for seed in (2000, 2001, 2002):
            h = orc.synth_normal(SEED, seed, 1.0, 2048)
            out, sels, wts = c.moe_block(0, h, want_routing=True)
            err, redo = check_block(orc, L, h.reshape(1, -1), out, sels, wts)
            print("impl %d seed %d: %.3g" % (impl, seed, err))
            assert err <= 1e-3 and redo == 0
            for _ in range(3):  # the third call replays the captured graph
                out2 = c.moe_block(0, h)
                assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
            stack = c.moe_stack(h.reshape(1, -1))
            assert rel_err(stack, (h + out).astype(np.float32).reshape(1, -1)) <= 1e-6
        assert c.device_status() == 0
    finally:
        c.set_gemv_impl(0)


@pytest.mark.parametrize("shape", [(1024, 512, 32, 4, True), (2048, 1024, 16, 2, False), (1024, 512, 64, 10, True)])
def test_fused_decode_other_shapes(orc, shape):
    """The fused one-token kernel away from config 1: fewer down units than CTAs, an odd and an
    even number of segments, two 256-blocks per K half, the most segments 148 SMs take at ff 512."""
    from denno_beta_b200 import cuda as cu

    e, ff, ne, k, shared = shape
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        L = make_layer(orc, c, 0, orc.IQ3_XXS, e, ff, ne, k, shared=shared)
        for seed in (2300, 2301):
            h = orc.synth_normal(SEED, seed, 1.0, e)
            out, sels, wts = c.moe_block(0, h, want_routing=True)
            err, _ = check_block(orc, L, h.reshape(1, -1), out, sels, wts)
            assert err <= 1e-3, "%r seed %d: %.3g" % (shape, seed, err)
            c.set_gemv_impl(3)
            try:
                ref = c.moe_block(0, h)
            finally:
                c.set_gemv_impl(0)
            assert rel_err(out, ref) <= 2e-5
            launches = c.launch_count()
            c.moe_block(0, h)
            # stage-in + the one-kernel block; a shape whose shared memory leaves no room for the router
            # phase (ff 1024) keeps the router as a kernel of its own in front of the fused kernel
            assert c.launch_count() - launches == (3 if ff == 1024 else 2)
            c.set_gemv_impl(5)
            try:
                split = c.moe_block(0, h, want_routing=True)
            finally:
                c.set_gemv_impl(0)
            # the router inside the block kernel and the router kernel give the same routing bits
            assert np.array_equal(split[1], sels) and np.array_equal(split[2].view(np.uint32), wts.view(np.uint32))
            assert np.array_equal(split[0].view(np.uint32), out.view(np.uint32))
        assert c.device_status() == 0
    finally:
        c.close()


def test_config1_batches(orc, config1):
    c, L = config1
    for nt in (8, 32):
        h = orc.synth_normal(SEED, 2100 + nt, 1.0, nt * 2048).reshape(nt, 2048)
        out, sels, wts = c.moe_block(0, h, want_routing=True)
        idx = [0, nt // 2, nt - 1]
        err, _ = check_block(orc, L, h[idx], out[idx], sels[idx], wts[idx])
        assert err <= 1e-3


@pytest.fixture(scope="module")
def config2(orc):
    """Benchmark config 2 at full size: the same block with Q4_K experts and a Zipf router bias."""
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    assert c.moe_config(1, 2048, 512, 512, 10)
    L = make_layer(orc, c, 0, orc.Q4_K, 2048, 512, 512, 10, bias=True)
    yield c, L
    c.close()


def test_config2_prefill_chunk(orc, config2):
    c, L = config2
    nt = 512
    h = orc.synth_normal(SEED, 3000, 1.0, nt * 2048).reshape(nt, 2048)
    out, sels, wts = c.moe_block(0, h, want_routing=True)
    # Zipf skew: some experts see > 100 tokens, most see 0-2
    counts = np.bincount(sels.ravel(), minlength=512)
    assert counts.max() > 100 and np.median(counts) <= 2
    # oracle on a sample of tokens (each token's result is independent of the others)
    idx = np.array([0, 1, 17, 100, 255, 256, 300, 511])
    err, redo = check_block(orc, L, h[idx], out[idx], sels[idx], wts[idx])
    assert err <= 1e-3, err
    # routing of the whole chunk against the oracle's router
    x = orc.rmsnorm(h, np.ones(2048, np.float32))
    osels, _, _ = orc.router(x, L.keep["router_w"], L.keep["router_bias"], 10)
    assert np.mean(np.any(osels != sels, axis=1)) <= 0.01
    # chunk vs the one-token decode kernels: same routing, values equal to rounding
    for t in (3, 200, 511):
        one, osel, _ = c.moe_block(0, h[t:t + 1], want_routing=True)
        assert np.array_equal(osel[0], sels[t])
        assert rel_err(one[0], out[t]) <= 5e-4
    # ragged tail chunk (14,018 = 27 x 512 + 194)
    out194 = c.moe_block(0, h[:194])
    assert np.array_equal(out194.view(np.uint32), out[:194].view(np.uint32))


def test_stack_residual(orc, small):
    """identity mixers: h <- h + block_l(h), layers in order, device-resident in between."""
    c, layers = small
    nt = 3
    h = orc.synth_normal(SEED, 4000, 1.0, nt * 512).reshape(nt, 512)
    got = c.moe_stack(h)
    ref = h.copy()
    for L in layers:
        o, _, _ = orc.moe_block(L, ref)
        ref = (ref + o).astype(np.float32)
    assert rel_err(got, ref) <= 1e-3


def test_synth_device_equals_host(orc, small):
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, 512, 256, 8, 2)
        for ty in (orc.Q4_K, orc.IQ3_XXS, orc.Q6_K, orc.Q8_0):
            assert c.synth_experts(0, cu.GATE, ty, 512, 256, 8, 1234)
            nb = 8 * 256 * 512 // orc.blck_size(ty)
            host = orc.synth_blocks(ty, 1234, 0, nb)
            eb = host.size // 8
            for ex in (0, 7):
                dev = c.download_expert(0, cu.GATE, ex, eb)
                assert np.array_equal(dev, host[ex * eb:(ex + 1) * eb]), "type %d expert %d" % (ty, ex)
    finally:
        c.close()


def test_router_topk_ties_and_many_survivors(orc):
    """The selection rule on exact ties (larger value first, ties to the lower index) in the
    shapes the top-k kernel treats differently: a few tied rows (threshold shortcut), every
    row tied (more than 32 candidates reach the threshold: selection rounds), and one clear
    winner among ties.  Selections and weights must equal the CPU rule's."""
    from denno_beta_b200 import cuda as cu

    e, ne, k, nt = 256, 128, 6, 9
    x = orc.synth_normal(SEED, 991, 1.0, nt * e).reshape(nt, e)
    base = orc.synth_normal(SEED, 992, 0.05, ne * e).reshape(ne, e)
    cases = {}
    w = base.copy()
    w[40] = w[7]; w[90] = w[7]; w[91] = w[12]            # small groups of exactly equal logits
    cases["few ties"] = w
    cases["all tied"] = np.repeat(base[:1], ne, axis=0)   # 128 equal probabilities
    w = np.repeat(base[:1], ne, axis=0)
    w[77] = base[1] * 4.0
    cases["one winner"] = w
    for name, w in cases.items():
        c = cu.CudaCtx(0)
        try:
            assert c.moe_config(1, e, 256, ne, k)
            c.register_router(0, w, None, None, None)
            sels, wts, _ = c.router_topk(0, x)
            osels, owts, _ = orc.router(x, w, None, k)
            assert np.array_equal(sels, osels), name
            assert np.max(np.abs(wts - owts)) < 2e-6, name
        finally:
            c.close()


@pytest.mark.parametrize("nt", [1, 4, 40])
def test_block_remaining_gguf_formats(orc, nt):
    """The block types real checkpoints use for their other tensors (IQ4_XS / IQ3_S,
    IQ4_NL / IQ2_S, Q4_0 / Q2_0 as gate+up / down): decode, a small batch and a chunk."""
    from denno_beta_b200 import cuda as cu

    e, ff, ne, k = 512, 256, 16, 3
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(3, e, ff, ne, k)
        layers = [make_layer(orc, c, 0, orc.IQ4_XS, e, ff, ne, k, ty_down=orc.IQ3_S, bias=True),
                  make_layer(orc, c, 1, orc.IQ4_NL, e, ff, ne, k, ty_down=orc.IQ2_S, gate_row=True),
                  make_layer(orc, c, 2, orc.Q4_0, e, ff, ne, k, ty_down=orc.Q2_0, shared=False)]
        for li, L in enumerate(layers):
            h = orc.synth_normal(SEED, 1200 + 10 * li + nt, 1.0, nt * e).reshape(nt, e)
            out, sels, wts = c.moe_block(li, h, want_routing=True)
            err, redo = check_block(orc, L, h, out, sels, wts)
            assert err <= 1e-3 and redo == 0, "layer %d nt %d: %.3g" % (li, nt, err)
            assert np.array_equal(out.view(np.uint32), c.moe_block(li, h).view(np.uint32))
        assert c.device_status() == 0
    finally:
        c.close()
