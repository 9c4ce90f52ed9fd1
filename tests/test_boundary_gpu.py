"""Boundary behaviour on the GPU: waits that run out are reported (never a hang, never a
silent stale result), the legacy three-launch entry points, the standalone router GEMV, the
grouped GEMM entry point on both kernel families and the device-built routing tables.

The time-out cases make a wait run out on purpose without faulting anything: a barrier target
that nothing can reach, and a group of two ranks of which one does not exist.  Both waits are
given a limit of a few thousand polls first, so the kernels return within milliseconds."""
import ctypes as C

import numpy as np
import pytest

from helpers import SEED, make_layer, rel_err

pytestmark = pytest.mark.gpu


def test_grid_barrier_that_runs_out_declines_and_leaves_out_untouched(orc):
    """cuda.rs:21024-21027 / 8785-8788: a call that did not complete returns "false" and leaves
    `out` alone.  The fused one-token kernel is given a barrier target one arrival beyond what
    its grid can deliver: every CTA gives up after its poll limit, records status 23 and skips
    the down phase.  The call must report DECLINED, must not touch the caller's buffer, and the
    context must go on working (on the two-launch form, which has no inter-CTA wait)."""
    from denno_beta_b200 import _lib, cuda as cu

    e, ff, ne, k = 1024, 512, 32, 4
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        L = make_layer(orc, c, 0, orc.IQ3_XXS, e, ff, ne, k)
        h = orc.synth_normal(SEED, 8801, 1.0, e).reshape(1, e)
        want = c.moe_block(0, h)
        n0 = c.launch_count()
        c.moe_block(0, h)
        assert c.launch_count() - n0 == 2, "the one-kernel block should be in use"
        c.set_wait_limits(barrier_polls=4000, barrier_bias=1)
        out = np.full((1, e), 7.25, np.float32)
        assert c.moe_block_into(0, h, out) is False
        assert "status 23" in _lib.last_error()
        assert np.all(out == 7.25), "a declined call must not write the caller's buffer"
        assert c.device_status() == 0, "the entry point clears the word after reporting it"
        c.set_wait_limits()  # defaults, no bias
        again = c.moe_block(0, h)
        assert again is not None and rel_err(again, want) <= 2e-5
        n0 = c.launch_count()
        c.moe_block(0, h)
        assert c.launch_count() - n0 == 4, "after a barrier time-out the context uses the two-launch form"
        err = rel_err(again, orc.moe_block(L, h)[0])
        assert err <= 1e-3
    finally:
        c.close()


def test_expert_parallel_wait_for_an_absent_rank_runs_out(orc):
    """A group of two ranks in which rank 1 never runs (every peer pointer is rank 0's own arena):
    the waits for rank 1's counts, rows and results run out, the block call returns, the status
    word names the wait, dnb_sync reports DECLINED until the word is cleared, and the context is
    still usable afterwards."""
    from denno_beta_b200 import _lib, cuda as cu

    e, ff, ne, k, nt = 512, 256, 32, 4, 24
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        nl = ne // 2
        c.set_expert_shard(0, nl)
        for m, (ni, no, n) in ((cu.GATE, (e, ff, nl)), (cu.UP, (e, ff, nl)), (cu.DOWN, (ff, e, nl)),
                               (cu.SHARED_GATE, (e, ff, 1)), (cu.SHARED_UP, (e, ff, 1)), (cu.SHARED_DOWN, (ff, e, 1))):
            assert c.synth_experts(0, m, orc.Q4_K, ni, no, n, SEED)
        c.register_router(0, orc.synth_normal(SEED, 6, 0.02, ne * e), None, np.ones(e, np.float32), None)
        handle = np.zeros(64, np.uint8)
        _lib.check(c.lib.dnb_ep_init(c.h, 0, 2, 64, C.c_void_p(handle.ctypes.data)))
        _lib.check(c.lib.dnb_ep_connect_loopback(c.h))
        c.set_wait_limits(flag_polls=3000)
        h = orc.synth_normal(SEED, 8802, 1.0, nt * e).reshape(nt, e)
        d_h, d_o = c.dev_alloc(h.nbytes), c.dev_alloc(h.nbytes)
        c.upload(d_h, h)
        _lib.check(c.lib.dnb_ep_block_dev(c.h, 0, C.c_void_p(d_h), nt, C.c_void_p(d_o)))
        assert c.sync() is False, "a wait that ran out must not look like success"
        assert c.device_status() in (21, 22)
        c.clear_status()
        assert c.device_status() == 0 and c.sync() is True
        sels, wts, _ = c.router_topk(0, orc.rmsnorm(h, np.ones(e, np.float32)))  # the context still works
        assert sels.shape == (nt, k)
        c.dev_free(d_h)
        c.dev_free(d_o)
    finally:
        c.close()


@pytest.fixture(scope="module")
def q4k_layer(orc):
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    e, ff, ne, k = 512, 256, 32, 4
    assert c.moe_config(1, e, ff, ne, k)
    L = make_layer(orc, c, 0, orc.Q4_K, e, ff, ne, k, bias=True)
    yield c, L
    c.close()


def test_legacy_three_launch_form(orc, q4k_layer):
    """cuda.rs:7638 moe_gemv_seg_pair + host silu + cuda.rs:7689 moe_gemv_seg_one: the tables of
    expert_batch.rs:143-170 (gate/up share x, down reads one activation row per segment); the
    host-side SwiGLU and weighted sum then give the block's routed half."""
    from denno_beta_b200 import _lib, cuda as cu

    c, L = q4k_layer
    e, ff, k = L.e, L.ff, L.k
    ids = [3, 9, 17, 30]
    x = orc.synth_normal(SEED, 8810, 1.0, e)
    seg_gu = np.array([[ex, 1, 0, s * ff] for s, ex in enumerate(ids)], np.uint32)
    seg_dn = np.array([[ex, 1, s * ff, s * e] for s, ex in enumerate(ids)], np.uint32)
    g = np.zeros(k * ff, np.float32)
    u = np.zeros(k * ff, np.float32)
    assert cu.moe_gemv_seg_pair(c, 0, seg_gu, x, g, u)
    gb, db = L.keep["gate"].size // L.ne, L.keep["down"].size // L.ne
    for s, ex in enumerate(ids):
        wg = orc.gemv_scalar(orc.Q4_K, L.keep["gate"][ex * gb:(ex + 1) * gb], e, ff, x)
        wu = orc.gemv_scalar(orc.Q4_K, L.keep["up"][ex * gb:(ex + 1) * gb], e, ff, x)
        assert rel_err(g[s * ff:(s + 1) * ff], wg) <= 2e-5 and rel_err(u[s * ff:(s + 1) * ff], wu) <= 2e-5
    act = (g / (1.0 + np.exp(-g.astype(np.float64))) * u).astype(np.float32)
    hrows = np.zeros(k * e, np.float32)
    assert cu.moe_gemv_seg_one(c, 0, seg_dn, act, hrows)
    for s, ex in enumerate(ids):
        wd = orc.gemv_scalar(orc.Q4_K, L.keep["down"][ex * db:(ex + 1) * db], ff, e, act[s * ff:(s + 1) * ff])
        assert rel_err(hrows[s * e:(s + 1) * e], wd) <= 2e-5
    # two tokens in one segment (m = 2) take the tiled kernel
    x2 = orc.synth_normal(SEED, 8811, 1.0, 2 * e)
    out2 = np.zeros(2 * ff, np.float32)
    assert c.seg_gemv(0, cu.GATE, np.array([[5, 2, 0, 0]], np.uint32), x2, out2)
    for t in range(2):
        want = orc.gemv_scalar(orc.Q4_K, L.keep["gate"][5 * gb:6 * gb], e, ff, x2[t * e:(t + 1) * e])
        assert rel_err(out2[t * ff:(t + 1) * ff], want) <= 2e-5
    # a segment that reaches beyond the buffers is refused (expert_batch.rs:233-260 seg_extents)
    with pytest.raises(_lib.DnbError):
        c.seg_gemv(0, cu.GATE, np.array([[5, 3, 0, 0]], np.uint32), x2, out2)
    with pytest.raises(_lib.DnbError):
        c.seg_gemv(0, cu.GATE, np.array([[5, 0, 0, 0]], np.uint32), x2, out2)  # m = 0


def test_router_gemv_alone(orc, q4k_layer):
    from denno_beta_b200 import cuda as cu

    c, L = q4k_layer
    nt = 5
    x = orc.synth_normal(SEED, 8820, 1.0, nt * L.e).reshape(nt, L.e)
    out = np.empty((nt, L.ne), np.float32)
    assert cu.maybe_gpu_router_gemv_into(c, 0, x, out)
    want = x.astype(np.float64) @ L.keep["router_w"].reshape(L.ne, L.e).astype(np.float64).T + L.keep["router_bias"]
    assert np.max(np.abs(out - want)) <= 1e-5 * np.max(np.abs(want))
    again = c.router_gemv(0, x)
    assert np.array_equal(out.view(np.uint32), again.view(np.uint32))


@pytest.mark.parametrize("e,ne,nt", [(2048, 512, 512), (2048, 512, 300), (512, 128, 128), (1024, 132, 257), (2048, 512, 16), (2048, 512, 40)])
def test_router_logits_on_tensor_cores(orc, e, ne, nt):
    """cuda.rs:48695 pf_router_dev_topk: the router of a chunk.  From 16 tokens the logits come from the tcgen05
    kernel (three bf16 parts per operand, six products).  They must be as close to the exact sum as the fp32 FMA
    kernel's are, the top-k built on them must be the CPU router's, and two runs must agree bit for bit.  Shapes:
    full tiles, ragged token tiles down to the smallest call, the smallest expert count, and an expert count that is no
    multiple of 128.  A token's logits must not depend on what else is in the call."""
    from denno_beta_b200 import cuda as cu

    k = 8
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, 256, ne, k)
        rw = orc.synth_normal(SEED, 8830, 0.02, ne * e).reshape(ne, e)
        rb = orc.synth_zipf_bias(SEED, 8831, 1.1, ne)
        c.register_router(0, rw, rb, None, None)
        x = orc.synth_normal(SEED, 8832, 1.0, nt * e).reshape(nt, e)
        want = x.astype(np.float64) @ rw.astype(np.float64).T + rb
        n0 = c.launch_count()
        tc = c.router_gemv(0, x)
        assert c.launch_count() - n0 >= 2, "split + tensor-core GEMM (+ reduce)"
        assert np.array_equal(tc.view(np.uint32), c.router_gemv(0, x).view(np.uint32))
        c.set_router_tc(False)
        n0 = c.launch_count()
        fp = c.router_gemv(0, x)
        assert c.launch_count() - n0 == 1
        c.set_router_tc(True)
        err_tc, err_fp = np.max(np.abs(tc - want)), np.max(np.abs(fp - want))
        scale = np.max(np.abs(want))
        print("router logits max|err|: tcgen05 %.3g  fp32 FMA %.3g  (max|logit| %.3g)" % (err_tc, err_fp, scale))
        assert err_tc <= max(2.0 * err_fp, 4e-7 * scale)
        if nt >= 32:  # the same rows in a smaller call (another tile occupancy): the same bits
            part = c.router_gemv(0, x[5:5 + 16])
            assert np.array_equal(part.view(np.uint32), tc[5:5 + 16].view(np.uint32))
        sels, wts, _ = c.router_topk(0, x)
        osel, owts, _ = orc.router(x, rw, rb, k)
        assert np.array_equal(sels, osel)
        assert np.max(np.abs(wts - owts)) <= 2e-6
    finally:
        c.close()


def test_grouped_gemm_entry_point_on_tcgen05(orc, q4k_layer):
    """cuda.rs:7065 moe_grouped_gemm_layer with enough rows for the tensor-core kernel: ragged
    segments (one above 128 tokens, one single row) on the gate matrix (K = n_embd) and the down
    matrix (K = n_ff), against the CPU grouped GEMM and against the fp32 tiled kernel."""
    from denno_beta_b200 import cuda as cu

    c, L = q4k_layer
    segs = np.array([[3, 70, 0, 0], [0, 130, 70, 70], [31, 1, 200, 200], [7, 17, 201, 201]], np.uint32)
    m_total = 218
    for matrix, n_in, n_out, key in ((cu.GATE, L.e, L.ff, "gate"), (cu.DOWN, L.ff, L.e, "down")):
        xs = orc.synth_normal(SEED, 8830 + matrix, 1.0, m_total * n_in).reshape(m_total, n_in)
        n0 = c.launch_count()
        got = cu.moe_grouped_gemm_layer(c, 0, matrix, segs, xs, n_out)
        assert c.launch_count() - n0 == 2, "operand split + tcgen05 grouped GEMM expected"
        want = orc.grouped_gemm(orc.Q4_K, L.keep[key], n_in, n_out, segs, xs)
        assert rel_err(got, want) <= 5e-4
        c.set_gemv_impl(2)
        try:
            tiled = cu.moe_grouped_gemm_layer(c, 0, matrix, segs, xs, n_out)
        finally:
            c.set_gemv_impl(0)
        assert rel_err(tiled, want) <= 2e-5 and rel_err(got, tiled) <= 5e-4
        assert np.array_equal(got.view(np.uint32), c.grouped_gemm(0, matrix, segs, xs, n_out).view(np.uint32))
    assert c.device_status() == 0


@pytest.mark.parametrize("shape", [(300, 4, 32, 0.0), (512, 10, 512, 1.1), (194, 10, 512, 1.1), (7, 3, 16, 0.0), (90, 1, 16, 0.0),
                                   (33, 1, 8, 0.0), (65, 2, 8, 1.1)])
def test_routing_tables_equal_build_grouped_batch(orc, shape):
    """moe_expert.rs:8309-8390: segments by token count descending, ties by expert ascending; the
    rows of an expert in ascending token order.  The device-built table (route_tables_kernel) must
    equal the CPU construction entry for entry.  The shapes include one selection per token (the rows an
    expert-parallel rank receives) and expert counts that fit one CTA of the kernel."""
    from denno_beta_b200 import cuda as cu

    nt, k, ne, zipf = shape
    rng = np.random.default_rng(nt * 131 + k)
    p = None
    if zipf:
        p = 1.0 / np.arange(1, ne + 1) ** zipf
        p = rng.permutation(p / p.sum())
    sels = np.stack([np.sort(rng.choice(ne, size=k, replace=False, p=p)) for _ in range(nt)]).astype(np.int32)
    c = cu.CudaCtx(0)
    try:
        e, ff = 256, 256
        assert c.moe_config(1, e, ff, ne, k)
        for m, (ni, no) in ((cu.GATE, (e, ff)), (cu.UP, (e, ff)), (cu.DOWN, (ff, e))):
            assert c.synth_experts(0, m, orc.Q8_0, ni, no, ne, SEED)
        segs, rtok, pos = c.build_grouped_batch(0, sels)
        osegs, ortok, orslot = orc.build_segments(sels, ne)
        assert np.array_equal(segs, osegs)
        assert np.array_equal(rtok, ortok)
        # pos[t][slot] is the inverse of (row_token, row_slot)
        for row in range(nt * k):
            assert pos[ortok[row], orslot[row]] == row
        counts = np.bincount(sels.ravel(), minlength=ne)
        assert segs.shape[0] == int((counts > 0).sum())
        assert np.all(np.diff(segs[:, 1].astype(np.int64)) <= 0)
    finally:
        c.close()
