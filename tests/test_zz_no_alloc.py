"""The allocation-free router entry point against the regular one, through the C ABI.

Some users of the library cannot allocate while they run -- a serving loop that fixed
its memory budget at start-up, a host application that bans cudaMalloc on the inference
thread because it stalls the whole device, code inside a stream capture.  For them
dnb_router_topk_static keeps its intermediate logits in a fixed array inside the
library.  This test drives it with caller-owned device buffers, twice in a row with
different inputs (the second call reuses the array the first one wrote), and requires
the selections to be identical and the weights bit-identical to dnb_router_topk; it
also checks that a call larger than the array is refused.  The file sorts last so a
run that stops at the first failure has already executed every other test."""
import numpy as np
import pytest

from helpers import SEED, make_layer

pytestmark = pytest.mark.gpu


def test_static_router_matches_regular_router_twice(orc):
    from denno_beta_b200 import _lib, cuda as cu

    c = cu.CudaCtx(0)
    try:
        e, ff, ne, k = 512, 256, 64, 6
        assert c.moe_config(1, e, ff, ne, k)
        make_layer(orc, c, 0, orc.Q4_K, e, ff, ne, k, bias=True)
        nt_max = 96
        d_x = c.dev_alloc(nt_max * e * 4)
        d_sels = c.dev_alloc(nt_max * k * 4)
        d_wts = c.dev_alloc(nt_max * k * 4)
        d_sum = c.dev_alloc(nt_max * 4)
        for call, nt in enumerate((96, 17)):
            x = orc.synth_normal(SEED, 6000 + call, 1.0, nt * e).reshape(nt, e)
            want_sels, want_wts, want_sum = c.router_topk(0, x)
            c.upload(d_x, x)
            assert c.router_topk_static(0, d_x, nt, d_sels, d_wts, d_sum)
            c.sync()
            sels = c.download(d_sels, np.empty((nt, k), np.int32))
            wts = c.download(d_wts, np.empty((nt, k), np.float32))
            rowsum = c.download(d_sum, np.empty(nt, np.float32))
            assert np.array_equal(sels, want_sels), "call %d: selections differ" % call
            assert np.array_equal(wts.view(np.uint32), want_wts.view(np.uint32)), "call %d: weights differ" % call
            assert np.array_equal(rowsum.view(np.uint32), want_sum.view(np.uint32))
            # and both agree with the CPU oracle's router
            osels, owts, _ = orc.router(x, orc.synth_normal(SEED, 6, 0.02, ne * e).reshape(ne, e),
                                        orc.synth_zipf_bias(SEED, 7, 1.1, ne), k)
            assert np.array_equal(sels, osels) and np.max(np.abs(wts - owts)) < 2e-6
        # rowsum is optional
        assert c.router_topk_static(0, d_x, 17, d_sels, d_wts, None)
        c.sync()
        # 65536 logits is the limit: 1025 tokens x 64 experts does not fit and is refused outright
        with pytest.raises(_lib.DnbError) as ei:
            c.router_topk_static(0, d_x, 1025, d_sels, d_wts, d_sum)
        assert ei.value.code == _lib.ERR_ARG and "static scratch" in str(ei.value)
        for p in (d_x, d_sels, d_wts, d_sum):
            c.dev_free(p)
    finally:
        c.close()


def _n_gpus():
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_static_router_on_a_second_device_after_the_first(orc):
    """Two contexts in one process, one per GPU.  The entry point must select its own context's
    device on every call: here it runs on GPU 1 right after GPU 0's context was used (so the
    calling thread's current device is 0), and again on GPU 0 after GPU 1."""
    from denno_beta_b200 import cuda as cu

    e, ff, ne, k, nt = 512, 256, 64, 6, 33
    ctxs = [cu.CudaCtx(0), cu.CudaCtx(1)]
    try:
        bufs = []
        for c in ctxs:
            assert c.moe_config(1, e, ff, ne, k)
            make_layer(orc, c, 0, orc.Q4_K, e, ff, ne, k, bias=True)
            bufs.append([c.dev_alloc(nt * e * 4), c.dev_alloc(nt * k * 4), c.dev_alloc(nt * k * 4)])
        x = orc.synth_normal(SEED, 6100, 1.0, nt * e).reshape(nt, e)
        want_sels, want_wts, _ = ctxs[0].router_topk(0, x)  # leaves device 0 current
        for order in ((1, 0), (0, 1)):
            for d in order:
                c, (d_x, d_sels, d_wts) = ctxs[d], bufs[d]
                c.upload(d_x, x)
                ctxs[1 - d].sync()  # the other context's call makes ITS device the current one
                assert c.router_topk_static(0, d_x, nt, d_sels, d_wts, None)
                assert c.sync()
                sels = c.download(d_sels, np.empty((nt, k), np.int32))
                wts = c.download(d_wts, np.empty((nt, k), np.float32))
                assert np.array_equal(sels, want_sels), "device %d" % d
                assert np.array_equal(wts.view(np.uint32), want_wts.view(np.uint32)), "device %d" % d
    finally:
        for c in ctxs:
            c.close()
