"""Expert-parallel exchange: host logic on CPU ranks (gloo, world size 2 and 4), and the
full path on real GPUs when at least two are present.  Ranks run as child processes
(tests/ep_ranks.py)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run_ranks(kind, world, port, timeout):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_ranks.py"), kind, str(r), str(world), str(port)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out))
    assert all(rc == 0 for rc, _ in outs), "\n".join(o[-3000:] for _, o in outs)
    return outs


@pytest.mark.parametrize("world", [2, 4])
def test_dispatch_and_return_on_cpu_ranks(world):
    _run_ranks("cpu", world, 29600 + world, 300)


def test_plan_is_stable_and_grouped():
    import torch

    from denno_beta_b200 import ep

    sels = torch.tensor([[0, 5, 6], [1, 2, 7], [4, 5, 6]], dtype=torch.int32)
    perm, counts, local = ep.plan_dispatch(sels, 4)  # ranks: experts 0-3 -> 0, 4-7 -> 1
    assert counts.tolist()[:2] == [3, 6]
    assert perm.tolist() == [0, 3, 4, 1, 2, 5, 6, 7, 8]      # (token, slot) order kept inside a rank
    assert local.tolist() == [0, 1, 2, 1, 2, 3, 0, 1, 2]


def _n_gpus():
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.gpu
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_equals_single_gpu():
    """Each rank holds half of the experts and its own 40 tokens; the block output must
    equal the single-GPU block on the same tokens (the combine order is the same), be
    bit-identical run to run, and no bounded wait may have given up."""
    outs = _run_ranks("gpu", 2, 29650, 900)
    for _, o in outs:
        print(o[-600:])


@pytest.mark.gpu
@pytest.mark.parametrize("ty_name", ["Q4_K", "IQ3_XXS"])
def test_peer_memory_path_on_one_gpu(ty_name):
    """World of one: the dispatch, the tables, the down epilogue's row destinations and the
    flags all run against the rank's own arena.  The block must equal the ordinary
    single-GPU block bit for bit (Q4_K: three-product tcgen05 kernel; IQ3_XXS: exact-weight kernel)."""
    import numpy as np

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED, make_layer

    e, ff, ne, k, nt = 512, 256, 32, 4, 50
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        make_layer(orc, c, 0, getattr(orc, ty_name), e, ff, ne, k, bias=True, gate_row=True)
        h = orc.synth_normal(SEED, 7702, 1.0, nt * e).reshape(nt, e)
        want = c.moe_block(0, h)
        pm = ep.PeerMemoryExpertParallel(c, max_tokens=64, rank=0, world=1)
        d_h, d_o = c.dev_alloc(h.nbytes), c.dev_alloc(h.nbytes)
        c.upload(d_h, h)
        for _ in range(2):
            pm.block_dev(0, d_h, nt, d_o)
            c.sync()
            got = c.download(d_o, np.empty((nt, e), np.float32))
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert c.device_status() == 0
    finally:
        c.close()


@pytest.mark.gpu
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_peer_memory_expert_parallel_equals_single_gpu():
    outs = _run_ranks("gpu_p2p", 2, 29660, 900)
    for _, o in outs:
        print(o[-600:])


@pytest.mark.gpu
@pytest.mark.parametrize("ty_name", ["IQ3_XXS", "Q4_K"])
def test_decode_exchange_on_one_gpu(ty_name):
    """Expert-parallel decode with a world of one: tables, push, flag wait and combine all run against
    the rank's own arena.  Batches of 1, 5 and 16 tokens take the decode GEMV kernels, 33 the tiled
    kernels; each must agree with the ordinary single-GPU block to rounding (the kernels differ), be
    bit-identical run to run, and the stack entry point must equal the layer-by-layer sum."""
    import numpy as np

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED, make_layer, rel_err

    ty = orc.TYPE_BY_NAME[ty_name]
    e, ff, ne, k = 512, 256, 32, 4
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(2, e, ff, ne, k)
        make_layer(orc, c, 0, ty, e, ff, ne, k, bias=True, gate_row=True)
        make_layer(orc, c, 1, ty, e, ff, ne, k)
        pd = ep.PeerMemoryDecode(c, max_tokens=40, rank=0, world=1)
        for nt in (1, 5, 16, 33):
            h = orc.synth_normal(SEED, 7800 + nt, 1.0, nt * e).reshape(nt, e)
            want = c.moe_block(0, h)
            d_h, d_o = c.dev_alloc(h.nbytes), c.dev_alloc(h.nbytes)
            c.upload(d_h, h)
            outs = []
            for _ in range(2):
                pd.block_dev(0, d_h, nt, d_o)
                assert c.sync()
                outs.append(c.download(d_o, np.empty((nt, e), np.float32)))
            assert rel_err(outs[0], want) <= 5e-4, "nt %d: %.3g" % (nt, rel_err(outs[0], want))
            assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
            ref = h.copy()
            for l in range(2):
                c.upload(d_h, ref)
                pd.block_dev(l, d_h, nt, d_o)
                assert c.sync()
                ref = (ref + c.download(d_o, np.empty((nt, e), np.float32))).astype(np.float32)
            c.upload(d_h, h)
            pd.stack_dev(d_h, nt)
            assert c.sync()
            got = c.download(d_h, np.empty((nt, e), np.float32))
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), "stack vs layer by layer, nt %d" % nt
            c.dev_free(d_h)
            c.dev_free(d_o)
        assert c.device_status() == 0
    finally:
        c.close()


@pytest.mark.gpu
def test_decode_exchange_waits_for_an_absent_rank_and_gives_up():
    """A group of two ranks of which only rank 0 exists: the wait for rank 1's rows runs out (status 24),
    the call returns, dnb_sync reports DECLINED, the output buffer is untouched, the context stays usable."""
    import numpy as np

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED

    e, ff, ne, k, nt = 512, 256, 32, 4, 3
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        nl = ne // 2
        c.set_expert_shard(0, nl)
        for m, (ni, no, n) in ((cu.GATE, (e, ff, nl)), (cu.UP, (e, ff, nl)), (cu.DOWN, (ff, e, nl)),
                               (cu.SHARED_GATE, (e, ff, 1)), (cu.SHARED_UP, (e, ff, 1)), (cu.SHARED_DOWN, (ff, e, 1))):
            assert c.synth_experts(0, m, orc.IQ3_XXS, ni, no, n, SEED)
        c.register_router(0, orc.synth_normal(SEED, 6, 0.02, ne * e), None, np.ones(e, np.float32), None)
        pd = ep.PeerMemoryDecode(c, max_tokens=8, rank=0, world=2, loopback=True)
        c.set_wait_limits(flag_polls=3000)
        h = orc.synth_normal(SEED, 7810, 1.0, nt * e).reshape(nt, e)
        d_h, d_o = c.dev_alloc(h.nbytes), c.dev_alloc(h.nbytes)
        c.upload(d_h, h)
        c.upload(d_o, np.full((nt, e), 3.5, np.float32))
        pd.block_dev(0, d_h, nt, d_o)
        assert c.sync() is False
        assert c.device_status() == 24
        assert np.all(c.download(d_o, np.empty((nt, e), np.float32)) == 3.5), "a call that gave up must not write its output"
        c.clear_status()
        assert c.sync() is True
        c.dev_free(d_h)
        c.dev_free(d_o)
    finally:
        c.close()


@pytest.mark.gpu
@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_decode_exchange_two_gpus_equals_one():
    outs = _run_ranks("gpu_epd", 2, 29670, 900)
    for _, o in outs:
        print(o[-600:])
