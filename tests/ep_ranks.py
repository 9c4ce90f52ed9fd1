"""Rank workers of the expert-parallel tests: `python ep_ranks.py cpu|gpu RANK WORLD PORT`.
Each exits 0 when its checks pass."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _init(rank, world, port, backend):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend, rank=rank, world_size=world)


def cpu_rank(rank, world, port):
    """Each rank owns 7 tokens; the fake expert e maps a row x to x * (e + 1) + e."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from denno_beta_b200 import ep

    _init(rank, world, port, "gloo")
    try:
        ne, k, e, nt = 8, 3, 5, 7
        n_local = ne // world
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(nt, e, generator=g)
        sels = torch.stack([torch.sort(torch.randperm(ne, generator=g)[:k]).values for _ in range(nt)]).to(torch.int32)
        wts = torch.rand(nt, k, generator=g)
        recv_x, recv_ids, state = ep.dispatch(x, sels, n_local)
        # rows arrive grouped by source rank; every id is local to this rank
        assert recv_ids.numel() == recv_x.shape[0]
        assert recv_ids.numel() == 0 or (int(recv_ids.min()) >= 0 and int(recv_ids.max()) < n_local)
        gid = recv_ids.to(torch.float32) + rank * n_local
        h_rows = recv_x * (gid + 1).unsqueeze(1) + gid.unsqueeze(1)
        h_slots = ep.gather_back(h_rows, state)
        out = (h_slots.reshape(nt, k, e) * wts.unsqueeze(2)).sum(1)
        ge = sels.to(torch.float32)
        want = ((x.unsqueeze(1) * (ge + 1).unsqueeze(2) + ge.unsqueeze(2)) * wts.unsqueeze(2)).sum(1)
        ok = bool(torch.allclose(out, want, rtol=0, atol=1e-6))
        total = torch.tensor([recv_x.shape[0]])
        dist.all_reduce(total)
        assert ok, "rank %d: combined output differs" % rank
        assert int(total) == world * nt * k
    finally:
        dist.destroy_process_group()


def gpu_rank(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED, make_layer, rel_err

    torch.cuda.set_device(rank)
    _init(rank, world, port, "nccl")
    try:
        e, ff, ne, k, nt = 512, 256, 32, 4, 40
        results = {}
        for layer_ty in (orc.Q4_K, orc.IQ3_XXS):
            # reference on this rank: the whole model on one GPU, all tokens
            full = cu.CudaCtx(rank)
            assert full.moe_config(1, e, ff, ne, k)
            L = make_layer(orc, full, 0, layer_ty, e, ff, ne, k, bias=True, gate_row=True)
            h_all = orc.synth_normal(SEED, 7700, 1.0, world * nt * e).reshape(world * nt, e)
            want = full.moe_block(0, h_all)[rank * nt:(rank + 1) * nt]
            full.close()
            # expert-parallel: this rank's shard
            c = cu.CudaCtx(rank)
            assert c.moe_config(1, e, ff, ne, k)
            nl = ne // world
            c.set_expert_shard(rank * nl, nl)
            kp = L.keep
            gb, db = kp["gate"].size // ne, kp["down"].size // ne
            sl = slice(rank * nl * gb, (rank + 1) * nl * gb)
            sd = slice(rank * nl * db, (rank + 1) * nl * db)
            assert c.register_experts(0, cu.GATE, layer_ty, e, ff, nl, kp["gate"][sl])
            assert c.register_experts(0, cu.UP, layer_ty, e, ff, nl, kp["up"][sl])
            assert c.register_experts(0, cu.DOWN, layer_ty, ff, e, nl, kp["down"][sd])
            assert c.register_experts(0, cu.SHARED_GATE, layer_ty, e, ff, 1, kp["sg"])
            assert c.register_experts(0, cu.SHARED_UP, layer_ty, e, ff, 1, kp["su"])
            assert c.register_experts(0, cu.SHARED_DOWN, layer_ty, ff, e, 1, kp["sd"])
            c.register_router(0, kp["router_w"], kp["router_bias"], kp["norm_w"], kp["sgr"])
            blk = ep.ExpertParallelBlock(c, e, ne, k)
            h = torch.from_numpy(h_all[rank * nt:(rank + 1) * nt].copy()).cuda()
            out1 = blk.block(0, h).cpu().numpy()
            out2 = blk.block(0, h).cpu().numpy()
            results[int(layer_ty)] = (rel_err(out1, want), bool(np.array_equal(out1.view(np.uint32), out2.view(np.uint32))),
                                      c.device_status())
            torch.cuda.synchronize()
            c.close()
        for ty, (err, same, status) in results.items():
            print("rank %d type %d: err %.3g bit-identical %s status %d" % (rank, ty, err, same, status), flush=True)
            assert err <= 5e-4 and same and status == 0
    finally:
        dist.destroy_process_group()


def gpu_p2p_rank(rank, world, port):
    """Peer-memory expert parallel (dnb_ep_*): each rank holds ne/world experts and its own
    tokens; the output must equal the single-GPU block bit for bit, twice."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED, make_layer, rel_err

    torch.cuda.set_device(rank)
    _init(rank, world, port, "nccl")
    try:
        e, ff, ne, k, nt = 512, 256, 32, 4, 40 + 3 * rank  # ragged: the ranks own different token counts
        starts = [sum(40 + 3 * r for r in range(q)) for q in range(world + 1)]
        full = cu.CudaCtx(rank)
        assert full.moe_config(1, e, ff, ne, k)
        L = make_layer(orc, full, 0, orc.Q4_K, e, ff, ne, k, bias=True, gate_row=True)
        h_all = orc.synth_normal(SEED, 7701, 1.0, starts[world] * e).reshape(starts[world], e)
        want = full.moe_block(0, h_all)[starts[rank]:starts[rank + 1]]
        full.close()
        c = cu.CudaCtx(rank)
        assert c.moe_config(1, e, ff, ne, k)
        nl = ne // world
        c.set_expert_shard(rank * nl, nl)
        kp = L.keep
        gb, db = kp["gate"].size // ne, kp["down"].size // ne
        sl = slice(rank * nl * gb, (rank + 1) * nl * gb)
        sd = slice(rank * nl * db, (rank + 1) * nl * db)
        assert c.register_experts(0, cu.GATE, orc.Q4_K, e, ff, nl, kp["gate"][sl])
        assert c.register_experts(0, cu.UP, orc.Q4_K, e, ff, nl, kp["up"][sl])
        assert c.register_experts(0, cu.DOWN, orc.Q4_K, ff, e, nl, kp["down"][sd])
        assert c.register_experts(0, cu.SHARED_GATE, orc.Q4_K, e, ff, 1, kp["sg"])
        assert c.register_experts(0, cu.SHARED_UP, orc.Q4_K, e, ff, 1, kp["su"])
        assert c.register_experts(0, cu.SHARED_DOWN, orc.Q4_K, ff, e, 1, kp["sd"])
        c.register_router(0, kp["router_w"], kp["router_bias"], kp["norm_w"], kp["sgr"])
        pm = ep.PeerMemoryExpertParallel(c, max_tokens=64)
        h = np.ascontiguousarray(h_all[starts[rank]:starts[rank + 1]])
        d_h, d_o = c.dev_alloc(h.nbytes), c.dev_alloc(h.nbytes)
        c.upload(d_h, h)
        outs = []
        for _ in range(3):
            pm.block_dev(0, d_h, nt, d_o)
            c.sync()
            outs.append(c.download(d_o, np.empty((nt, e), np.float32)))
        status = c.device_status()
        dist.barrier()  # nobody tears its arena down while a peer may still store into it
        err = rel_err(outs[0], want)
        same_as_one_gpu = bool(np.array_equal(outs[0].view(np.uint32), want.view(np.uint32)))
        repeat = all(np.array_equal(outs[0].view(np.uint32), o.view(np.uint32)) for o in outs[1:])
        print("rank %d p2p: err %.3g equals-single-gpu %s repeatable %s status %d" % (rank, err, same_as_one_gpu, repeat, status),
              flush=True)
        assert status == 0 and repeat and err <= 5e-4 and same_as_one_gpu
        c.close()
    finally:
        dist.destroy_process_group()


def gpu_epd_rank(rank, world, port):
    """Expert-parallel decode (dnb_epd_*): every rank holds ne/world experts and ALL tokens of the batch.
    For batches of 1, 8 and 32 tokens and a two-layer stack the result must be the same bits on every
    rank, the same bits as the same exchange run with a world of one (all experts on this GPU), and
    agree with the ordinary single-GPU block to rounding."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle as orc
    from denno_beta_b200 import cuda as cu, ep
    from helpers import SEED, make_layer, rel_err

    torch.cuda.set_device(rank)
    _init(rank, world, port, "nccl")
    try:
        e, ff, ne, k = 512, 256, 32, 4
        for ty in (orc.IQ3_XXS, orc.Q4_K):
            full = cu.CudaCtx(rank)
            assert full.moe_config(2, e, ff, ne, k)
            Ls = [make_layer(orc, full, 0, ty, e, ff, ne, k, bias=True, gate_row=True), make_layer(orc, full, 1, ty, e, ff, ne, k)]
            one = ep.PeerMemoryDecode(full, max_tokens=32, rank=0, world=1)
            c = cu.CudaCtx(rank)
            assert c.moe_config(2, e, ff, ne, k)
            nl = ne // world
            c.set_expert_shard(rank * nl, nl)
            for l, L in enumerate(Ls):
                kp = L.keep
                gb, db = kp["gate"].size // ne, kp["down"].size // ne
                sl = slice(rank * nl * gb, (rank + 1) * nl * gb)
                sd = slice(rank * nl * db, (rank + 1) * nl * db)
                assert c.register_experts(l, cu.GATE, ty, e, ff, nl, kp["gate"][sl])
                assert c.register_experts(l, cu.UP, ty, e, ff, nl, kp["up"][sl])
                assert c.register_experts(l, cu.DOWN, ty, ff, e, nl, kp["down"][sd])
                assert c.register_experts(l, cu.SHARED_GATE, ty, e, ff, 1, kp["sg"])
                assert c.register_experts(l, cu.SHARED_UP, ty, e, ff, 1, kp["su"])
                assert c.register_experts(l, cu.SHARED_DOWN, ty, ff, e, 1, kp["sd"])
                c.register_router(l, kp["router_w"], kp["router_bias"], kp["norm_w"], kp["sgr"])
            pd = ep.PeerMemoryDecode(c, max_tokens=32)
            for nt in (1, 8, 32):
                h = orc.synth_normal(SEED, 7820 + nt, 1.0, nt * e).reshape(nt, e)
                want = full.moe_block(0, h)
                bufs = {}
                for name, ctx_, pd_ in (("one", full, one), ("ep", c, pd)):
                    d_h, d_o = ctx_.dev_alloc(h.nbytes), ctx_.dev_alloc(h.nbytes)
                    ctx_.upload(d_h, h)
                    pd_.block_dev(0, d_h, nt, d_o)
                    assert ctx_.sync()
                    blk = ctx_.download(d_o, np.empty((nt, e), np.float32))
                    pd_.stack_dev(d_h, nt)
                    assert ctx_.sync()
                    bufs[name] = (blk, ctx_.download(d_h, np.empty((nt, e), np.float32)))
                    ctx_.dev_free(d_h)
                    ctx_.dev_free(d_o)
                assert rel_err(bufs["ep"][0], want) <= 5e-4
                assert np.array_equal(bufs["ep"][0].view(np.uint32), bufs["one"][0].view(np.uint32)), "block differs from world 1"
                assert np.array_equal(bufs["ep"][1].view(np.uint32), bufs["one"][1].view(np.uint32)), "stack differs from world 1"
                t = torch.from_numpy(bufs["ep"][1].view(np.int32).astype(np.int64)).cuda()
                lo, hi = t.clone(), t.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                assert bool(torch.equal(lo, hi)), "ranks ended with different bits"
                print("rank %d type %d nt %d: err %.3g, same bits as world 1 and on every rank" % (rank, ty, nt, rel_err(bufs["ep"][0], want)), flush=True)
            assert c.device_status() == 0
            torch.cuda.synchronize()
            dist.barrier()  # nobody tears its arena down while a peer may still store into it
            c.close()
            full.close()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    kind, rank, world, port = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    {"cpu": cpu_rank, "gpu": gpu_rank, "gpu_p2p": gpu_p2p_rank, "gpu_epd": gpu_epd_rank}[kind](rank, world, port)
