"""Expert-parallel MoE block over several GPUs of one node.

The reference (denno-beta) is single-GPU.  On an 8 x B200 box the experts shard
naturally: rank g keeps experts [g*ne/G, (g+1)*ne/G) of every layer, the router, norm
and shared expert are replicated, and every rank owns its own tokens.  One block is

    route (local) -> dispatch all-to-all -> local experts -> return all-to-all -> combine

The exchange plan (which row goes where, in which order) is pure index arithmetic and
lives in `plan_dispatch`; it is the same on CPU tensors with gloo (tests) and on CUDA
tensors with NCCL.  The combine sums a token's slots in ascending expert index exactly
as the single-GPU path does, so the result does not depend on the number of ranks.

torch is used for device buffers, index shuffles and torch.distributed; the kernels are
the library's (route / expert rows / combine entry points of include/dnb200.h).
"""
import ctypes as C

import torch
import torch.distributed as dist


def plan_dispatch(sels, n_local):
    """sels: int tensor [nt, k] of global expert ids (ascending per token).

    Returns (perm, dest_counts, local_ids) where row j of the send buffer is the
    (token, slot) pair perm[j] = token*k + slot, rows are grouped by destination rank in
    ascending rank order and keep (token, slot) order inside a group (stable), and
    local_ids[j] is the expert's index on its destination rank."""
    flat = sels.reshape(-1).to(torch.int64)
    dest = torch.div(flat, n_local, rounding_mode="floor")
    perm = torch.sort(dest, stable=True).indices
    world = dist.get_world_size() if dist.is_initialized() else int(dest.max().item()) + 1
    dest_counts = torch.bincount(dest, minlength=world)
    local_ids = (flat - dest * n_local)[perm].to(torch.int32)
    return perm, dest_counts, local_ids


def exchange_counts(dest_counts):
    """All-to-all of the per-destination row counts -> rows this rank will receive per source."""
    recv = torch.empty_like(dest_counts)
    dist.all_to_all_single(recv, dest_counts)
    return recv


def dispatch(x, sels, n_local):
    """Send every (token, slot) row of x [nt, e] to the rank that owns its expert.

    Returns (recv_x [rows, e], recv_ids [rows] int32, state) where state carries what
    `gather_back` needs."""
    nt, k = sels.shape
    perm, dest_counts, local_ids = plan_dispatch(sels, n_local)
    send_counts = dest_counts.cpu().tolist()
    recv_counts = exchange_counts(dest_counts).cpu().tolist()
    send_x = x.index_select(0, torch.div(perm, k, rounding_mode="floor"))
    rows = int(sum(recv_counts))
    recv_x = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
    recv_ids = torch.empty((rows,), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_x, send_x, recv_counts, send_counts)
    dist.all_to_all_single(recv_ids, local_ids, recv_counts, send_counts)
    return recv_x, recv_ids, (perm, send_counts, recv_counts, nt * k)


def gather_back(h_rows, state):
    """Return the expert outputs to the ranks that own the tokens; row t*k+slot of the
    result is the output of token t's slot."""
    perm, send_counts, recv_counts, n = state
    ret = torch.empty((n, h_rows.shape[1]), dtype=h_rows.dtype, device=h_rows.device)
    dist.all_to_all_single(ret, h_rows, send_counts, recv_counts)
    h_slots = torch.empty_like(ret)
    h_slots.index_copy_(0, perm, ret)
    return h_slots


class ExpertParallelBlock:
    """One rank of an expert-parallel MoE model on its GPU.

    `ctx` is a CudaCtx whose model was configured with dnb_moe_config, then
    `set_expert_shard(rank * n_local, n_local)`, then the rank's n_local experts per layer
    (plus router, norm and shared expert, replicated)."""

    def __init__(self, ctx, n_embd, n_expert, k, rank=None, world=None):
        self.ctx = ctx
        self.e, self.ne, self.k = n_embd, n_expert, k
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        assert n_expert % self.world == 0, "experts must divide evenly over the ranks"
        self.n_local = n_expert // self.world
        self.dev = torch.device("cuda", ctx.device)
        # The library's kernels and torch's copies/collectives must share one stream.
        # torch's default stream has handle 0, which the library reads as "use your own
        # stream", so a dedicated torch stream is created and made current in block().
        self.stream = torch.cuda.Stream(device=self.dev)
        ctx.set_stream(self.stream.cuda_stream)

    def _p(self, t):
        return C.c_void_p(t.data_ptr())

    def route(self, layer, h):
        from ._lib import check

        nt = h.shape[0]
        x = torch.empty_like(h)
        sels = torch.empty((nt, self.k), dtype=torch.int32, device=self.dev)
        wts = torch.empty((nt, self.k), dtype=torch.float32, device=self.dev)
        check(self.ctx.lib.dnb_moe_route_dev(self.ctx.h, layer, self._p(h), nt, self._p(x), self._p(sels), self._p(wts)))
        return x, sels, wts

    def expert_rows(self, layer, x_rows, local_ids, shared=False):
        from ._lib import check

        rows = x_rows.shape[0]
        out = torch.empty_like(x_rows)
        if rows == 0:
            return out
        ids = None if shared else self._p(local_ids)
        check(self.ctx.lib.dnb_expert_rows_dev(self.ctx.h, layer, self._p(x_rows), ids, rows, 1 if shared else 0,
                                               self._p(out)))
        return out

    def combine(self, layer, h_slots, wts, shared, x):
        from ._lib import check

        nt = wts.shape[0]
        out = torch.empty((nt, self.e), dtype=torch.float32, device=self.dev)
        check(self.ctx.lib.dnb_moe_combine_dev(self.ctx.h, layer, self._p(h_slots), self._p(wts),
                                               None if shared is None else self._p(shared), self._p(x), nt, self._p(out)))
        return out

    def block(self, layer, h, has_shared=True):
        """h: this rank's tokens [nt, e] (fp32, on this rank's GPU) -> block output [nt, e]."""
        self.stream.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(self.stream):
            h = h.contiguous()
            x, sels, wts = self.route(layer, h)
            recv_x, recv_ids, state = dispatch(x, sels, self.n_local)
            sh = self.expert_rows(layer, x, None, shared=True) if has_shared else None
            h_rows = self.expert_rows(layer, recv_x.contiguous(), recv_ids)
            h_slots = gather_back(h_rows, state)
            out = self.combine(layer, h_slots, wts, sh, x)
        torch.cuda.current_stream(self.dev).wait_stream(self.stream)
        return out


class PeerMemoryExpertParallel:
    """One rank of an expert-parallel model whose ranks exchange rows through each other's
    memory (dnb_ep_* entry points): no collective between the kernels of a block and no
    host round trip.  torch.distributed is used once, to all-gather the 64-byte memory
    handles.  `ctx`: configured with dnb_moe_config, set_expert_shard(rank * n_local,
    n_local) and this rank's experts (router, norm, shared expert replicated)."""

    def __init__(self, ctx, max_tokens, rank=None, world=None, group=None):
        import numpy as np

        from ._lib import check

        self.ctx = ctx
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        handle = np.zeros(64, np.uint8)
        check(ctx.lib.dnb_ep_init(ctx.h, self.rank, self.world, max_tokens, C.c_void_p(handle.ctypes.data)))
        if self.world > 1:
            # the handles are plain bytes: gather them with whatever backend the group has
            dev = torch.device("cuda", ctx.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            mine = torch.from_numpy(handle).to(dev)
            got = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(got, mine, group=group)
            handles = np.concatenate([g.cpu().numpy() for g in got])
        else:
            handles = handle
        handles = np.ascontiguousarray(handles, np.uint8)
        check(ctx.lib.dnb_ep_connect(ctx.h, C.c_void_p(handles.ctypes.data)))
        if self.world > 1:
            dist.barrier(group=group)  # every arena is mapped before anyone stores into one

    def block_dev(self, layer, h_dev, nt, out_dev):
        """Device pointers (ints): h [nt][e] -> out [nt][e] for this rank's own tokens."""
        from ._lib import check

        check(self.ctx.lib.dnb_ep_block_dev(self.ctx.h, layer, C.c_void_p(h_dev), nt, C.c_void_p(out_dev)))

    def stack_dev(self, h_dev, nt):
        """All layers in place with identity mixers: h <- h + block_l(h) for this rank's nt tokens."""
        from ._lib import check

        check(self.ctx.lib.dnb_ep_stack_dev(self.ctx.h, C.c_void_p(h_dev), nt))


class PeerMemoryDecode:
    """One rank of an expert-parallel DECODE group (dnb_epd_* entry points): the residual stream is
    replicated, every rank computes the (token, slot) pairs of its own experts and stores the result
    rows into every rank's memory; one flag wait per layer.  `ctx`: configured with dnb_moe_config,
    set_expert_shard(rank * n_local, n_local) and this rank's experts (router, norm, shared expert
    replicated).  world == 1 needs no torch.distributed."""

    def __init__(self, ctx, max_tokens, rank=None, world=None, group=None, loopback=False):
        import numpy as np

        from ._lib import check

        self.ctx = ctx
        self.rank = (dist.get_rank() if rank is None else rank)
        self.world = (dist.get_world_size() if world is None else world)
        handle = np.zeros(64, np.uint8)
        check(ctx.lib.dnb_epd_init(ctx.h, self.rank, self.world, max_tokens, C.c_void_p(handle.ctypes.data)))
        if loopback:
            check(ctx.lib.dnb_epd_connect(ctx.h, None))
            return
        if self.world > 1:
            dev = torch.device("cuda", ctx.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            mine = torch.from_numpy(handle).to(dev)
            got = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(got, mine, group=group)
            handles = np.concatenate([g.cpu().numpy() for g in got])
        else:
            handles = handle
        handles = np.ascontiguousarray(handles, np.uint8)
        check(ctx.lib.dnb_epd_connect(ctx.h, C.c_void_p(handles.ctypes.data)))
        if self.world > 1:
            dist.barrier(group=group)  # every arena is mapped before anyone stores into one

    def block_dev(self, layer, h_dev, nt, out_dev):
        from ._lib import check

        check(self.ctx.lib.dnb_epd_block_dev(self.ctx.h, layer, C.c_void_p(h_dev), nt, C.c_void_p(out_dev)))

    def stack_dev(self, h_dev, nt):
        from ._lib import check

        check(self.ctx.lib.dnb_epd_stack_dev(self.ctx.h, C.c_void_p(h_dev), nt))
