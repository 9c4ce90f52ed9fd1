#!/usr/bin/env python3
"""Benchmark of the quantised-MoE expert path on B200 (one JSON line on stdout).

Headline workload (N=1): config 1 of the benchmark set -- one sparse-MoE block, decode, 1 token:
RMSNorm -> router (512 x 2048 fp32) -> softmax top-10 + renorm -> 10 routed + 1 shared
IQ3_XXS expert (gate/up 512x2048, down 2048x512) -> SwiGLU -> weighted sum.  A "step"
is one token through one block; the block rotates over LAYERS independent weight
copies (> L2) and over a pool of input vectors, so every step streams its weights
from HBM.

  value     steps/s with inputs and outputs resident in HBM (dnb_moe_block_dev)
  e2e       the same through dnb_moe_block with host buffers (H2D + D2H inside)
  roofline  the dominant kernel's algorithmic bytes / its mean launch time, both
            measured live with events around every launch (dnb_profile_*)
  cpu_baseline  the multi-threaded CPU port of the reference path on this box's cores

`--impl reference` times that CPU path alone (rank 0 only under torchrun).
With --gpus N > 1 every rank runs the same block on its own GPU and its own tokens
(weak scaling, no collective on the data path); value is the sum over ranks of
steps / max-over-ranks time.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 0xD3770B200
E, FF, NE, K = 2048, 512, 512, 10
IQ3_XXS, Q4_K = 18, 12
LAYERS = 16          # rotating weight copies: 16 x 17.4 MB touched per cycle > 126 MB L2
POOL = 64            # distinct input tokens
ROW_BYTES = {IQ3_XXS: {2048: 784, 512: 196}, Q4_K: {2048: 1152, 512: 288}}


def expert_bytes(ty):
    return FF * ROW_BYTES[ty][E], E * ROW_BYTES[ty][FF]


class Clocks:
    """Samples nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu, self.rows, self.p = gpu, [], None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.p = None

    def _read(self):
        for line in self.p.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.p:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def recorded_traffic():
    """DRAM bytes of one launch (read + write) per decode kernel on the headline workload: constants
    recorded from one profiler capture of each kernel, not measured in this run."""
    src = "recorded constant: dram__bytes_read.sum + dram__bytes_write.sum of one profiler capture of this kernel on this workload"
    return {k: {"dram_bytes": v, "source": src} for k, v in
            (("decode_block", 17587584), ("decode_gate_up_down", 13474560), ("gemv_gate_up", 8991744),
             ("gemv_down_combine", 4813568), ("router_decode_fused", 4275456))}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1677.1)), "measured"
    return 6650.0, 1590.0, "fallback"


def placed_zipf_bias(rb, shards=8):
    """The same Zipf bias values, assigned to expert indices so that contiguous shards of NE / shards experts
    carry about equal expected load (and so do unions of adjacent shards: 4 or 2 GPUs).  Expert placement by
    expected load, decided at load time from the router bias alone: experts are taken in descending bias
    (rank r, expected share of a chunk's tokens ~ 1 - exp(-5.5 (r + 1)^-1.1): the hottest experts are chosen by
    nearly every token, so their load saturates) and each goes to the least loaded shard that still has room.
    Which expert is hot is arbitrary in a synthetic model; a deployment would permute the expert tensors and
    the router rows the same way."""
    ne = rb.size
    order = np.argsort(-rb, kind="stable")          # expert indices by descending bias
    w = 1.0 - np.exp(-5.5 * (np.arange(ne) + 1.0) ** -1.1)
    cap = ne // shards
    load = np.zeros(shards)
    members = [[] for _ in range(shards)]
    for r in range(ne):
        free = [s_ for s_ in range(shards) if len(members[s_]) < cap]
        s_ = min(free, key=lambda q: (load[q], q))
        members[s_].append(r)
        load[s_] += w[r]
    out = np.empty_like(rb)
    vals = rb[order]
    for s_ in range(shards):
        for j, r in enumerate(members[s_]):
            out[s_ * cap + j] = vals[r]
    return out


def router_bias(oracle, l, bias):
    """bias: False = none, True = the seeded Zipf bias, "placed" = the same values placed by expected load."""
    if not bias:
        return None
    rb = oracle.synth_zipf_bias(SEED, l * 16 + 7, 1.1, NE)
    return placed_zipf_bias(rb) if bias == "placed" else rb


def build_model(ctx, cu, ty, layers, bias, ty_of_layer=None):
    """Expert tables filled on the device; routers (small) from the host generator."""
    import oracle  # only its seeded host generator is used here (inputs, not results)

    assert ctx.moe_config(layers, E, FF, NE, K)
    base_ty = ty
    for l in range(layers):
        ty = ty_of_layer(l) if ty_of_layer else base_ty
        assert ctx.synth_experts(l, cu.GATE, ty, E, FF, NE, SEED)
        assert ctx.synth_experts(l, cu.UP, ty, E, FF, NE, SEED)
        assert ctx.synth_experts(l, cu.DOWN, ty, FF, E, NE, SEED)
        assert ctx.synth_experts(l, cu.SHARED_GATE, ty, E, FF, 1, SEED)
        assert ctx.synth_experts(l, cu.SHARED_UP, ty, E, FF, 1, SEED)
        assert ctx.synth_experts(l, cu.SHARED_DOWN, ty, FF, E, 1, SEED)
        rw = oracle.synth_normal(SEED, l * 16 + 6, 0.02, NE * E)
        rb = router_bias(oracle, l, bias)
        ctx.register_router(l, rw, rb, np.ones(E, np.float32), None)
    ctx.sync()


def run_ours(args, rank, world, local_rank):
    import oracle
    from denno_beta_b200 import cuda as cu

    ctx = cu.CudaCtx(local_rank)
    if args.decode_impl:
        ctx.set_gemv_impl(args.decode_impl)
    build_model(ctx, cu, IQ3_XXS, LAYERS, False)
    pool = oracle.synth_normal(SEED, 7000 + rank, 1.0, POOL * E).reshape(POOL, E)
    d_pool = ctx.dev_alloc(pool.nbytes)
    d_out = ctx.dev_alloc(E * 4)
    ctx.upload(d_pool, pool)

    d_h = ctx.dev_alloc(E * 4)

    def dev_steps(s):
        """LAYERS steps with one call: a token enters block 0 and its residual stream
        passes through the LAYERS rotating blocks (h <- h + block_l(h)), all on the device."""
        ctx.dev_copy(d_h, d_pool + (s % POOL) * E * 4, E * 4)
        assert ctx.moe_stack_dev(d_h, 1)

    def dev_step(s):
        assert ctx.moe_block_dev(s % LAYERS, d_pool + (s % POOL) * E * 4, 1, d_out)

    out_host = np.empty((1, E), np.float32)
    h_ptrs = [cu.host_ptr(pool[i:i + 1]) for i in range(POOL)]  # host buffers named once, as a caller's staging buffers are
    out_ptr = cu.host_ptr(out_host)

    def host_step(s):
        assert ctx.moe_block_into(s % LAYERS, h_ptrs[s % POOL], out_ptr, 1)

    def barrier():
        ctx.sync()
        if world > 1:
            import torch.distributed as dist

            dist.barrier()

    # A step = one token through one block.  EXACTLY args.steps steps are timed per repeat: whole
    # passes of LAYERS blocks through the stack entry point plus the remaining blocks one by one.
    # The timed region is repeated (each repeat bracketed by a synchronisation, and a barrier at
    # N > 1) until it adds up to >= ~0.1 s; the reported time is the median repeat.
    K_, W_ = args.steps, max(args.warmup, 3)
    full, rem = divmod(K_, LAYERS)

    def k_steps(s0):
        for c_ in range(full):
            dev_steps(s0 + c_)
        for r_ in range(rem):
            ctx.dev_copy(d_h, d_pool + ((s0 + full + r_) % POOL) * E * 4, E * 4)
            assert ctx.moe_block_dev(r_ % LAYERS, d_h, 1, d_out)

    host_calls = 2 * (full + rem)
    for s in range(max(3, (W_ + K_ - 1) // K_)):  # >= 3 passes: direct, graph capture, replay
        k_steps(s)
    barrier()
    ctx.stall(1.0)
    ctx.timer_start()
    k_steps(0)
    est_ms = max(ctx.timer_stop(), 1e-3)
    repeats = int(min(2000, max(5, np.ceil(100.0 / est_ms))))
    stall_ms = min(20.0, 0.3 + 0.01 * host_calls)
    clocks = Clocks(local_rank)
    clocks.start()
    rep_ms = []
    launches = 0
    for r in range(repeats):
        barrier()
        ctx.stall(stall_ms)  # the K steps queue up behind it: no host launch gaps inside the event interval
        l0 = ctx.launch_count()
        ctx.timer_start()
        k_steps(r)
        rep_ms.append(ctx.timer_stop())
        launches = ctx.launch_count() - l0
    barrier()
    # end to end through the host-buffer entry point, one block per call
    for s in range(max(W_, 2 * LAYERS)):
        host_step(s)
    barrier()
    e2e_repeats = int(min(2000, max(5, np.ceil(100.0 / max(est_ms * 1.6, 1e-3)))))
    e2e_ms = []
    for r in range(e2e_repeats):
        barrier()
        t0 = time.perf_counter()
        for s in range(K_):
            host_step(W_ + r * K_ + s)
        ctx.sync()
        e2e_ms.append((time.perf_counter() - t0) * 1e3)
    clk = clocks.stop()
    barrier()
    status = ctx.device_status()
    assert status == 0, "a bounded device wait gave up during the timed region (status %d): the numbers are void" % status
    # per-kernel pass: events around every launch; each chunk is enqueued behind a
    # short GPU-side stall so the kernels run back to back and the event intervals
    # hold no host launch gaps
    ctx.profile(True)
    done = 0
    while done < 960:
        ctx.stall(8.0)
        for s in range(48):
            dev_step(W_ + done + s)
        ctx.sync()
        done += 48
    prof = ctx.profile_read()
    ctx.profile(False)

    rep_ms = np.asarray(rep_ms, np.float64)
    e2e_ms = np.asarray(e2e_ms, np.float64)
    if world > 1:
        import torch
        import torch.distributed as dist

        # max over ranks of every repeat, then the median repeat
        t = torch.tensor(np.concatenate([rep_ms, e2e_ms]), dtype=torch.float64, device="cuda:%d" % local_rank)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t = t.cpu().numpy()
        rep_ms, e2e_ms = t[:rep_ms.size], t[rep_ms.size:]
    ms_dev, ms_e2e = float(np.median(rep_ms)), float(np.median(e2e_ms))
    if world > 1:
        pass
    if world > 1 and ctx is not None:
        ctx.close()
        ctx = None
    if rank != 0:
        if world > 1 and not args.no_extras:
            guarded_ep_extras(None, cu, oracle, rank, world, local_rank)
        return None

    hbm_peak, _, peak_kind = peaks()
    g_b, d_b = expert_bytes(IQ3_XXS)
    alg = {  # algorithmic bytes per launch: weight bytes + activations in/out
        # gate/up + down of the block in one kernel: all expert rows once, x in, the block's result out
        # the whole block in one kernel: router rows, all expert rows once, the token row in, the result out
        "decode_block": NE * E * 4 + (K + 1) * (2 * g_b + d_b) + 2 * E * 4,
        "decode_gate_up_down": (K + 1) * (2 * g_b + d_b) + 3 * E * 4,
        "gemv_gate_up": (K + 1) * 2 * g_b + E * 4 + (K + 1) * FF * 4,
        "gemv_down": (K + 1) * d_b + (K + 1) * FF * 4 + (K + 1) * E * 4,
        "gemv_down_combine": (K + 1) * d_b + (K + 1) * FF * 4 + E * 4,
        "router_decode_fused": NE * E * 4 + 2 * E * 4 + NE * 4,
        "seg_gate_up_m1": K * 2 * g_b + E * 4 + K * FF * 4,
        "seg_matmul_m1": K * d_b + K * FF * 4 + K * E * 4,
        "router_logits": NE * E * 4 + E * 4 + NE * 4,
    }
    # DRAM bytes per launch (read + write) of each decode kernel: constants recorded from one profiler
    # capture per kernel on this workload, kept as data next to the capture summaries
    ncu_traffic = recorded_traffic()
    top = max((k for k in prof if k in alg), key=lambda k: prof[k]["ms"])
    per_launch_s = prof[top]["ms"] / prof[top]["launches"] * 1e-3
    achieved = alg[top] / per_launch_s / 1e9
    block_bytes = NE * E * 4 + (K + 1) * (2 * g_b + d_b)
    res = {
        "metric": "moe_decode_tok_s", "value": world * K_ / (ms_dev * 1e-3), "unit": "token*layer/s (1 MoE block per step)",
        "n_gpus": world, "steps": K_, "warmup": W_, "ms_per_step": ms_dev / K_, "higher_is_better": True,
        "repeats": int(rep_ms.size), "timed_region_s": float(rep_ms.sum() * 1e-3),
        "repeat_ms": {"min": float(rep_ms.min()), "median": ms_dev, "max": float(rep_ms.max()),
                      "note": "each repeat = exactly `steps` steps, event-timed; value uses the median repeat"},
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config1: 1 MoE block decode, 1 token, e2048 ff512 512 experts top-10 + 1 shared, IQ3_XXS",
                   "l2": "inputs larger than L2: %d rotating layer copies (%.0f MB of weights per cycle) and %d tokens"
                         % (LAYERS, LAYERS * block_bytes / 1e6, POOL),
                   "call": "value: %d blocks per dnb_moe_stack_dev call (residual stream stays on the device), the last "
                           "steps %% %d as single dnb_moe_block_dev calls; e2e: one block per dnb_moe_block call with host "
                           "buffers" % (LAYERS, LAYERS),
                   "parallelism": "replicas x%d" % world if world > 1 else "1 GPU"},
        "e2e": {"value": world * K_ / (ms_e2e * 1e-3), "unit": "token*layer/s", "h2d_bytes_per_step": E * 4,
                "d2h_bytes_per_step": E * 4, "repeats": int(e2e_ms.size), "us_per_call": ms_e2e / K_ * 1e3},
        "device_status": status,
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": ncu_traffic.get(top, {}).get("dram_bytes"),
                     "traffic_source": ncu_traffic.get(top, {}).get("source", "none recorded for this kernel"),
                     "bytes_per_launch": alg[top], "us_per_launch": per_launch_s * 1e6,
                     "how": "launches separated by events behind a GPU stall (no overlap between neighbouring launches); "
                            "back to back in the timed region a launch takes ms_per_step, see block_hbm_gbs"},
        "block_hbm_gbs": block_bytes / (ms_dev / K_ * 1e-3) / 1e9,
        "kernels_ms": {k: round(v["ms"], 4) for k, v in prof.items()},
    }
    if world > 1 and not args.no_extras:
        res["extras"] = {"config2_q4k_prefill_512_expert_parallel": guarded_ep_extras(res, cu, oracle, rank, world, local_rank)}
    if world == 1 and not args.no_extras:
        res["extras"] = extras(ctx, cu, oracle)
        ctx.close()
        ctx = None
        res["extras"]["config2_q4k_prefill_512"] = prefill_extras(cu, oracle, local_rank)
        if not args.no_stack:
            res["extras"].update(stack_extras(cu, oracle, local_rank))
    if world == 1 and not args.no_cpu:
        res["cpu_baseline"] = cpu_baseline(oracle, budget_s=10.0)
    if ctx is not None:
        ctx.close()
    return res


def build_shard(ctx, cu, oracle, ty_of_layer, layers, rank, world, bias):
    """Rank `rank`'s part of the model: experts [rank * NE / world, (rank + 1) * NE / world) of every layer
    (the same bytes the single-GPU model holds there: the generator is indexed by position in the full
    tensor), router, norm and shared expert replicated."""
    nl = NE // world
    assert ctx.moe_config(layers, E, FF, NE, K)
    ctx.set_expert_shard(rank * nl, nl)
    for l in range(layers):
        ty = ty_of_layer(l)
        for m, (ni, no, n) in ((cu.GATE, (E, FF, nl)), (cu.UP, (E, FF, nl)), (cu.DOWN, (FF, E, nl)),
                               (cu.SHARED_GATE, (E, FF, 1)), (cu.SHARED_UP, (E, FF, 1)), (cu.SHARED_DOWN, (FF, E, 1))):
            assert ctx.synth_experts(l, m, ty, ni, no, n, SEED)
        rw = oracle.synth_normal(SEED, l * 16 + 6, 0.02, NE * E)
        rb = router_bias(oracle, l, bias)
        ctx.register_router(l, rw, rb, np.ones(E, np.float32), None)
    ctx.sync()


def same_on_all_ranks(arr, local_rank):
    """True when every rank holds the same bits in `arr`."""
    import torch
    import torch.distributed as dist

    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int32).astype(np.int64)).cuda(local_rank)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return bool(torch.equal(lo, hi))


def run_ours_ep(args, rank, world, local_rank):
    """N > 1: the SAME workload as N = 1 (config 1: one token through one MoE block per step, IQ3_XXS,
    LAYERS rotating layer copies) with the experts sharded NE / N per GPU.  Strong scaling: the token is
    not multiplied by N.  The residual stream is replicated, every rank computes the (token, slot)
    pairs of its own experts and the result rows cross NVLink once per layer (dnb_epd_*)."""
    import torch
    import torch.distributed as dist

    import oracle
    from denno_beta_b200 import cuda as cu, ep

    ctx = cu.CudaCtx(local_rank)
    build_shard(ctx, cu, oracle, lambda l: IQ3_XXS, LAYERS, rank, world, False)
    pd = ep.PeerMemoryDecode(ctx, max_tokens=1)
    pool = oracle.synth_normal(SEED, 7000, 1.0, POOL * E).reshape(POOL, E)  # the same tokens on every rank
    d_pool = ctx.dev_alloc(pool.nbytes)
    d_out = ctx.dev_alloc(E * 4)
    d_h = ctx.dev_alloc(E * 4)
    ctx.upload(d_pool, pool)

    def barrier():
        ctx.sync()
        dist.barrier()

    K_, W_ = args.steps, max(args.warmup, 3)
    full, rem = divmod(K_, LAYERS)

    def k_steps(s0):
        for c_ in range(full):
            ctx.dev_copy(d_h, d_pool + ((s0 + c_) % POOL) * E * 4, E * 4)
            pd.stack_dev(d_h, 1)
        for r_ in range(rem):
            ctx.dev_copy(d_h, d_pool + ((s0 + full + r_) % POOL) * E * 4, E * 4)
            pd.block_dev(r_ % LAYERS, d_h, 1, d_out)

    # parity with one GPU: rank 0 also holds the whole model and runs the same exchange with a world of one
    want = None
    if rank == 0:
        one = cu.CudaCtx(local_rank)
        build_shard(one, cu, oracle, lambda l: IQ3_XXS, LAYERS, 0, 1, False)
        pd1 = ep.PeerMemoryDecode(one, max_tokens=1, rank=0, world=1)
        d1 = one.dev_alloc(E * 4)
        one.upload(d1, pool[3])
        pd1.stack_dev(d1, 1)
        assert one.sync()
        want = one.download(d1, np.empty(E, np.float32))
        one.close()
    barrier()  # the ranks enter their first exchange together: a peer's wait for this rank's rows is bounded (~a second)
    ctx.upload(d_h, pool[3])
    pd.stack_dev(d_h, 1)
    assert ctx.sync()
    got = ctx.download(d_h, np.empty(E, np.float32))
    same_ranks = same_on_all_ranks(got, local_rank)
    parity = bool(rank == 0 and np.array_equal(got.view(np.uint32), want.view(np.uint32)))

    for s in range(max(3, (W_ + K_ - 1) // K_)):
        k_steps(s)
    barrier()
    ctx.timer_start()
    k_steps(0)
    est_ms = max(ctx.timer_stop(), 1e-3)
    t = torch.tensor([est_ms], dtype=torch.float64, device="cuda:%d" % local_rank)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    repeats = int(min(500, max(5, np.ceil(100.0 / float(t)))))
    clocks = Clocks(local_rank)
    clocks.start()
    rep_ms = []
    launches = 0
    for r in range(repeats):
        barrier()
        l0 = ctx.launch_count()
        ctx.timer_start()
        k_steps(r)
        rep_ms.append(ctx.timer_stop())
        launches = ctx.launch_count() - l0
    barrier()
    # end to end: the token row from pinned host memory to the device, one block, the result row back
    out_host = np.empty(E, np.float32)
    e2e_n = min(K_, 200)
    for s in range(8):
        ctx.upload(d_h, pool[s % POOL])
        pd.block_dev(s % LAYERS, d_h, 1, d_out)
        ctx.download(d_out, out_host)
    e2e_ms = []
    for r in range(5):
        barrier()
        t0 = time.perf_counter()
        for s in range(e2e_n):
            ctx.upload(d_h, pool[(r * e2e_n + s) % POOL])
            pd.block_dev(s % LAYERS, d_h, 1, d_out)
            ctx.download(d_out, out_host)
        e2e_ms.append((time.perf_counter() - t0) * 1e3 / e2e_n * K_)
    clk = clocks.stop()
    barrier()
    status = ctx.device_status()
    ctx.profile(True)
    for s in range(4):
        k_steps(s) if full else None
    ctx.sync()
    prof = ctx.profile_read()
    ctx.profile(False)
    barrier()
    t = torch.tensor(np.concatenate([rep_ms, e2e_ms, [float(status)]]), dtype=torch.float64, device="cuda:%d" % local_rank)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t = t.cpu().numpy()
    rep_ms, e2e_ms, status = t[:len(rep_ms)], t[len(rep_ms):-1], int(t[-1])
    assert status == 0, "a bounded device wait gave up during the timed region (status %d): the numbers are void" % status
    dist.barrier()
    ctx.close()
    if rank != 0:
        if not args.no_extras:
            guarded_ep_extras(None, cu, oracle, rank, world, local_rank)
        return None
    ms_dev, ms_e2e = float(np.median(rep_ms)), float(np.median(e2e_ms))
    hbm_peak, _, peak_kind = peaks()
    g_b, d_b = expert_bytes(IQ3_XXS)
    block_bytes = NE * E * 4 + (K + 1) * (2 * g_b + d_b)
    achieved = block_bytes / (ms_dev / K_ * 1e-3) / 1e9
    res = {
        "metric": "moe_decode_tok_s", "value": K_ / (ms_dev * 1e-3), "unit": "token*layer/s (1 MoE block per step)",
        "n_gpus": world, "steps": K_, "warmup": W_, "ms_per_step": ms_dev / K_, "higher_is_better": True,
        "repeats": int(len(rep_ms)), "timed_region_s": float(np.sum(rep_ms) * 1e-3),
        "repeat_ms": {"min": float(np.min(rep_ms)), "median": ms_dev, "max": float(np.max(rep_ms)),
                      "note": "each repeat = exactly `steps` steps, event-timed, max over ranks; value uses the median repeat"},
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config1: 1 MoE block decode, 1 token, e2048 ff512 512 experts top-10 + 1 shared, IQ3_XXS",
                   "l2": "inputs larger than L2: %d rotating layer copies (%.0f MB of weights per cycle over all GPUs) and %d tokens"
                         % (LAYERS, LAYERS * block_bytes / 1e6, POOL),
                   "call": "value: %d blocks per dnb_epd_stack_dev call on every rank, the last steps %% %d as single "
                           "dnb_epd_block_dev calls; e2e: token row host -> device, one dnb_epd_block_dev, result row back"
                           % (LAYERS, LAYERS),
                   "parallelism": "expert-parallel %d/%d: %d experts per GPU, residual stream replicated, result rows stored "
                                  "into every rank's memory over NVLink once per layer (no collective library on the data path); "
                                  "the ONE token is not multiplied by the GPU count, so a step is latency-bound and more GPUs do "
                                  "not make it faster" % (NE, world, NE // world)},
        "e2e": {"value": K_ / (ms_e2e * 1e-3), "unit": "token*layer/s", "h2d_bytes_per_step": E * 4, "d2h_bytes_per_step": E * 4,
                "us_per_call": ms_e2e / K_ * 1e3, "note": "per rank; max over ranks"},
        "device_status": status, "parity_vs_1gpu": parity, "same_bits_on_every_rank": same_ranks,
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": {"bound": "hbm", "kernel": "all kernels of a step (the block's bytes over the step time, %d GPUs)" % world,
                     "achieved": achieved, "peak": hbm_peak * world, "unit": "GB/s", "frac": achieved / (hbm_peak * world),
                     "peak_kind": peak_kind, "traffic": None, "bytes_per_launch": block_bytes, "us_per_launch": ms_dev / K_ * 1e3},
        "kernels_ms_rank0": {k: round(v["ms"], 4) for k, v in prof.items()},
    }
    if not args.no_extras:
        res["extras"] = guarded_ep_extras(res, cu, oracle, rank, world, local_rank)
    return res


def extras(ctx, cu, oracle):
    """Config 0 (single Q4_K GEMV 4096x4096, HBM GB/s) on rotating weight copies, and the
    same GEMV in the path's other block formats (IQ3_XXS, Q6_K, Q8_0)."""
    out = {}
    k = n = 4096
    x = oracle.synth_normal(SEED, 9001, 1.0, k)
    dx = ctx.dev_alloc(k * 4)
    do = ctx.dev_alloc(n * 4)
    ctx.upload(dx, x)
    for name, ty in (("q4k", Q4_K), ("iq3xxs", IQ3_XXS), ("q6k", 14), ("q80", 8)):
        rb = oracle.row_bytes(ty, k)
        copies = (320 * 1024 * 1024 + n * rb - 1) // (n * rb)  # > 126 MB of L2 several times over
        w = oracle.synth_blocks(ty, SEED, 9000 + ty, n * (k // oracle.blck_size(ty)))
        dw = ctx.dev_alloc(copies * n * rb)
        for i in range(copies):
            ctx.upload(dw + i * n * rb, w)
        for i in range(8):
            ctx.gemv_dev(ty, dw + (i % copies) * n * rb, k, n, dx, do, 1)
        ctx.sync()
        reps = 256
        ctx.stall(10.0)  # the launches below queue up behind it and then run back to back
        ctx.timer_start()
        for i in range(reps):
            ctx.gemv_dev(ty, dw + (i % copies) * n * rb, k, n, dx, do, 1)
        ms = ctx.timer_stop()
        alg = n * rb + k * 4 + n * 4
        out["config0_%s_gemv_4096" % name] = {"us_per_gemv": ms / reps * 1e3, "hbm_gbs": alg / (ms / reps * 1e-3) / 1e9,
                                              "bytes": alg, "launches": reps, "rotating_copies": copies,
                                              "frac_of_measured_hbm": alg / (ms / reps * 1e-3) / 1e9 / peaks()[0]}
        ctx.dev_free(dw)
    # The same kernel on a launch 16 times as large (4096 x 65536: 100-290 MB per launch, two rotating copies):
    # what it reaches when a launch is not mostly ramp and drain.
    n_big = 16 * n
    do_big = ctx.dev_alloc(n_big * 4)
    for name, ty in (("q4k", Q4_K), ("iq3xxs", IQ3_XXS), ("q6k", 14), ("q80", 8)):
        rb = oracle.row_bytes(ty, k)
        w = oracle.synth_blocks(ty, SEED, 9000 + ty, n * (k // oracle.blck_size(ty)))
        dw = ctx.dev_alloc(2 * n_big * rb)
        for i in range(32):
            ctx.upload(dw + i * n * rb, w)
        for i in range(3):
            ctx.gemv_dev(ty, dw + (i % 2) * n_big * rb, k, n_big, dx, do_big, 1)
        ctx.sync()
        reps = 16
        ctx.timer_start()
        for i in range(reps):
            ctx.gemv_dev(ty, dw + (i % 2) * n_big * rb, k, n_big, dx, do_big, 1)
        ms = ctx.timer_stop()
        alg = n_big * rb + k * 4 + n_big * 4
        out["config0_x16_%s_gemv_4096x65536" % name] = {"us_per_gemv": ms / reps * 1e3, "hbm_gbs": alg / (ms / reps * 1e-3) / 1e9, "bytes": alg,
                                                        "frac_of_measured_hbm": alg / (ms / reps * 1e-3) / 1e9 / peaks()[0]}
        ctx.dev_free(dw)
    ctx.dev_free(do_big)
    for p in (dx, do):
        ctx.dev_free(p)
    return out


def prefill_extras(cu, oracle, device, layers=4, ty=Q4_K):
    """Config 2: one MoE block, one 512-token chunk, Q4_K experts, Zipf router bias.
    Rotates over `layers` layer copies (0.9 GB of weights each); tokens stay on the device."""
    nt = 512
    ctx = cu.CudaCtx(device)
    out = {}
    try:
        build_model(ctx, cu, ty, layers, True)
        h = oracle.synth_normal(SEED, 8000, 1.0, nt * E).reshape(nt, E)
        d_h = ctx.dev_alloc(h.nbytes)
        d_o = ctx.dev_alloc(h.nbytes)
        ctx.upload(d_h, h)
        for l in range(2 * layers):
            assert ctx.moe_block_dev(l % layers, d_h, nt, d_o)
        ctx.sync()
        reps = 24
        ctx.stall(5.0)
        ctx.timer_start()
        for l in range(reps):
            assert ctx.moe_block_dev(l % layers, d_h, nt, d_o)
        ms = ctx.timer_stop() / reps
        ctx.profile(True)
        for l in range(layers):
            ctx.stall(2.0)
            assert ctx.moe_block_dev(l % layers, d_h, nt, d_o)
        prof = ctx.profile_read()
        ctx.profile(False)
        sels = ctx.router_topk(0, oracle.rmsnorm(h, np.ones(E, np.float32)))[0]
        counts = np.bincount(sels.ravel(), minlength=NE)
        active = int((counts > 0).sum())
        flops = 2.0 * 3 * E * FF * (nt * K + nt) + 2.0 * nt * NE * E
        g_b, d_b = expert_bytes(ty)
        bytes_ = (active + 1) * (2 * g_b + d_b) + NE * E * 4 + 2 * nt * E * 4
        hbm, tf, _ = peaks()
        out = {"ms_per_chunk_layer": ms, "tok_per_s_layer": nt / (ms * 1e-3), "algorithmic_tflops": flops / (ms * 1e-3) / 1e12,
               "frac_of_measured_bf16": flops / (ms * 1e-3) / 1e12 / tf, "algorithmic_gbs": bytes_ / (ms * 1e-3) / 1e9,
               "frac_of_measured_hbm": bytes_ / (ms * 1e-3) / 1e9 / hbm, "active_experts": active,
               "max_tokens_per_expert": int(counts.max()), "median_tokens_per_expert": float(np.median(counts)),
               "kernels_ms_per_layer": {k: round(v["ms"] / layers, 4) for k, v in prof.items()}}
        ctx.dev_free(d_h)
        ctx.dev_free(d_o)
    finally:
        ctx.close()
    return out


_EMIT = {"fd": None}


def guarded_ep_extras(partial, cu, oracle, rank, world, local_rank, limit_s=600.0):
    """The expert-parallel extras under a watchdog: whatever happens to them (an exception on
    one rank leaves the others waiting in a collective), rank 0 still prints the bench line,
    with the reason in place of the extras, and every rank exits 0."""
    import threading

    def bail(why):
        if partial is not None and _EMIT["fd"] is not None:
            partial["extras"] = {"error": why}
            os.write(_EMIT["fd"], (json.dumps(partial) + "\n").encode())
        # This rank's arena is memory its peers' kernels may still be storing into.  Every device-side
        # wait of the exchange gives up after ~0.25 s (three of them per block at most), so a few
        # seconds from now no peer kernel can still be running against it; only then leave.
        time.sleep(4.0)
        os._exit(0)

    timer = threading.Timer(limit_s, bail, args=("expert-parallel extras did not finish in %.0f s" % limit_s,))
    timer.daemon = True
    timer.start()
    try:
        out = {"config3_decode_stack48_expert_parallel": ep_decode_stack(cu, oracle, rank, world, local_rank)}
        out["config2_q4k_prefill_512_expert_parallel"] = ep_prefill_extras(cu, oracle, rank, world, local_rank)
        out["config4_prefill_stack48_14018_expert_parallel"] = ep_stack_prefill(cu, oracle, rank, world, local_rank)
        # the same two with the hot experts placed by expected load instead of where the seed put them
        out["config2_q4k_prefill_512_expert_parallel_placed"] = ep_prefill_extras(cu, oracle, rank, world, local_rank, "placed")
        out["config4_prefill_stack48_14018_expert_parallel_placed"] = ep_stack_prefill(cu, oracle, rank, world, local_rank, "placed")
    except Exception as ex:  # the other ranks run into their own watchdog
        bail("expert-parallel extras failed on rank %d: %s" % (rank, ex))
    timer.cancel()
    return out


def ep_decode_stack(cu, oracle, rank, world, local_rank):
    """Config 3 across `world` GPUs: the 48-layer decode stack (40 IQ3_XXS + 8 Q4_K layers, every sixth),
    experts sharded 512 / world per GPU, batches of 1, 8 and 32 tokens, one dnb_epd_stack_dev call per
    step.  The same weights and tokens as the single-GPU line; rank 0 also holds the whole model and
    checks that the expert-parallel result has the bits of the same exchange run with a world of one."""
    import torch
    import torch.distributed as dist

    from denno_beta_b200 import ep

    ty_of = lambda l: Q4_K if l % 6 == 5 else IQ3_XXS
    ctx = cu.CudaCtx(local_rank)
    build_shard(ctx, cu, oracle, ty_of, 48, rank, world, False)
    pd = ep.PeerMemoryDecode(ctx, max_tokens=32)
    one = pd1 = None
    if rank == 0:
        one = cu.CudaCtx(local_rank)
        build_shard(one, cu, oracle, ty_of, 48, 0, 1, False)
        pd1 = ep.PeerMemoryDecode(one, max_tokens=32, rank=0, world=1)
    out = {"experts_per_rank": NE // world,
           "exchange": "result rows stored into every rank's memory by this library's kernels, one flag wait per layer"}
    for B in (1, 8, 32):
        h = oracle.synth_normal(SEED, 8100 + B, 1.0, B * E).reshape(B, E)
        d_src, d_h = ctx.dev_alloc(h.nbytes), ctx.dev_alloc(h.nbytes)
        ctx.upload(d_src, h)
        ctx.sync()
        dist.barrier()  # enter the exchange together (the waits for a peer's rows are bounded)
        for _ in range(3):
            ctx.dev_copy(d_h, d_src, h.nbytes)
            pd.stack_dev(d_h, B)
        ctx.sync()
        got = ctx.download(d_h, np.empty((B, E), np.float32))
        parity = None
        if rank == 0:
            d1 = one.dev_alloc(h.nbytes)
            one.upload(d1, h)
            pd1.stack_dev(d1, B)
            assert one.sync()
            parity = bool(np.array_equal(got.view(np.uint32), one.download(d1, np.empty((B, E), np.float32)).view(np.uint32)))
            one.dev_free(d1)
        dist.barrier()
        same = same_on_all_ranks(got, local_rank)
        reps = 10
        dist.barrier()
        ctx.timer_start()
        for _ in range(reps):
            ctx.dev_copy(d_h, d_src, h.nbytes)
            pd.stack_dev(d_h, B)
        ms = torch.tensor([ctx.timer_stop() / reps], dtype=torch.float64, device="cuda:%d" % local_rank)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        out["batch%d" % B] = {"ms_per_step": float(ms), "tok_per_s": B / (float(ms) * 1e-3), "parity_vs_1gpu": parity,
                              "same_bits_on_every_rank": same}
        ctx.dev_free(d_src)
        ctx.dev_free(d_h)
    out["device_status"] = ctx.device_status()
    dist.barrier()
    ctx.close()
    if one is not None:
        one.close()
    return out


def ep_prefill_extras(cu, oracle, rank, world, local_rank, bias=True):
    """Config 2 across `world` GPUs, expert parallel: 512/world experts per GPU (the same weights as the
    single-GPU line), the 512-token chunk split evenly over the ranks (strong scaling), or one chunk per
    rank.  Timed with events on the block's stream, max over ranks.  Rank 0 also holds the whole layer
    and checks that the expert-parallel output has the single-GPU block's bits."""
    import torch
    import torch.distributed as dist

    from denno_beta_b200 import ep

    layers, nt_total = 4, 512
    nl, nt = NE // world, nt_total // world
    ctx = cu.CudaCtx(local_rank)
    build_shard(ctx, cu, oracle, lambda l: Q4_K, layers, rank, world, bias)
    h_all = oracle.synth_normal(SEED, 8000, 1.0, nt_total * E).reshape(nt_total, E)

    def timed(step, reps=16):
        ctx.sync()
        dist.barrier()  # enter the exchange together (the device-side waits for a peer are bounded)
        for l in range(2 * layers):
            step(l % layers)
        ctx.sync()
        dist.barrier()
        ctx.timer_start()
        for l in range(reps):
            step(l % layers)
        ms = torch.tensor([ctx.timer_stop() / reps], dtype=torch.float64, device="cuda:%d" % local_rank)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    out = {"experts_per_rank": nl}
    # (a) rows exchanged by NCCL all-to-all between this library's calls (host plans the split sizes)
    blk = ep.ExpertParallelBlock(ctx, E, NE, K)
    h = torch.from_numpy(h_all[rank * nt:(rank + 1) * nt].copy()).cuda(local_rank)
    ms = timed(lambda l: blk.block(l, h))
    out["nccl_all_to_all_strong"] = {"ms_per_chunk_layer": ms, "tok_per_s_layer": nt_total / (ms * 1e-3), "tokens_per_rank": nt,
                                     "exchange": "NCCL all_to_all_single (dispatch rows fp32 + ids, return rows fp32)",
                                     "scaling": "strong (one 512-token chunk over %d GPUs)" % world}
    ctx.set_stream(None)
    # (b), (c) rows stored into the peers' memory by this library's kernels, no collective, no host round trip
    pm = ep.PeerMemoryExpertParallel(ctx, max_tokens=nt_total)
    d_h = ctx.dev_alloc(nt_total * E * 4)
    d_o = ctx.dev_alloc(nt_total * E * 4)
    ctx.upload(d_h, np.ascontiguousarray(h_all[rank * nt:(rank + 1) * nt]))
    ms = timed(lambda l: pm.block_dev(l, d_h, nt, d_o))
    # parity: the ranks' outputs of layer 0, gathered, against the single-GPU block on the whole chunk
    pm.block_dev(0, d_h, nt, d_o)
    ctx.sync()
    mine = torch.from_numpy(ctx.download(d_o, np.empty((nt, E), np.float32))).cuda(local_rank)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    parity = None
    if rank == 0:
        one = cu.CudaCtx(local_rank)
        build_shard(one, cu, oracle, lambda l: Q4_K, 1, 0, 1, bias)
        d1, d2 = one.dev_alloc(h_all.nbytes), one.dev_alloc(h_all.nbytes)
        one.upload(d1, h_all)
        assert one.moe_block_dev(0, d1, nt_total, d2)
        one.sync()
        want = one.download(d2, np.empty((nt_total, E), np.float32))
        one.close()
        got = torch.cat(parts).cpu().numpy()
        parity = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
    out["peer_memory_strong"] = {"ms_per_chunk_layer": ms, "tok_per_s_layer": nt_total / (ms * 1e-3), "tokens_per_rank": nt,
                                 "exchange": "peer stores from the dispatch kernel and the down-GEMM epilogue, flag-ordered",
                                 "scaling": "strong (one 512-token chunk over %d GPUs)" % world, "parity_vs_1gpu": parity}
    # every rank owns a whole 512-token chunk (a prompt's chunks spread over the ranks)
    ctx.upload(d_h, np.ascontiguousarray(oracle.synth_normal(SEED, 8000 + rank, 1.0, nt_total * E)))
    ms = timed(lambda l: pm.block_dev(l, d_h, nt_total, d_o))
    out["peer_memory_chunk_per_rank"] = {"ms_per_step_layer": ms, "ms_per_chunk_layer": ms / world,
                                         "tok_per_s_layer": world * nt_total / (ms * 1e-3), "tokens_per_rank": nt_total,
                                         "exchange": "peer stores from the dispatch kernel and the down-GEMM epilogue, flag-ordered",
                                         "scaling": "%d chunks of 512 tokens in flight, one per GPU" % world}
    # per-kernel times of one rank's step (events around every launch; waits on peers included)
    ctx.sync()
    dist.barrier()
    ctx.profile(True)
    for l in range(layers):
        pm.block_dev(l, d_h, nt_total, d_o)
    ctx.sync()
    prof = ctx.profile_read()
    ctx.profile(False)
    out["peer_memory_chunk_per_rank"]["kernels_ms_per_layer_rank0"] = {k: round(v["ms"] / layers, 4) for k, v in prof.items()}
    out["device_status"] = ctx.device_status()
    dist.barrier()
    ctx.close()
    out["placement"] = "hot experts placed by expected load (placed_zipf_bias)" if bias == "placed" else "experts where the seed put them"
    return out


def ep_stack_prefill(cu, oracle, rank, world, local_rank, bias=True):
    """Config 4 across `world` GPUs: 48 all-Q4_K blocks (the single-GPU line's weights), a 14,018-token
    prompt in 512-token chunks (27 x 512 + 194) dealt to the ranks round-robin, every chunk-step through
    all 48 layers with the peer-memory exchange and the identity mixers' residual add (dnb_ep_stack_dev,
    direct launches; the single-GPU line replays a CUDA graph).  Rank 0 also holds the whole model and
    checks that its first chunk comes out with the single-GPU stack's bits."""
    import torch
    import torch.distributed as dist

    from denno_beta_b200 import ep

    n_layer, n_tok = 48, 14018
    # 512-token chunks dealt round-robin in waves of `world`; the tokens that do not fill a whole wave (1,730 of
    # 14,018 at 8 GPUs: three chunks and the 194-token rest) are cut into `world` equal chunks instead, so the
    # last wave keeps every GPU busy.  A token's result does not depend on the chunk it is in.
    waves = (n_tok // 512) // world
    rest = n_tok - waves * world * 512
    tail = [rest // world + (1 if r_ < rest % world else 0) for r_ in range(world)] if rest else []
    chunks = [512] * (waves * world) + [t_ for t_ in tail if t_ > 0]
    steps = waves + (1 if rest else 0)
    mine = [512] * waves + ([max(tail[rank], 1)] if rest else [])  # a rank with nothing in the tail runs 1 dummy token
    ctx = cu.CudaCtx(local_rank)
    build_shard(ctx, cu, oracle, lambda l: Q4_K, n_layer, rank, world, bias)
    pm = ep.PeerMemoryExpertParallel(ctx, max_tokens=512)
    h = oracle.synth_normal(SEED, 8200, 1.0, 512 * E).reshape(512, E)  # every chunk reuses these rows, as on one GPU
    d_src = ctx.dev_alloc(h.nbytes)
    d_h = ctx.dev_alloc(h.nbytes)
    ctx.upload(d_src, h)

    def prompt():
        for nt in mine:
            ctx.dev_copy(d_h, d_src, nt * E * 4)
            pm.stack_dev(d_h, nt)
    ctx.sync()
    dist.barrier()
    prompt()
    ctx.sync()
    parity = None
    # the last chunk-step this rank ran (nt = mine[-1]) against the single-GPU stack on the same rows
    got = ctx.download(d_h, np.empty((512, E), np.float32))[:mine[-1]]
    if rank == 0:
        one = cu.CudaCtx(local_rank)
        build_model(one, cu, Q4_K, n_layer, bias)
        d1 = one.dev_alloc(h.nbytes)
        one.upload(d1, h)
        assert one.moe_stack_dev(d1, mine[-1])
        one.sync()
        want = one.download(d1, np.empty((512, E), np.float32))[:mine[-1]]
        one.close()
        parity = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
    dist.barrier()
    ctx.timer_start()
    prompt()
    ms = torch.tensor([ctx.timer_stop()], dtype=torch.float64, device="cuda:%d" % local_rank)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    status = ctx.device_status()
    dist.barrier()
    ctx.close()
    return {"placement": "hot experts placed by expected load (placed_zipf_bias)" if bias == "placed" else "experts where the seed put them",
            "seconds": ms * 1e-3, "tok_per_s": n_tok / (ms * 1e-3), "chunk_steps": steps, "chunks": len(chunks),
            "algorithmic_tflops": n_tok * n_layer * (11 * 6291456 + 2097152) / (ms * 1e-3) / 1e12,
            "exchange": "peer memory (dnb_ep_stack_dev), 512-token chunks dealt round-robin to %d GPUs, the last partial wave cut into equal chunks" % world, "device_status": status,
            "parity_vs_1gpu": parity}


def stack_extras(cu, oracle, device, n_layer=48, batches=(1, 8, 32), prefill=True):
    """Configs 3 and 4: the 48-block stack (identity mixers, h <- h + block(h)).
    Decode: 40 IQ3_XXS + 8 Q4_K layers (every sixth), batch 1 / 8 / 32, one
    dnb_moe_stack_dev call per step (CUDA-graph replay).  Prefill: all-Q4_K layers with
    the Zipf router bias, a 14,018-token prompt in 512-token chunks (27 x 512 + 194)."""
    out = {}
    g3, d3 = expert_bytes(IQ3_XXS)
    g4, d4 = expert_bytes(Q4_K)
    ctx = cu.CudaCtx(device)
    try:
        build_model(ctx, cu, IQ3_XXS, n_layer, False, ty_of_layer=lambda l: Q4_K if l % 6 == 5 else IQ3_XXS)
        n4 = n_layer // 6
        step_bytes = (n_layer - n4) * (NE * E * 4 + 11 * (2 * g3 + d3)) + n4 * (NE * E * 4 + 11 * (2 * g4 + d4))
        hbm = peaks()[0]
        for B in batches:
            h = oracle.synth_normal(SEED, 8100 + B, 1.0, B * E).reshape(B, E)
            d_src = ctx.dev_alloc(h.nbytes)
            d_h = ctx.dev_alloc(h.nbytes)
            ctx.upload(d_src, h)
            for _ in range(3):
                ctx.dev_copy(d_h, d_src, h.nbytes)
                assert ctx.moe_stack_dev(d_h, B)
            ctx.sync()
            reps = 12
            ctx.timer_start()
            for _ in range(reps):
                ctx.dev_copy(d_h, d_src, h.nbytes)
                assert ctx.moe_stack_dev(d_h, B)
            ms = ctx.timer_stop() / reps
            res = {"ms_per_step": ms, "tok_per_s": B / (ms * 1e-3)}
            if B == 1:
                res["algorithmic_bytes_per_step"] = step_bytes
                res["hbm_gbs"] = step_bytes / (ms * 1e-3) / 1e9
                res["frac_of_measured_hbm"] = res["hbm_gbs"] / hbm
            out["config3_decode_stack%d_batch%d" % (n_layer, B)] = res
            ctx.dev_free(d_src)
            ctx.dev_free(d_h)
    finally:
        ctx.close()
    if not prefill:
        return out
    ctx = cu.CudaCtx(device)
    try:
        build_model(ctx, cu, Q4_K, 48, True)
        n_tok = 14018
        chunks = [512] * 27 + [194]
        h = oracle.synth_normal(SEED, 8200, 1.0, 512 * E).reshape(512, E)
        d_src = ctx.dev_alloc(h.nbytes)
        d_h = ctx.dev_alloc(h.nbytes)
        ctx.upload(d_src, h)
        for nt in (512, 194, 512, 194):  # warm-up: workspace, graphs
            ctx.dev_copy(d_h, d_src, nt * E * 4)
            assert ctx.moe_stack_dev(d_h, nt)
        ctx.sync()
        ctx.timer_start()
        for nt in chunks:
            ctx.dev_copy(d_h, d_src, nt * E * 4)
            assert ctx.moe_stack_dev(d_h, nt)
        ms = ctx.timer_stop()
        flops = n_tok * 48.0 * (11 * 6291456 + 2097152)
        out["config4_prefill_stack48_14018"] = {"seconds": ms * 1e-3, "tok_per_s": n_tok / (ms * 1e-3),
                                                "algorithmic_tflops": flops / (ms * 1e-3) / 1e12,
                                                "frac_of_measured_bf16": flops / (ms * 1e-3) / 1e12 / peaks()[1],
                                                "chunks": "27 x 512 + 194 (every chunk reuses the same 512 seeded rows)"}
        ctx.dev_free(d_src)
        ctx.dev_free(d_h)
    finally:
        ctx.close()
    return out


def cpu_layer(oracle, ty=IQ3_XXS, bias=False):
    nb = lambda rows, cols: rows * cols // 256
    gate = oracle.synth_blocks(ty, SEED, 0, NE * nb(FF, E))
    up = oracle.synth_blocks(ty, SEED, 1, NE * nb(FF, E))
    down = oracle.synth_blocks(ty, SEED, 2, NE * nb(E, FF))
    sh = (oracle.synth_blocks(ty, SEED, 3, nb(FF, E)), oracle.synth_blocks(ty, SEED, 4, nb(FF, E)),
          oracle.synth_blocks(ty, SEED, 5, nb(E, FF)))
    rw = oracle.synth_normal(SEED, 6, 0.02, NE * E).reshape(NE, E)
    rb = oracle.synth_zipf_bias(SEED, 7, 1.1, NE) if bias else None
    return oracle.Layer(E, FF, NE, K, ty, ty, ty, gate, up, down, rw, router_bias=rb, norm_w=np.ones(E, np.float32), shared=sh)


def host_threads():
    """Threads the CPU legs use: every core this process may run on.  Set explicitly on the OpenMP
    runtime (a launcher such as torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


CPU_NOTE = ("AVX2+FMA restatement of the reference's production CPU kernels (gemv_q4k_avx2, gemv_iq<3>, k-chunked "
            "gemm_q4k_avx2; 64-row parallel chunks), OpenMP; the Rust reference cannot be built here (no cargo). "
            "The reference publishes 31.2 GB/s at 8 threads for its IQ3_S AVX2 GEMV on its own desktop CPU")


def cpu_baseline(oracle, budget_s, with_other_configs=True):
    """The reference path's production CPU form on this box's cores: tokens of config 1 through one
    block until `budget_s` has passed; config 0 (one 4096 x 4096 Q4_K GEMV) and config 2 (one 512-token
    Q4_K chunk, Zipf bias) as bounded samples beside it."""
    threads = host_threads()
    oracle.set_threads(threads)
    L = cpu_layer(oracle)
    pool = oracle.synth_normal(SEED, 7000, 1.0, POOL * E).reshape(POOL, E)
    for i in range(3):
        oracle.fast_moe_block(L, pool[i:i + 1])
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < budget_s:
        oracle.fast_moe_block(L, pool[n % POOL:n % POOL + 1])
        n += 1
    dt = time.perf_counter() - t0
    g_b, d_b = expert_bytes(IQ3_XXS)
    block_bytes = NE * E * 4 + (K + 1) * (2 * g_b + d_b)
    out = {"value": n / dt, "unit": "token*layer/s", "cores": threads, "threads": threads, "kind": "port",
           "sample": "%d tokens of config 1 through one block in %.1f s (one layer copy)" % (n, dt),
           "gb_s": block_bytes * n / dt / 1e9, "what": CPU_NOTE}
    del L
    if with_other_configs:
        k = n_ = 4096
        w = oracle.synth_blocks(Q4_K, SEED, 9000 + Q4_K, n_ * (k // 256))
        x = oracle.synth_normal(SEED, 9001, 1.0, k)
        oracle.fast_gemv(Q4_K, w, k, n_, x)
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 2.0:
            oracle.fast_gemv(Q4_K, w, k, n_, x)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        out["config0_q4k_gemv_4096"] = {"us_per_gemv": dt * 1e6, "gb_s": (w.nbytes + 2 * k * 4) / dt / 1e9, "launches": reps,
                                        "note": "one resident matrix (9.4 MB: served from the CPU's caches where they hold it)"}
        del w
        L2 = cpu_layer(oracle, Q4_K, bias=True)
        h = oracle.synth_normal(SEED, 8000, 1.0, 512 * E).reshape(512, E)
        oracle.fast_moe_block(L2, h[:64], grouped=True)
        t0 = time.perf_counter()
        oracle.fast_moe_block(L2, h, grouped=True)
        dt = time.perf_counter() - t0
        out["config2_q4k_prefill_512"] = {"ms_per_chunk_layer": dt * 1e3, "tok_per_s_layer": 512 / dt,
                                          "algorithmic_tflops": (2.0 * 3 * E * FF * (512 * K + 512) + 2.0 * 512 * NE * E) / dt / 1e12,
                                          "sample": "one 512-token chunk, once"}
        # configs 3 and 4 (48 layers) are not run on the CPU: extrapolated from the per-block times above
        t_chunk = dt
        for i in range(2):
            oracle.fast_moe_block(L2, h[i:i + 1])
        m, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 1.0:
            oracle.fast_moe_block(L2, h[m % 64:m % 64 + 1])
            m += 1
        t_q4 = (time.perf_counter() - t0) / m
        t_iq3 = 1.0 / out["value"]
        out["config3_decode_stack48_batch1"] = {"tok_per_s": 1.0 / (40 * t_iq3 + 8 * t_q4), "extrapolated": True,
                                                "from": "40 x the IQ3_XXS block time + 8 x a Q4_K block time (%d one-token blocks in 1 s)" % m}
        out["config4_prefill_stack48_14018"] = {"seconds": 48 * (14018 / 512.0) * t_chunk, "tok_per_s": 14018 / (48 * (14018 / 512.0) * t_chunk),
                                                "extrapolated": True, "from": "48 layers x 27.4 chunks x the config-2 chunk time"}
    return out


def run_reference(args, rank):
    """The reference arm: the path's CPU form (see CPU_NOTE) on this box's host cores, all threads,
    same workload / metric / unit as the GPU arm; a step = one token through one block."""
    if rank != 0:
        return None
    import oracle

    threads = host_threads()
    oracle.set_threads(threads)
    L = cpu_layer(oracle)
    pool = oracle.synth_normal(SEED, 7000, 1.0, POOL * E).reshape(POOL, E)
    K_, W_ = args.steps, max(args.warmup, 1)
    K_ = min(K_, 20000)
    for s in range(W_):
        oracle.fast_moe_block(L, pool[s % POOL:s % POOL + 1])
    t0 = time.perf_counter()
    for s in range(K_):
        i = (W_ + s) % POOL
        oracle.fast_moe_block(L, pool[i:i + 1])
    dt = time.perf_counter() - t0
    v = K_ / dt
    g_b, d_b = expert_bytes(IQ3_XXS)
    block_bytes = NE * E * 4 + (K + 1) * (2 * g_b + d_b)
    return {
        "impl": "reference", "metric": "moe_decode_tok_s", "value": v, "unit": "token*layer/s (1 MoE block per step)",
        "n_gpus": args.gpus, "steps": K_, "warmup": W_, "ms_per_step": dt / K_ * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config1: 1 MoE block decode, 1 token, e2048 ff512 512 experts top-10 + 1 shared, IQ3_XXS",
                   "note": CPU_NOTE},
        "cpu_baseline": {"value": v, "unit": "token*layer/s", "cores": threads, "threads": threads, "kind": "port",
                         "sample": "%d tokens, one layer copy" % K_, "gb_s": block_bytes * v / 1e9},
        "threads": threads,
        "e2e": {"value": v, "unit": "token*layer/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    global LAYERS
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON
    # line there.  Everything but the final line goes to stderr.
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    _EMIT["fd"] = real_stdout
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="rotating layer copies (default %d; fewer for profiler captures)" % LAYERS)
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the config-2 prefill measurement (small: for profiler captures)")
    ap.add_argument("--decode-impl", type=int, default=0, choices=[0, 3, 4, 5],
                    help="one-token kernels of the headline line: 0 the whole block as one mma.sync kernel (default), 5 router "
                         "kernel + fused gate/up + down kernel, 4 router + mma.sync gate/up + down kernels, 3 register-decode "
                         "kernels (for A/B runs and profiler captures of those kernels)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the config-0/2/3/4 lines")
    ap.add_argument("--no-stack", action="store_true", help="skip the 48-layer stack lines (configs 3 and 4)")
    ap.add_argument("--prefill-type", default="q4k", choices=["q4k", "iq3xxs"],
                    help="block format of --prefill-only (config 2 is Q4_K; IQ3_XXS runs the exact-weight tcgen05 kernel)")
    ap.add_argument("--stack-only", type=int, default=0, metavar="BATCH",
                    help="only the decode stack of config 3 at this batch size, with --layers layers (small enough for a profiler capture)")
    ap.add_argument("--gemv-only", action="store_true",
                    help="only the config-0 single-matrix GEMV lines (small enough for a profiler capture)")
    args = ap.parse_args()
    if args.layers > 0:
        LAYERS = args.layers
    else:
        # The rotating layer copies are walked by ONE stack call; a step count they divide needs no single-block
        # calls for the remainder (20 steps: 20 copies, one call).  16 to 32 copies: 279 to 557 MB per cycle, all > L2.
        LAYERS = next((l_ for l_ in (16, 20, 24, 25, 18, 30, 32, 28, 21, 27, 22, 26, 17, 19, 23, 29, 31) if args.steps % l_ == 0), 16)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.prefill_only:
        import oracle
        from denno_beta_b200 import cuda as cu

        res = {"config2_%s_prefill_512" % args.prefill_type: prefill_extras(
            cu, oracle, local_rank, layers=max(args.layers, 1), ty=Q4_K if args.prefill_type == "q4k" else IQ3_XXS)}
    elif args.stack_only:
        import oracle
        from denno_beta_b200 import cuda as cu

        res = stack_extras(cu, oracle, local_rank, n_layer=max(args.layers, 1), batches=(args.stack_only,), prefill=False)
    elif args.gemv_only:
        import oracle
        from denno_beta_b200 import cuda as cu

        ctx = cu.CudaCtx(local_rank)
        res = extras(ctx, cu, oracle)
        ctx.close()
    elif args.impl == "reference":
        res = run_reference(args, rank)
    else:
        if world > 1:
            import torch
            import torch.distributed as dist

            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda:%d" % local_rank))
        res = run_ours_ep(args, rank, world, local_rank) if world > 1 else run_ours(args, rank, world, local_rank)
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
            dist.destroy_process_group()
    sys.stdout.flush()
    if res is not None:
        os.write(real_stdout, (json.dumps(res) + "\n").encode())


if __name__ == "__main__":
    main()
