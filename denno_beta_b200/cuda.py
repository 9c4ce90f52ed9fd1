"""Host-side mirror of denno-engine's GPU dispatch interface for the MoE expert path.

The functions keep the names, argument meaning and error behaviour of the `pub fn`s
of crates/denno-engine/src/cuda.rs that model/qwen4exp.rs and model/linear_gguf.rs
call on this path; each forwards to one C-ABI entry point of libdnb200.  As in the
reference a `False` return means "the GPU did not run this, nothing was written,
take your own route" and misuse raises.  There is no CPU fallback in here.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import DnbError, check

# ggml type ids (kquant.rs:72-104)
Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, IQ3_XXS = 7, 8, 12, 13, 14, 18
Q4_0, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS, Q2_0 = 2, 20, 21, 22, 23, 42
GATE, UP, DOWN, SHARED_GATE, SHARED_UP, SHARED_DOWN = range(6)

TYPE_SIZE = {Q5_1: 24, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ3_XXS: 98,
             Q4_0: 18, IQ4_NL: 18, IQ3_S: 110, IQ2_S: 82, IQ4_XS: 136, Q2_0: 18}
BLOCK_ELEMS = {Q5_1: 32, Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, IQ3_XXS: 256,
               Q4_0: 32, IQ4_NL: 32, IQ3_S: 256, IQ2_S: 256, IQ4_XS: 256, Q2_0: 64}


def row_bytes(ty, n_in):
    """moe_expert.rs:84-100."""
    if ty not in TYPE_SIZE or n_in <= 0 or n_in % BLOCK_ELEMS[ty]:
        raise ValueError("n_in=%d is not a whole number of blocks of ggml type %d" % (n_in, ty))
    return n_in // BLOCK_ELEMS[ty] * TYPE_SIZE[ty]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def host_ptr(a):
    """ctypes pointer to a contiguous array's first byte, for reuse across calls (the array must
    stay alive and in place)."""
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _f32(a, shape=None):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a if shape is None else a.reshape(shape)


_shared = {}


def cuda_enabled():
    """cuda.rs:18029-18044: True when a context on device 0 can be made."""
    try:
        shared_ctx()
        return True
    except (DnbError, ImportError, OSError):
        return False


def shared_ctx(device=0):
    """cuda.rs:18066-18082: the lazily created per-device context."""
    if device not in _shared:
        _shared[device] = CudaCtx(device)
    return _shared[device]


class CudaCtx:
    """One device + one stream (cuda.rs CudaCtx).  Not re-entrant."""

    def __init__(self, device=0):
        self.lib = _lib.load()
        h = C.c_void_p()
        check(self.lib.dnb_init(device, C.byref(h)))
        self.h = h
        self.device = device
        self.model = None

    def close(self):
        if self.h:
            self.lib.dnb_shutdown(self.h)
            self.h = None

    # -- plumbing -------------------------------------------------------------
    def set_stream(self, cuda_stream):
        check(self.lib.dnb_set_stream(self.h, C.c_void_p(cuda_stream) if cuda_stream else None))

    def sync(self):
        """Waits for the context's streams; False when a bounded device wait gave up since the
        status was last cleared (the device-pointer calls since then cannot be trusted)."""
        return check(self.lib.dnb_sync(self.h), True)

    def clear_status(self):
        check(self.lib.dnb_clear_status(self.h))

    def set_wait_limits(self, barrier_polls=400000, flag_polls=1 << 21, barrier_bias=0):
        check(self.lib.dnb_set_wait_limits(self.h, barrier_polls, flag_polls, barrier_bias))

    def launch_count(self):
        return int(self.lib.dnb_launch_count(self.h))

    def device_status(self):
        v = C.c_int(0)
        check(self.lib.dnb_device_status(self.h, C.byref(v)))
        return v.value

    def timer_start(self):
        check(self.lib.dnb_timer_start(self.h))

    def timer_stop(self):
        ms = C.c_float()
        check(self.lib.dnb_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def use_graphs(self, on):
        check(self.lib.dnb_use_graphs(self.h, int(on)))

    def stall(self, ms):
        check(self.lib.dnb_stall(self.h, C.c_float(ms)))

    def profile(self, on):
        check(self.lib.dnb_profile_enable(self.h, int(on)))

    def profile_read(self):
        import json
        buf = C.create_string_buffer(16384)
        check(self.lib.dnb_profile_read(self.h, buf, len(buf)))
        return json.loads(buf.value.decode())

    def flush_l2(self):
        check(self.lib.dnb_flush_l2(self.h))

    def dev_alloc(self, nbytes):
        p = C.c_void_p()
        check(self.lib.dnb_dev_alloc(self.h, nbytes, C.byref(p)))
        return p.value

    def dev_free(self, ptr):
        check(self.lib.dnb_dev_free(self.h, C.c_void_p(ptr)))

    def upload(self, ptr, arr):
        arr = np.ascontiguousarray(arr)
        check(self.lib.dnb_dev_upload(self.h, C.c_void_p(ptr), _p(arr), arr.nbytes))

    def dev_copy(self, dst, src, nbytes):
        check(self.lib.dnb_dev_copy(self.h, C.c_void_p(dst), C.c_void_p(src), nbytes))

    def download(self, ptr, arr):
        check(self.lib.dnb_dev_download(self.h, _p(arr), C.c_void_p(ptr), arr.nbytes))
        return arr

    # -- GEMV_V3 path -----------------------------------------------------------
    def register_matrix(self, uid, ty, blocks, k, n):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        return check(self.lib.dnb_register_matrix(self.h, uid, ty, _p(blocks), blocks.nbytes, k, n), True)

    def gemv(self, uid, x, out):
        return check(self.lib.dnb_gemv(self.h, uid, _p(x), _p(out)), True)

    def gemv_dev(self, ty, w_ptr, k, n, x_ptr, out_ptr, nvec=1):
        return check(self.lib.dnb_gemv_dev(self.h, ty, C.c_void_p(w_ptr), k, n, C.c_void_p(x_ptr), C.c_void_p(out_ptr),
                                           nvec), True)

    def set_gemv_impl(self, impl):
        check(self.lib.dnb_set_gemv_impl(self.h, impl))

    def set_tc_min_tokens(self, iq3_xxs_min_tokens):
        """IQ3_XXS layers: token count from which a batch takes the exact-weight tcgen05 grouped GEMM."""
        check(self.lib.dnb_set_tc_min_tokens(self.h, iq3_xxs_min_tokens))

    def set_q4k_int(self, on):
        """Q4_K chunks: three-product bf16 tcgen05 kernel (default, on=False) or the integer-weight kernel (more exact, slower)."""
        check(self.lib.dnb_set_q4k_int(self.h, int(on)))

    def set_router_tc(self, on):
        """Router logits of calls of 16 tokens or more: tcgen05 kernel (default) or the fp32 FMA kernel."""
        check(self.lib.dnb_set_router_tc(self.h, int(on)))

    # -- MoE model ----------------------------------------------------------------
    def moe_config(self, n_layer, n_embd, n_ff, n_expert, n_expert_used, n_shared_ff=0, rms_eps=1e-6,
                   norm_topk_prob=True):
        ok = check(self.lib.dnb_moe_config(self.h, n_layer, n_embd, n_ff, n_shared_ff, n_expert, n_expert_used,
                                           C.c_float(rms_eps), int(norm_topk_prob)), True)
        if ok:
            self.model = dict(n_layer=n_layer, e=n_embd, ff=n_ff, ne=n_expert, k=n_expert_used,
                              sff=n_shared_ff or n_ff)
        return ok

    def set_expert_shard(self, first_expert, n_local):
        """Expert parallel: this context holds routed experts [first, first + n_local)."""
        check(self.lib.dnb_moe_set_expert_shard(self.h, first_expert, n_local))

    def register_experts(self, layer, matrix, ty, n_in, n_out, n_expert, blocks):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        return check(self.lib.dnb_register_experts(self.h, layer, matrix, ty, n_in, n_out, n_expert, _p(blocks),
                                                   blocks.nbytes), True)

    def synth_experts(self, layer, matrix, ty, n_in, n_out, n_expert, seed):
        return check(self.lib.dnb_synth_experts(self.h, layer, matrix, ty, n_in, n_out, n_expert, seed), True)

    def download_expert(self, layer, matrix, expert, nbytes):
        out = np.empty(nbytes, np.uint8)
        check(self.lib.dnb_download_expert(self.h, layer, matrix, expert, _p(out), nbytes))
        return out

    def register_router(self, layer, w, bias=None, norm_w=None, shared_gate_row=None):
        w = _f32(w)
        bias = None if bias is None else _f32(bias)
        norm_w = None if norm_w is None else _f32(norm_w)
        sgr = None if shared_gate_row is None else _f32(shared_gate_row)
        assert w.size == self.model["ne"] * self.model["e"]
        check(self.lib.dnb_register_router(self.h, layer, _p(w), _p(bias), _p(norm_w), _p(sgr)))

    # -- MoE block ------------------------------------------------------------------
    def moe_block(self, layer, h, want_routing=False):
        """Host in, host out.  Returns out[nt,e] (and sels, wts) or None when declined."""
        e, k = self.model["e"], self.model["k"]
        h = _f32(h, (-1, e))
        nt = h.shape[0]
        out = np.empty((nt, e), np.float32)
        sels = np.empty((nt, k), np.int32) if want_routing else None
        wts = np.empty((nt, k), np.float32) if want_routing else None
        if not check(self.lib.dnb_moe_block(self.h, layer, _p(h), nt, _p(out), _p(sels), _p(wts)), True):
            return None
        return (out, sels, wts) if want_routing else out

    def moe_block_into(self, layer, h, out, nt=None):
        """The allocation-free form used in timed loops.  h, out: contiguous fp32 arrays, or the
        pointers host_ptr() made of them once (building a ctypes pointer from an array costs ~2 us,
        a tenth of a decode call); with pointers the token count nt must be given."""
        if nt is None:
            nt = h.shape[0]
        hp = h if isinstance(h, C.c_void_p) else _p(h)
        op = out if isinstance(out, C.c_void_p) else _p(out)
        return check(self.lib.dnb_moe_block(self.h, layer, hp, nt, op, None, None), True)

    def moe_block_dev(self, layer, h_ptr, nt, out_ptr):
        return check(self.lib.dnb_moe_block_dev(self.h, layer, C.c_void_p(h_ptr), nt, C.c_void_p(out_ptr)), True)

    def moe_experts(self, layer, x, sels, wts):
        e = self.model["e"]
        x = _f32(x, (-1, e))
        sels = np.ascontiguousarray(sels, np.int32)
        wts = _f32(wts)
        out = np.empty_like(x)
        if not check(self.lib.dnb_moe_experts(self.h, layer, _p(x), x.shape[0], _p(sels), _p(wts), _p(out)), True):
            return None
        return out

    def router_topk(self, layer, x):
        e, k = self.model["e"], self.model["k"]
        x = _f32(x, (-1, e))
        nt = x.shape[0]
        sels = np.empty((nt, k), np.int32)
        wts = np.empty((nt, k), np.float32)
        rowsum = np.empty(nt, np.float32)
        if not check(self.lib.dnb_router_topk(self.h, layer, _p(x), nt, _p(sels), _p(wts), _p(rowsum)), True):
            return None
        return sels, wts, rowsum

    def router_topk_static(self, layer, x_ptr, nt, sels_ptr, wts_ptr, rowsum_ptr=None):
        """Allocation-free router + top-k on device pointers (asynchronous; see dnb200.h)."""
        return check(self.lib.dnb_router_topk_static(self.h, layer, C.c_void_p(x_ptr), nt, C.c_void_p(sels_ptr),
                                                     C.c_void_p(wts_ptr),
                                                     C.c_void_p(rowsum_ptr) if rowsum_ptr else None), True)

    def grouped_gemm(self, layer, matrix, segs, xs, n_out):
        segs = np.ascontiguousarray(segs, np.uint32)
        xs = _f32(xs)
        m_total = int(segs[:, 1].sum())
        outs = np.empty((m_total, n_out), np.float32)
        if not check(self.lib.dnb_grouped_gemm(self.h, layer, matrix, _p(segs), segs.shape[0], _p(xs), _p(outs)), True):
            return None
        return outs

    def build_grouped_batch(self, layer, sels):
        """moe_expert.rs:8309 build_grouped_batch on the device: (segs[nseg,4], row_token[nt*k], pos[nt,k])."""
        sels = np.ascontiguousarray(sels, np.int32)
        nt, k = sels.shape
        segs = np.zeros((self.model["ne"], 4), np.uint32)
        nseg = C.c_int32(0)
        rtok = np.empty(nt * k, np.int32)
        pos = np.empty((nt, k), np.int32)
        if not check(self.lib.dnb_build_grouped_batch(self.h, layer, _p(sels), nt, _p(segs), C.byref(nseg), _p(rtok), _p(pos)),
                     True):
            return None
        return segs[:nseg.value].copy(), rtok, pos

    def seg_gemv(self, layer, matrix, seg, x, out):
        """Legacy segmented GEMV (cuda.rs:7689 moe_gemv_seg_one): seg[nseg,4] = (expert, m, x_off, out_off)."""
        seg = np.ascontiguousarray(seg, np.uint32)
        x = _f32(x)
        assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"]
        return check(self.lib.dnb_seg_gemv(self.h, layer, matrix, _p(seg), seg.shape[0], _p(x), x.size, _p(out), out.size), True)

    def seg_gemv_pair(self, layer, seg, x, out_g, out_u):
        """cuda.rs:7638 moe_gemv_seg_pair: gate and up of the same segments."""
        seg = np.ascontiguousarray(seg, np.uint32)
        x = _f32(x)
        assert out_g.size == out_u.size
        return check(self.lib.dnb_seg_gemv_pair(self.h, layer, _p(seg), seg.shape[0], _p(x), x.size, _p(out_g), _p(out_u),
                                                out_g.size), True)

    def router_gemv(self, layer, x):
        """cuda.rs:25836 maybe_gpu_router_gemv_into: logits[nt, n_expert], or None when declined."""
        e, ne = self.model["e"], self.model["ne"]
        x = _f32(x, (-1, e))
        out = np.empty((x.shape[0], ne), np.float32)
        if not check(self.lib.dnb_router_gemv(self.h, layer, _p(x), x.shape[0], _p(out)), True):
            return None
        return out

    def register_hc(self, layer, hc, low_rank, w_norm, w_down_inject, w_up):
        """Hyper-connection weights of a layer (model/hyper.rs): fp32, shapes [hc, e], [low_rank + hc, hc * e], [hc * e, low_rank]."""
        e = self.model["e"]
        w_norm, w_down_inject, w_up = _f32(w_norm), _f32(w_down_inject), _f32(w_up)
        assert w_norm.size == hc * e and w_down_inject.size == (low_rank + hc) * hc * e and w_up.size == hc * e * low_rank
        check(self.lib.dnb_register_hc(self.h, layer, hc, low_rank, _p(w_norm), _p(w_down_inject), _p(w_up)))
        self.model.setdefault("hc", {})[layer] = hc

    def hc_moe_block(self, layer, res):
        """res [nt, hc, e] -> out [nt, hc, e] = hc_combine(res, moe_block(hc_mix(res)), inject); None when declined."""
        e = self.model["e"]
        res = _f32(res)
        hc = self.model.get("hc", {}).get(layer, res.shape[-2] if res.ndim >= 2 else 1)
        res = res.reshape(-1, hc, e)
        out = np.empty_like(res)
        if not check(self.lib.dnb_hc_moe_block(self.h, layer, _p(res), res.shape[0], _p(out)), True):
            return None
        return out

    def moe_stack(self, h):
        e = self.model["e"]
        h = _f32(h, (-1, e))
        out = np.empty_like(h)
        if not check(self.lib.dnb_moe_stack(self.h, _p(h), h.shape[0], _p(out)), True):
            return None
        return out

    def moe_stack_dev(self, h_ptr, nt):
        return check(self.lib.dnb_moe_stack_dev(self.h, C.c_void_p(h_ptr), nt), True)


# ---- free functions with the reference's names ----------------------------------

_registered = {}


def maybe_gpu_gguf_gemv_into(uid, ty, blocks, k, n, x, out):
    """cuda.rs:21028-21036.  Weights go resident on first use of `uid`; out[n] is
    written only when True is returned."""
    x = _f32(x)
    if x.size != k or out.size != n or out.dtype != np.float32:
        raise ValueError("gemv: x has %d elements (k=%d), out %d (n=%d)" % (x.size, k, out.size, n))
    ctx = shared_ctx()
    key = (ctx.device, uid)
    if key not in _registered:
        if ty not in TYPE_SIZE or k % BLOCK_ELEMS[ty]:
            return False
        if not ctx.register_matrix(uid, ty, blocks, k, n):
            return False
        _registered[key] = (ty, k, n)
    elif _registered[key] != (ty, k, n):
        raise ValueError("gemv: uid %d was registered as %r" % (uid, _registered[key]))
    return ctx.gemv(uid, x, out)


def pf_router_dev_topk(ctx, layer, xs):
    """cuda.rs:48695-48708: (sels, wts, rowsum) for nt rows, or None."""
    return ctx.router_topk(layer, xs)


def moe_seg_layer_sum(ctx, layer, sels, w, x):
    """cuda.rs:8088-8107: selected experts of one layer for one token (or nt tokens),
    weighted sum in ascending expert order, shared expert added.  None = declined."""
    return ctx.moe_experts(layer, x, sels, w)


def moe_grouped_gemm_layer(ctx, layer, matrix, segs, xs, n_out):
    """cuda.rs:7065-7075 on one matrix: per-segment expert GEMM on packed rows."""
    return ctx.grouped_gemm(layer, matrix, segs, xs, n_out)


def moe_gemv_seg_pair(ctx, layer, seg, x, out_g, out_u):
    """cuda.rs:7638-7650: gate and up segmented GEMVs, results to the host (False = not run)."""
    return ctx.seg_gemv_pair(layer, seg, x, out_g, out_u)


def moe_gemv_seg_one(ctx, layer, seg, x, out):
    """cuda.rs:7689-7698: the down segmented GEMV of the legacy three-launch form."""
    return ctx.seg_gemv(layer, DOWN, seg, x, out)


def maybe_gpu_router_gemv_into(ctx, layer, x, out):
    """cuda.rs:25836: router logits of one row into `out`; False = the caller computes them itself."""
    got = ctx.router_gemv(layer, x)
    if got is None:
        return False
    out[...] = got.reshape(out.shape)
    return True
