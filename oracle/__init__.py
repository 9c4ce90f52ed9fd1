"""CPU oracle (test infrastructure): ctypes view of ``oracle/dnb_oracle.c``.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the library in ``denno_beta_b200`` never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libdnb_oracle.so")

# ggml type ids (kquant.rs:72-104 of the reference)
Q4_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K = 2, 7, 8, 12, 13, 14
IQ3_XXS, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS, Q2_0 = 18, 20, 21, 22, 23, 42
TYPE_BY_NAME = {
    "Q4_0": Q4_0, "Q4_0_EDGE": Q4_0, "Q5_1": Q5_1, "Q8_0": Q8_0, "Q4_K": Q4_K, "Q5_K": Q5_K, "Q6_K": Q6_K,
    "IQ3_XXS": IQ3_XXS, "IQ4_NL": IQ4_NL, "IQ3_S": IQ3_S, "IQ2_S": IQ2_S, "IQ4_XS": IQ4_XS, "Q2_0": Q2_0,
}


def build(force=False):
    """Compile the oracle with the Makefile next to it (gcc, a second or two)."""
    srcs = [os.path.join(_HERE, f) for f in ("dnb_oracle.c", "dnb_cpu_fast.c", "dnb_oracle.h", "Makefile")]
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(f) for f in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


class MoeLayer(C.Structure):
    _fields_ = [
        ("e", C.c_long), ("ff", C.c_long), ("ne", C.c_long), ("k", C.c_long), ("sff", C.c_long),
        ("norm_topk", C.c_int),
        ("ty_gate", C.c_int), ("ty_up", C.c_int), ("ty_down", C.c_int),
        ("ty_sgate", C.c_int), ("ty_sup", C.c_int), ("ty_sdown", C.c_int),
        ("eps", C.c_float),
        ("norm_w", C.c_void_p), ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
        ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
        ("sgate", C.c_void_p), ("sup", C.c_void_p), ("sdown", C.c_void_p),
        ("shared_gate_row", C.c_void_p),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_row_bytes.restype = C.c_long
        L.orc_row_bytes.argtypes = [C.c_int, C.c_long]
        L.orc_silu.restype = C.c_float
        L.orc_silu.argtypes = [C.c_float]
        L.orc_sigmoid.restype = C.c_float
        L.orc_sigmoid.argtypes = [C.c_float]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def type_size(ty):
    return lib().orc_type_size(ty)


def blck_size(ty):
    return lib().orc_blck_size(ty)


def row_bytes(ty, n_in):
    rb = lib().orc_row_bytes(ty, n_in)
    if rb < 0:
        raise ValueError("n_in=%d is not a whole number of blocks of type %d" % (n_in, ty))
    return rb


def dequant_row(ty, blocks, n):
    blocks = _u8(blocks)
    out = np.empty(n, np.float32)
    if lib().orc_dequant_row(C.c_int(ty), _p(blocks), C.c_long(n), _p(out)) != 0:
        raise ValueError("dequant_row: bad type/length")
    return out


def gemv_scalar(ty, blocks, n_in, n_out, x):
    blocks, x = _u8(blocks), _f32(x)
    assert blocks.size == n_out * row_bytes(ty, n_in) and x.size == n_in
    out = np.empty(n_out, np.float32)
    lib().orc_gemv_scalar(C.c_int(ty), _p(blocks), C.c_long(n_in), C.c_long(n_out), _p(x), _p(out))
    return out


def gemv_f64(ty, blocks, n_in, n_out, x):
    blocks, x = _u8(blocks), _f32(x)
    out = np.empty(n_out, np.float64)
    lib().orc_gemv_f64(C.c_int(ty), _p(blocks), C.c_long(n_in), C.c_long(n_out), _p(x), _p(out))
    return out


def gemv_mt(ty, blocks, n_in, n_out, x):
    blocks, x = _u8(blocks), _f32(x)
    out = np.empty(n_out, np.float32)
    lib().orc_gemv_mt(C.c_int(ty), _p(blocks), C.c_long(n_in), C.c_long(n_out), _p(x), _p(out))
    return out


def rmsnorm(x, w, eps=1e-6):
    x = _f32(x)
    w = _f32(w)
    cols = w.size
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), C.c_long(x.size // cols), C.c_long(cols), C.c_float(eps), _p(out))
    return out


def softmax(x):
    x = _f32(x).copy()
    lib().orc_softmax(_p(x), C.c_long(x.size))
    return x


def hc_mix(x, w_norm, w_down_inject, w_up, low_rank, eps=1e-6):
    """model/hyper.rs:160-222 for one token: x [hc, e] -> (mixed [e], inject [hc], xn [hc, e])."""
    x = _f32(x)
    hc, e = x.shape
    w_norm, w_down_inject, w_up = _f32(w_norm), _f32(w_down_inject), _f32(w_up)
    assert w_norm.size == hc * e and w_down_inject.size == (low_rank + hc) * hc * e and w_up.size == hc * e * low_rank
    mixed = np.empty(e, np.float32)
    inject = np.empty(hc, np.float32)
    xn = np.empty((hc, e), np.float32)
    L = lib()
    L.orc_hc_mix.restype = None
    L.orc_hc_mix.argtypes = [C.c_void_p] * 4 + [C.c_long] * 3 + [C.c_float] + [C.c_void_p] * 3
    L.orc_hc_mix(_p(x), _p(w_norm), _p(w_down_inject), _p(w_up), hc, e, low_rank, eps, _p(mixed), _p(inject), _p(xn))
    return mixed, inject, xn


def hc_combine(residual, block, inject):
    """model/hyper.rs:384-416: residual [hc, e], block [e], inject [hc] -> [hc, e]."""
    residual, block, inject = _f32(residual), _f32(block), _f32(inject)
    hc, e = residual.shape
    out = np.empty((hc, e), np.float32)
    L = lib()
    L.orc_hc_combine.restype = None
    L.orc_hc_combine.argtypes = [C.c_void_p] * 3 + [C.c_long] * 2 + [C.c_void_p]
    L.orc_hc_combine(_p(residual), _p(block), _p(inject), hc, e, _p(out))
    return out


def select_topk(probs, k):
    probs = _f32(probs)
    out = np.empty(k, np.int32)
    lib().orc_select_topk(_p(probs), C.c_long(probs.size), C.c_long(k), _p(out))
    return out


def router(x, w_r, bias, k, norm_topk=True):
    """Returns (sels[nt,k] int32 ascending, wts[nt,k], probs[nt,ne])."""
    w_r = _f32(w_r)
    ne, e = w_r.shape
    x = _f32(x).reshape(-1, e)
    nt = x.shape[0]
    bias = None if bias is None else _f32(bias)
    sels = np.empty((nt, k), np.int32)
    wts = np.empty((nt, k), np.float32)
    probs = np.empty((nt, ne), np.float32)
    lib().orc_router(_p(x), C.c_long(nt), C.c_long(e), _p(w_r), _p(bias), C.c_long(ne), C.c_long(k),
                     C.c_int(1 if norm_topk else 0), _p(sels), _p(wts), _p(probs))
    return sels, wts, probs


def moe_ffn_f32(x, k, norm_topk, gate_inp, bias, gate_exps, up_exps, down_exps, shared=None):
    """moe.rs::moe_ffn on fp32 tensors. gate_exps [ne,ff,e], down_exps [ne,e,ff]."""
    x = _f32(x)
    gate_inp, gate_exps, up_exps, down_exps = map(_f32, (gate_inp, gate_exps, up_exps, down_exps))
    ne, ff, e = gate_exps.shape
    bias = None if bias is None else _f32(bias)
    sg = su = sd = None
    sff = 0
    if shared is not None:
        sg, su, sd = map(_f32, shared)
        sff = sg.shape[0]
    out = np.empty(e, np.float32)
    lib().orc_moe_ffn_f32(_p(x), C.c_long(e), C.c_long(ff), C.c_long(ne), C.c_long(k), C.c_int(int(norm_topk)),
                          _p(gate_inp), _p(bias), _p(gate_exps), _p(up_exps), _p(down_exps),
                          _p(sg), _p(su), _p(sd), C.c_long(sff), _p(out))
    return out


class Layer:
    """Keeps the numpy buffers of one MoE layer alive next to the C struct."""

    def __init__(self, e, ff, ne, k, ty_gate, ty_up, ty_down, gate, up, down, router_w, router_bias=None,
                 norm_w=None, eps=1e-6, shared=None, shared_types=None, shared_gate_row=None, norm_topk=True):
        self.keep = dict(gate=_u8(gate), up=_u8(up), down=_u8(down), router_w=_f32(router_w))
        self.keep["router_bias"] = None if router_bias is None else _f32(router_bias)
        self.keep["norm_w"] = None if norm_w is None else _f32(norm_w)
        self.keep["sgr"] = None if shared_gate_row is None else _f32(shared_gate_row)
        sff = 0
        st = (0, 0, 0)
        if shared is not None:
            self.keep["sg"], self.keep["su"], self.keep["sd"] = map(_u8, shared)
            st = shared_types if shared_types is not None else (ty_gate, ty_up, ty_down)
            sff = self.keep["sg"].size // row_bytes(st[0], e)
        else:
            self.keep["sg"] = self.keep["su"] = self.keep["sd"] = None
        assert self.keep["gate"].size == ne * ff * row_bytes(ty_gate, e)
        assert self.keep["up"].size == ne * ff * row_bytes(ty_up, e)
        assert self.keep["down"].size == ne * e * row_bytes(ty_down, ff)
        assert self.keep["router_w"].size == ne * e
        kp = self.keep
        self.c = MoeLayer(e, ff, ne, k, sff, int(norm_topk), ty_gate, ty_up, ty_down, st[0], st[1], st[2], eps,
                          _p(kp["norm_w"]), _p(kp["router_w"]), _p(kp["router_bias"]),
                          _p(kp["gate"]), _p(kp["up"]), _p(kp["down"]), _p(kp["sg"]), _p(kp["su"]), _p(kp["sd"]),
                          _p(kp["sgr"]))
        self.e, self.ff, self.ne, self.k = e, ff, ne, k


def moe_block(layer, h, grouped=False):
    """(RMSNorm) -> router -> experts -> sum -> shared for nt tokens. Returns (out, sels, wts)."""
    h = _f32(h).reshape(-1, layer.e)
    nt = h.shape[0]
    out = np.empty((nt, layer.e), np.float32)
    sels = np.empty((nt, layer.k), np.int32)
    wts = np.empty((nt, layer.k), np.float32)
    fn = lib().orc_moe_block_grouped if grouped else lib().orc_moe_block
    rc = fn(C.byref(layer.c), _p(h), C.c_long(nt), _p(out), _p(sels), _p(wts))
    if rc != 0:
        raise ValueError("moe_block: bad layer description")
    return out, sels, wts


def moe_block_mt(layer, h):
    h = _f32(h).reshape(-1, layer.e)
    out = np.empty((h.shape[0], layer.e), np.float32)
    lib().orc_moe_block_mt(C.byref(layer.c), _p(h), C.c_long(h.shape[0]), _p(out))
    return out


# ---- the timed CPU baseline (oracle/dnb_cpu_fast.c): AVX2+FMA kernels in the reference's production form ----

def set_threads(n):
    """OpenMP threads of the timed legs (0 = the runtime's default).  Set explicitly: a launcher
    such as torch.distributed.run exports OMP_NUM_THREADS=1 to its children."""
    lib().orc_set_threads(C.c_int(int(n)))


def get_threads():
    return int(lib().orc_get_threads())


def fast_gemv(ty, blocks, n_in, n_out, x):
    blocks, x = _u8(blocks), _f32(x)
    assert blocks.size == n_out * row_bytes(ty, n_in) and x.size == n_in
    out = np.empty(n_out, np.float32)
    if lib().orc_fast_gemv(C.c_int(ty), _p(blocks), C.c_long(n_in), C.c_long(n_out), _p(x), _p(out)) != 0:
        raise ValueError("fast_gemv: bad type/length")
    return out


def fast_moe_block(layer, h, grouped=False):
    """One block for nt tokens: token by token in the decode form, or grouped by expert with the
    k-chunked batch kernels (the prefill form)."""
    h = _f32(h).reshape(-1, layer.e)
    out = np.empty((h.shape[0], layer.e), np.float32)
    fn = lib().orc_fast_moe_block_grouped if grouped else lib().orc_fast_moe_block
    if fn(C.byref(layer.c), _p(h), C.c_long(h.shape[0]), _p(out)) != 0:
        raise ValueError("fast_moe_block: layer shape not covered")
    return out


def moe_experts_given(layer, x, sels, wts):
    x = _f32(x).reshape(-1, layer.e)
    sels = np.ascontiguousarray(sels, np.int32)
    wts = _f32(wts)
    out = np.empty_like(x)
    lib().orc_moe_experts_given(C.byref(layer.c), _p(x), C.c_long(x.shape[0]), _p(sels), _p(wts), _p(out))
    return out


def grouped_gemm(ty, w_all, n_in, n_out, segs, xs):
    """segs: int array [nseg,4] = (expert, m, x_off rows, out_off rows)."""
    segs = np.ascontiguousarray(segs, np.uint32)
    xs = _f32(xs)
    m_total = int(segs[:, 1].sum())
    outs = np.empty((m_total, n_out), np.float32)
    w_all = _u8(w_all)
    lib().orc_grouped_gemm(C.c_int(ty), _p(w_all), C.c_long(n_in), C.c_long(n_out), _p(segs),
                           C.c_long(segs.shape[0]), _p(xs), _p(outs))
    return outs


def build_segments(sels, ne):
    sels = np.ascontiguousarray(sels, np.int32)
    nt, k = sels.shape
    segs = np.zeros((ne, 4), np.uint32)
    rtok = np.empty(nt * k, np.int32)
    rslot = np.empty(nt * k, np.int32)
    mt = C.c_long(0)
    nseg = lib().orc_build_segments(_p(sels), C.c_long(nt), C.c_long(k), C.c_long(ne), _p(segs), _p(rtok),
                                    _p(rslot), C.byref(mt))
    return segs[:nseg].copy(), rtok[:mt.value].copy(), rslot[:mt.value].copy()


def synth_blocks(ty, seed, tensor_id, n_blocks):
    out = np.empty(n_blocks * type_size(ty), np.uint8)
    lib().orc_synth_blocks(C.c_int(ty), C.c_uint64(seed), C.c_uint64(tensor_id), _p(out), C.c_uint64(n_blocks))
    return out


def synth_normal(seed, tensor_id, sigma, n):
    out = np.empty(n, np.float32)
    lib().orc_synth_normal(C.c_uint64(seed), C.c_uint64(tensor_id), C.c_float(sigma), _p(out), C.c_uint64(n))
    return out


def synth_zipf_bias(seed, tensor_id, s, n):
    out = np.empty(n, np.float32)
    lib().orc_synth_zipf_bias(C.c_uint64(seed), C.c_uint64(tensor_id), C.c_double(s), _p(out), C.c_uint32(n))
    return out
