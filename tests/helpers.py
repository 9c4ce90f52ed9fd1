"""Shared builders for the GPU parity tests: one synthetic MoE layer registered with
the CUDA library and described to the CPU oracle from the same bytes."""
import numpy as np

SEED = 0xD3770B200


def make_layer(orc, ctx, layer, ty, e, ff, ne, k, *, shared=True, bias=False, gate_row=False, norm=True, seed=SEED,
               ty_down=None):
    """Generates the layer on the host, registers it and returns the oracle's Layer."""
    from denno_beta_b200 import cuda as cu

    ty_down = ty if ty_down is None else ty_down
    tid = layer * 16
    nb_gu = ne * ff * e // orc.blck_size(ty)
    nb_d = ne * e * ff // orc.blck_size(ty_down)
    gate = orc.synth_blocks(ty, seed, tid + 0, nb_gu)
    up = orc.synth_blocks(ty, seed, tid + 1, nb_gu)
    down = orc.synth_blocks(ty_down, seed, tid + 2, nb_d)
    assert ctx.register_experts(layer, cu.GATE, ty, e, ff, ne, gate)
    assert ctx.register_experts(layer, cu.UP, ty, e, ff, ne, up)
    assert ctx.register_experts(layer, cu.DOWN, ty_down, ff, e, ne, down)
    sh = None
    if shared:
        sh = (orc.synth_blocks(ty, seed, tid + 3, ff * e // orc.blck_size(ty)),
              orc.synth_blocks(ty, seed, tid + 4, ff * e // orc.blck_size(ty)),
              orc.synth_blocks(ty_down, seed, tid + 5, e * ff // orc.blck_size(ty_down)))
        assert ctx.register_experts(layer, cu.SHARED_GATE, ty, e, ff, 1, sh[0])
        assert ctx.register_experts(layer, cu.SHARED_UP, ty, e, ff, 1, sh[1])
        assert ctx.register_experts(layer, cu.SHARED_DOWN, ty_down, ff, e, 1, sh[2])
    rw = orc.synth_normal(seed, tid + 6, 0.02, ne * e).reshape(ne, e)
    rb = orc.synth_zipf_bias(seed, tid + 7, 1.1, ne) if bias else None
    sgr = orc.synth_normal(seed, tid + 8, 0.02, e) if gate_row else None
    nw = np.ones(e, np.float32) if norm else None
    ctx.register_router(layer, rw, rb, nw, sgr)
    return orc.Layer(e, ff, ne, k, ty, ty, ty_down, gate, up, down, rw, router_bias=rb, norm_w=nw, shared=sh,
                     shared_types=(ty, ty, ty_down), shared_gate_row=sgr)


def rel_err(got, want):
    """max |got - want| / rms(want): the path's parity metric (bar 1e-3)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rms = np.sqrt(np.mean(want * want))
    return float(np.max(np.abs(got - want)) / max(rms, 1e-30))


def check_block(orc, L, h, out, sels, wts, tol=1e-3):
    """Parity protocol for a routed block: the selection is compared first; a token
    whose GPU selection differs is accepted only if the oracle's probabilities of the
    swapped experts tie to within 1e-5 relative, and is then re-evaluated under the
    GPU's selection.  Returns (max rel err, number of re-evaluated tokens)."""
    want, osels, owts = orc.moe_block(L, h)
    diff = np.nonzero(np.any(osels != sels, axis=1))[0]
    if diff.size:
        x = orc.rmsnorm(h, L.keep["norm_w"]) if L.keep["norm_w"] is not None else np.asarray(h, np.float32)
        x = x.reshape(-1, L.e)
        _, _, probs = orc.router(x[diff], L.keep["router_w"], L.keep["router_bias"], L.k)
        for n, t in enumerate(diff):
            a = set(osels[t].tolist()) ^ set(sels[t].tolist())
            pv = probs[n][sorted(a)]
            assert (pv.max() - pv.min()) <= 1e-5 * pv.max(), "token %d: selection differs beyond a tie: %r vs %r" % (
                t, osels[t], sels[t])
        want[diff] = orc.moe_experts_given(L, x[diff], sels[diff], wts[diff])
    assert np.max(np.abs(wts - owts)[np.all(osels == sels, axis=1)], initial=0.0) < 2e-6
    return rel_err(out, want), int(diff.size)


# ---- a minimal GGUF v3 writer (the tests write their own synthetic model files, as the reference's
# tests/moe_gguf.rs does) -------------------------------------------------------------------------------
import struct

_GT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
_FMT = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B", "u64": "<Q", "i64": "<q", "f64": "<d"}


def _gstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kvs, tensors, alignment=32, version=3):
    """kvs: [(key, kind, value)] with kind in _GT (arrays: value = (element kind, [values]));
    tensors: [(name, ggml_type, dims (ne0 first), bytes)].  Returns {name: absolute file offset}."""
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kvs))
    for key, kind, val in kvs:
        head += _gstr(key) + struct.pack("<I", _GT[kind])
        if kind == "str":
            head += _gstr(val)
        elif kind == "arr":
            ek, vals = val
            head += struct.pack("<IQ", _GT[ek], len(vals))
            for v in vals:
                head += _gstr(v) if ek == "str" else struct.pack(_FMT[ek], v)
        else:
            head += struct.pack(_FMT[kind], val)
    rel, infos, off = {}, b"", 0
    for name, ty, dims, data in tensors:
        off = (off + alignment - 1) // alignment * alignment
        rel[name] = off
        infos += _gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)
        off += len(data)
    start = (len(head) + len(infos) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + infos)
        f.write(b"\0" * (start - len(head) - len(infos)))
        pos = 0
        for name, ty, dims, data in tensors:
            f.write(b"\0" * (rel[name] - pos))
            f.write(bytes(data))
            pos = rel[name] + len(data)
    return {n: start + o for n, o in rel.items()}


def gguf_moe_layer_tensors(orc, blk, ty, e, ff, ne, seed, ty_down=None, shared=True, gate_row=True, bias=False):
    """The tensors of one MoE layer under the reference's names (qwen4exp.rs:1018-1025), as (name, type, dims, bytes)
    plus the oracle's Layer of the same bytes."""
    ty_down = ty if ty_down is None else ty_down
    tid = blk * 16
    nb = lambda t, rows, cols: rows * cols // orc.blck_size(t)
    gate = orc.synth_blocks(ty, seed, tid + 0, ne * nb(ty, ff, e))
    up = orc.synth_blocks(ty, seed, tid + 1, ne * nb(ty, ff, e))
    down = orc.synth_blocks(ty_down, seed, tid + 2, ne * nb(ty_down, e, ff))
    rw = orc.synth_normal(seed, tid + 6, 0.02, ne * e)
    p = "blk.%d." % blk
    ts = [(p + "ffn_gate_inp.weight", 0, [e, ne], rw.tobytes()),
          (p + "ffn_gate_exps.weight", ty, [e, ff, ne], gate.tobytes()),
          (p + "ffn_up_exps.weight", ty, [e, ff, ne], up.tobytes()),
          (p + "ffn_down_exps.weight", ty_down, [ff, e, ne], down.tobytes())]
    sh = sgr = rb = None
    if shared:
        sh = (orc.synth_blocks(ty, seed, tid + 3, nb(ty, ff, e)), orc.synth_blocks(ty, seed, tid + 4, nb(ty, ff, e)),
              orc.synth_blocks(ty_down, seed, tid + 5, nb(ty_down, e, ff)))
        ts += [(p + "ffn_gate_shexp.weight", ty, [e, ff], sh[0].tobytes()), (p + "ffn_up_shexp.weight", ty, [e, ff], sh[1].tobytes()),
               (p + "ffn_down_shexp.weight", ty_down, [ff, e], sh[2].tobytes())]
        if gate_row:
            sgr = orc.synth_normal(seed, tid + 8, 0.02, e)
            ts.append((p + "ffn_gate_inp_shexp.weight", 0, [e], sgr.tobytes()))
    if bias:
        rb = orc.synth_zipf_bias(seed, tid + 7, 1.1, ne)
        ts.append((p + "exp_probs_b.bias", 0, [ne], rb.tobytes()))
    nw = (1.0 + 0.1 * orc.synth_normal(seed, tid + 9, 1.0, e)).astype(np.float32)
    ts.append((p + "ffn_norm.weight", 0, [e], nw.tobytes()))
    L = orc.Layer(e, ff, ne, 0, ty, ty, ty_down, gate, up, down, rw.reshape(ne, e), router_bias=rb, norm_w=nw, shared=sh,
                  shared_types=(ty, ty, ty_down), shared_gate_row=sgr)
    return ts, L
