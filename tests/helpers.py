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
