"""Hyper-connection mix / combine around the MoE block (model/hyper.rs; call sites model/qwen4exp.rs:3722-3765).

CPU: the oracle's restatement against the reference's own hard-coded anchor (crates/denno-engine/tests/hyper.rs:321-365),
whose inputs come from the 64-bit LCG of that test file (tests/hyper.rs:15-35) and whose expected values the reference
fixed after checking them with an independent sequential-f32 implementation; and against its closed-form cases
(zero weights -> half the mean of the normed streams; inject 0 -> plain residual add).
GPU: the CUDA mix -> block -> combine against the oracle.
"""
import numpy as np
import pytest

from helpers import SEED, make_layer, rel_err

# tests/hyper.rs:353-365
ANCHOR_MIXED = np.array([-0.2145072, -0.1952698, 0.053666078, -0.19590339], np.float32)
ANCHOR_INJECT = np.array([-0.0070681423, 0.17874321], np.float32)
ANCHOR_COMBINE = np.array(
    [-0.050585628, -0.6392422, 1.6860697, -0.19153804, -0.004251361, -0.778245, 1.8945739, -0.26103944], np.float32
)


class Lcg:
    """tests/hyper.rs:15-35: x <- x * 6364136223846793005 + 1442695040888963407 (mod 2^64); top 24 bits / 2^23 - 1."""

    def __init__(self, seed):
        self.x = seed

    def vec(self, n):
        out = np.empty(n, np.float32)
        for i in range(n):
            self.x = (self.x * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            out[i] = np.float32(np.float32(self.x >> 40) / np.float32(8388608.0)) - np.float32(1.0)
        return out


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_oracle_matches_the_reference_anchor(orc):
    hc, e, lr = 2, 4, 3
    rng = Lcg(0x51ED0008)
    embd = rng.vec(e)
    x = np.tile(embd, (hc, 1))  # HyperStreams::from_embed: hc copies of the embedding
    w_norm = rng.vec(hc * e)
    w_down = rng.vec(lr * hc * e)
    w_up = rng.vec(hc * e * lr)
    inject_rows = rng.vec(hc * hc * e)
    mixed, inject, _ = orc.hc_mix(x, w_norm, np.concatenate([w_down, inject_rows]), w_up, lr, 1e-6)
    assert (bits(mixed) == bits(ANCHOR_MIXED)).all(), (mixed, ANCHOR_MIXED)
    assert (bits(inject) == bits(ANCHOR_INJECT)).all(), (inject, ANCHOR_INJECT)
    out = orc.hc_combine(x, np.array([0.5, -1.5, 2.25, -0.75], np.float32), ANCHOR_INJECT)
    assert (bits(out.reshape(-1)) == bits(ANCHOR_COMBINE)).all(), (out, ANCHOR_COMBINE)


def test_oracle_closed_forms(orc):
    # tests/hyper.rs:167-207: zero weights -> gate 0 -> sigmoid 0.5 -> half the mean of the normed streams
    hc, e, lr = 3, 4, 2
    x = np.ones((hc, e), np.float32)
    mixed, inject, _ = orc.hc_mix(x, np.ones(hc * e, np.float32), np.zeros((lr + hc) * hc * e, np.float32),
                                  np.zeros(hc * e * lr, np.float32), lr, 0.0)
    assert (bits(mixed) == bits(np.full(e, 0.5, np.float32))).all()
    assert (bits(inject) == 0).all()
    # tests/hyper.rs:57-100: inject 0 -> w = 1 -> plain residual add
    res = Lcg(0x51ED0001).vec(hc * e).reshape(hc, e)
    blk = np.array([0.25, -1.0, 3.0, 0.5], np.float32)
    out = orc.hc_combine(res, blk, np.zeros(hc, np.float32))
    assert (bits(out) == bits(res + blk[None, :])).all()
    # hc = 1 passes through (tests/hyper.rs:272-290)
    one = orc.hc_combine(res[:1], blk, np.zeros(1, np.float32))
    assert (bits(one) == bits(res[:1] + blk)).all()


def hc_weights(orc, hc, e, lr, layer):
    w_norm = 1.0 + 0.1 * orc.synth_normal(SEED, 7000 + layer, 1.0, hc * e)
    w_down = orc.synth_normal(SEED, 7100 + layer, 1.0 / np.sqrt(hc * e), (lr + hc) * hc * e)
    w_up = orc.synth_normal(SEED, 7200 + layer, 2.0 / np.sqrt(lr), hc * e * lr)
    return w_norm, w_down, w_up


@pytest.mark.gpu
@pytest.mark.parametrize("shape,nts", [((512, 256, 16, 4, 1, 4, 32), (1, 5)), ((2048, 512, 256, 8, 1, 4, 320), (1, 3, 40))])
def test_hc_block_matches_the_oracle(orc, shape, nts):
    from denno_beta_b200 import cuda as cu

    e, ff, ne, k, shared, hc, lr = shape
    c = cu.CudaCtx(0)
    try:
        assert c.moe_config(1, e, ff, ne, k)
        L = make_layer(orc, c, 0, orc.IQ3_XXS, e, ff, ne, k, shared=shared, norm=False)
        w_norm, w_down, w_up = hc_weights(orc, hc, e, lr, 0)
        assert c.hc_moe_block(0, np.zeros((1, hc, e), np.float32)) is None  # nothing registered yet: declined
        c.register_hc(0, hc, lr, w_norm, w_down, w_up)
        for nt in nts:
            res = orc.synth_normal(SEED, 7300 + nt, 1.0, nt * hc * e).reshape(nt, hc, e)
            got = c.hc_moe_block(0, res)
            again = c.hc_moe_block(0, res)
            assert (bits(got) == bits(again)).all(), "run-to-run bits"
            want = np.empty_like(res)
            mixed_all = np.empty((nt, e), np.float32)
            injects = []
            for t in range(nt):
                mixed_all[t], inj, _ = orc.hc_mix(res[t], w_norm, w_down, w_up, lr, 1e-6)
                injects.append(inj)
            blk = orc.moe_block(L, mixed_all)[0]
            for t in range(nt):
                want[t] = orc.hc_combine(res[t], blk[t], injects[t])
            err = rel_err(got, want)
            assert err <= 1e-3, "nt %d: %.3g" % (nt, err)
            # the streams differ only by the block's output times 2*sigmoid(inject[s])
            d = (got - res)[:, :, :]
            for t in range(nt):
                w = 2.0 / (1.0 + np.exp(-injects[t].astype(np.float64)))
                np.testing.assert_allclose(d[t, 1] * w[0], d[t, 0] * w[1], rtol=2e-3, atol=2e-4 * np.abs(d[t]).max())
    finally:
        c.close()
