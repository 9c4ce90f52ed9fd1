"""The oracle's MoE order against the known answers of the reference's model/moe.rs tests.

The synthetic tensors are the ones model/moe.rs:415-470 describes (n_embd 8, n_ffn 4,
4 experts); the expected outputs are the constants of its tests (moe.rs:538-931),
which came from an independent C program and are required bit for bit.
"""
import numpy as np
import pytest

E, FF, NE = 8, 4, 4
X = np.array([0.5, -1.0, 2.0, 0.25, -0.5, 1.5, -2.0, 1.0], np.float32)


def expert_weights():
    gate = np.zeros((NE, FF, E), np.float32)
    up = np.zeros((NE, FF, E), np.float32)
    down = np.zeros((NE, E, FF), np.float32)
    for e in range(NE):
        for r in range(FF):
            gate[e, r, (r + e) % E] = 1.0
            up[e, r, (r + e + 3) % E] = 1.0
        for j in range(E):
            for c in range(FF):
                down[e, j, c] = np.float32((e + 2 * j + 3 * c) % 7) * np.float32(0.25) - np.float32(0.75)
    return gate, up, down


def gate_inp_main():
    g = np.zeros((NE, E), np.float32)
    g[0, 7] = 1.0
    g[1, 2] = 1.0
    g[2, 0] = 1.0
    g[3, 1] = 0.5
    return g


def gate_inp_tie():
    g = np.zeros((NE, E), np.float32)
    g[0, 7] = 2.0
    g[1, 7] = 1.0
    g[2, 7] = 1.0
    g[3, 1] = 1.0
    return g


def shared_weights():
    sg = np.zeros((2, E), np.float32)
    su = np.zeros((2, E), np.float32)
    sd = np.zeros((E, 2), np.float32)
    sg[0, 3] = 1.0
    sg[1, 5] = 0.5
    su[0, 4] = 1.0
    su[1, 6] = 1.0
    sd[:4, 0] = 1.0
    sd[4:, 1] = 1.0
    return sg, su, sd


def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


BASIC = [1.12409294, 1.06980658, -0.94317919, 0.206427485, 0.475132346, -1.71606886, -0.216211364, 1.12409294]


def run(orc, k=2, norm=True, ginp=None, bias=None, shared=None):
    gate, up, down = expert_weights()
    return orc.moe_ffn_f32(X, k, norm, gate_inp_main() if ginp is None else ginp, bias, gate, up, down, shared)


def test_basic_top2_with_renorm(orc):  # moe.rs:544-578
    assert np.array_equal(bits(run(orc)), bits(BASIC))


def test_norm_topk_prob_false(orc):  # moe.rs:585-620
    want = [0.919029593, 0.874646544, -0.771119237, 0.168769822, 0.388456047, -1.40301406, -0.176768869,
            0.919029593]
    assert np.array_equal(bits(run(orc, norm=False)), bits(want))


def test_tie_breaks_to_lower_index(orc):  # moe.rs:627-671
    want = [1.67379582, -0.455810606, -0.531692863, 1.0155735, -1.08128226, -1.07397342, 0.453390002, 1.67379582]
    wrong = [1.30867004, -0.62427032, 0.230418414, 0.750555038, -1.41422176, -0.255204171, 0.00405269861,
             1.30867004]
    out = run(orc, ginp=gate_inp_tie())
    assert np.array_equal(bits(out), bits(want))
    assert not np.any(bits(out) == bits(wrong))


def test_k_equals_n_expert(orc):  # moe.rs:776-815
    want = [0.836599171, 1.04867744, -0.520942032, -0.011220919, 0.419793457, -1.27453101, -0.498376429,
            0.836599171]
    assert np.array_equal(bits(run(orc, k=NE, norm=False)), bits(want))


def test_shared_expert_adds_once(orc):  # moe.rs:823-856
    want = [1.05382085, 0.999534488, -1.01345122, 0.136155427, -0.543635726, -2.73483706, -1.23497939,
            0.105324864]
    assert np.array_equal(bits(run(orc, shared=shared_weights())), bits(want))


def test_shared_zero_weights_is_identity(orc):  # moe.rs:860-893
    z = (np.zeros((2, E), np.float32), np.zeros((2, E), np.float32), np.zeros((E, 2), np.float32))
    assert np.array_equal(bits(run(orc, shared=z)), bits(BASIC))


def test_gate_inp_bias_shifts_selection(orc):  # moe.rs:899-932
    want = [-0.305793315, 1.44556737, 1.1341424, -1.07012546, 0.368802756, 0.399282575, -1.9718765, -0.305793315]
    out = run(orc, bias=np.array([0, 0, 3.0, 0], np.float32))
    assert np.array_equal(bits(out), bits(want))


def test_select_topk_rules(orc):  # moe.rs:675-683, 759-767
    p = np.array([0.1, 0.3, 0.3, 0.3], np.float32)
    assert list(orc.select_topk(p, 1)) == [1]
    assert list(orc.select_topk(p, 2)) == [1, 2]
    assert list(orc.select_topk(p, 4)) == [0, 1, 2, 3]
    assert list(orc.select_topk(np.array([0.05, 0.4, 0.15, 0.4], np.float32), 3)) == [1, 2, 3]
    nan = np.float32("nan")
    assert list(orc.select_topk(np.array([nan, 0.5, 0.25, nan, 0.75], np.float32), 2)) == [0, 4]
    assert list(orc.select_topk(np.array([0.5, nan, 0.75, 0.25], np.float32), 2)) == [0, 2]
    assert list(orc.select_topk(np.arange(32, dtype=np.float32) % 3, 32)) == list(range(32))


def test_softmax_probabilities(orc):  # moe.rs:540-542 documents these values
    p = orc.softmax(np.array([1.0, 2.0, 0.5, -0.5], np.float32))
    assert np.allclose(p, [0.219879642, 0.597694814, 0.133363739, 0.0490617789], rtol=0, atol=1e-8)


def _quant_layer(orc, ty, e=512, ff=256, ne=16, k=4, shared=True, seed=11, bias=False, gate_row=False):
    nb_gu = ne * ff * e // orc.blck_size(ty)
    nb_d = ne * e * ff // orc.blck_size(ty)
    gate = orc.synth_blocks(ty, seed, 0, nb_gu)
    up = orc.synth_blocks(ty, seed, 1, nb_gu)
    down = orc.synth_blocks(ty, seed, 2, nb_d)
    sh = None
    if shared:
        sh = (orc.synth_blocks(ty, seed, 3, ff * e // orc.blck_size(ty)),
              orc.synth_blocks(ty, seed, 4, ff * e // orc.blck_size(ty)),
              orc.synth_blocks(ty, seed, 5, e * ff // orc.blck_size(ty)))
    rw = orc.synth_normal(seed, 6, 0.02, ne * e).reshape(ne, e)
    rb = orc.synth_zipf_bias(seed, 7, 1.1, ne) if bias else None
    sgr = orc.synth_normal(seed, 8, 0.02, e) if gate_row else None
    return orc.Layer(e, ff, ne, k, ty, ty, ty, gate, up, down, rw, router_bias=rb, norm_w=np.ones(e, np.float32),
                     shared=sh, shared_gate_row=sgr)


@pytest.mark.parametrize("ty_name", ["Q4_K", "IQ3_XXS"])
def test_grouped_form_equals_token_by_token(orc, ty_name):
    # qwen4exp.rs:28259 (batch prefill == sequential) restated for the oracle's two forms
    ty = orc.TYPE_BY_NAME[ty_name]
    L = _quant_layer(orc, ty, bias=True, gate_row=(ty_name == "Q4_K"))
    h = orc.synth_normal(3, 100, 1.0, 9 * L.e).reshape(9, L.e)
    a, sa, wa = orc.moe_block(L, h)
    b, sb, wb = orc.moe_block(L, h, grouped=True)
    assert np.array_equal(sa, sb) and np.array_equal(bits(wa), bits(wb))
    assert np.array_equal(bits(a), bits(b))
    assert np.all(np.diff(sa, axis=1) > 0)  # ascending expert index
    # experts_given with the oracle's own selection reproduces the block
    x = orc.rmsnorm(h, np.ones(L.e, np.float32))
    c = orc.moe_experts_given(L, x, sa, wa)
    assert np.array_equal(bits(a), bits(c))
    # the threaded baseline agrees to rounding
    d = orc.moe_block_mt(L, h)
    assert np.max(np.abs(d - a)) <= 1e-4 * np.sqrt(np.mean(a * a))


def test_segments_sorted_m_desc_then_expert(orc):
    # moe_expert.rs:8309-8390: m descending, ties expert ascending; rows token-ascending inside an expert
    sels = np.array([[0, 3], [1, 3], [2, 3], [0, 1]], np.int32)
    segs, rtok, rslot = orc.build_segments(sels, 4)
    assert segs[:, 0].tolist() == [3, 0, 1, 2] and segs[:, 1].tolist() == [3, 2, 2, 1]
    assert segs[:, 2].tolist() == [0, 3, 5, 7]
    assert rtok.tolist() == [0, 1, 2, 0, 3, 1, 3, 2] and rslot.tolist() == [1, 1, 1, 0, 0, 0, 1, 0]


def test_zipf_bias_is_a_permuted_log_rank(orc):
    b = orc.synth_zipf_bias(5, 7, 1.1, 512)
    want = np.sort((-1.1 * np.log(np.arange(512) + 1.0)).astype(np.float32))
    assert np.array_equal(np.sort(b), want)
    assert not np.array_equal(b, np.sort(b)[::-1])


def test_synth_blocks_distribution(orc):
    w = orc.synth_blocks(orc.Q4_K, 1, 0, 4096).reshape(4096, 144)
    d = w[:, 0:2].copy().view(np.float16).astype(np.float32).ravel()
    assert np.all(np.isfinite(d)) and np.all(d >= 0) and abs(d.mean() - 0.01 * np.sqrt(2 / np.pi)) < 5e-4
    assert abs(w[:, 16:].mean() - 127.5) < 1.0
    q = orc.synth_blocks(orc.IQ3_XXS, 1, 0, 4096).reshape(4096, 98)
    dq = q[:, 0:2].copy().view(np.float16).astype(np.float32).ravel()
    assert abs(dq.mean() - 0.02 * np.sqrt(2 / np.pi)) < 1e-3
    q6 = orc.synth_blocks(orc.Q6_K, 1, 0, 64).reshape(64, 210)
    sc = q6[:, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31
