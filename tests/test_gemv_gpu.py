"""GPU parity of the dequant-GEMV (the GEMV_V3 path) through the C ABI.

Mirrors the reference's GPU tests: tests/moe_gpu.rs (bit-equality of the sequential
kernel with the CPU scalar path) and cuda.rs:45059-45181 (cuda_gemv_v3_matches_cpu:
the fast kernel within a relative bound and different from the sequential one in at
least one row, which proves the fast path ran)."""
import numpy as np
import pytest

from helpers import SEED, rel_err

pytestmark = pytest.mark.gpu

TYPES = ["Q4_K", "IQ3_XXS", "Q6_K", "Q8_0", "Q5_K", "Q5_1", "Q4_0", "IQ4_NL", "IQ4_XS", "IQ3_S", "IQ2_S", "Q2_0"]


@pytest.fixture(scope="module")
def ctx():
    from denno_beta_b200 import cuda as cu

    c = cu.CudaCtx(0)
    yield c
    c.close()


def _case(orc, ty, k, n, tid):
    w = orc.synth_blocks(ty, SEED, tid, n * k // orc.blck_size(ty))
    x = orc.synth_normal(SEED, tid + 1000, 1.0, k)
    return w, x


@pytest.mark.parametrize("name", TYPES)
@pytest.mark.parametrize("k,n", [(4096, 256), (2048, 512), (512, 2048), (256, 40)])
def test_gemv_matches_oracle(orc, ctx, name, k, n):
    ty = orc.TYPE_BY_NAME[name]
    w, x = _case(orc, ty, k, n, ty * 7 + k)
    want = orc.gemv_scalar(ty, w, k, n, x)
    uid = (ty << 32) | (k << 12) | n
    assert ctx.register_matrix(uid, ty, w, k, n)
    got = np.full(n, np.nan, np.float32)
    assert ctx.gemv(uid, x, got)
    err = rel_err(got, want)
    assert err <= 1e-3, "%s %dx%d: max|d|/rms = %.3g" % (name, n, k, err)
    assert err <= 2e-5  # lane-split fp32 is far inside the bar
    again = np.empty_like(got)
    assert ctx.gemv(uid, x, again)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32)), "not bit-identical run to run"


@pytest.mark.parametrize("name", TYPES)
def test_sequential_kernel_is_bit_exact(orc, ctx, name):
    ty = orc.TYPE_BY_NAME[name]
    k, n = 2560, 64  # the shape of tests/moe_gpu.rs
    if k % orc.blck_size(ty):
        k = 2560
    w, x = _case(orc, ty, k, n, ty * 11)
    want = orc.gemv_scalar(ty, w, k, n, x)
    uid = (1 << 60) | ty
    assert ctx.register_matrix(uid, ty, w, k, n)
    fast = np.empty(n, np.float32)
    assert ctx.gemv(uid, x, fast)
    ctx.set_gemv_impl(1)
    try:
        seq = np.empty(n, np.float32)
        assert ctx.gemv(uid, x, seq)
    finally:
        ctx.set_gemv_impl(0)
    assert np.array_equal(seq.view(np.uint32), want.view(np.uint32))
    assert np.any(fast.view(np.uint32) != seq.view(np.uint32)), "fast path did not run"
    assert rel_err(fast, want) <= 2e-5


def test_config0_q4k_4096(orc, ctx):
    """Benchmark config 0: W [4096, 4096] Q4_K, x ~ N(0,1), batch 1."""
    from denno_beta_b200 import cuda as cu

    w, x = _case(orc, orc.Q4_K, 4096, 4096, 1)
    want = orc.gemv_scalar(orc.Q4_K, w, 4096, 4096, x)
    out = np.empty(4096, np.float32)
    assert cu.maybe_gpu_gguf_gemv_into(0xC0F160, cu.Q4_K, w, 4096, 4096, x, out)
    assert rel_err(out, want) <= 1e-3
    truth = orc.gemv_f64(orc.Q4_K, w, 4096, 4096, x)
    # the GPU's lane-split sum is at least as close to the exact result as the sequential one
    assert rel_err(out, truth) <= 2 * rel_err(want, truth) + 1e-7


def test_gemv_dev_multi_vector(orc, ctx):
    ty, k, n, nv = orc.Q4_K, 2048, 512, 6
    w, _ = _case(orc, ty, k, n, 77)
    xs = orc.synth_normal(SEED, 78, 1.0, nv * k).reshape(nv, k)
    dw = ctx.dev_alloc(w.nbytes)
    dx = ctx.dev_alloc(xs.nbytes)
    do = ctx.dev_alloc(nv * n * 4)
    try:
        ctx.upload(dw, w)
        ctx.upload(dx, xs)
        assert ctx.gemv_dev(ty, dw, k, n, dx, do, nv)
        got = ctx.download(do, np.empty((nv, n), np.float32))
    finally:
        for p in (dw, dx, do):
            ctx.dev_free(p)
    for v in range(nv):
        assert rel_err(got[v], orc.gemv_scalar(ty, w, k, n, xs[v])) <= 2e-5


def test_declines_and_errors(orc, ctx):
    from denno_beta_b200 import _lib

    x = np.zeros(256, np.float32)
    out = np.full(4, 7.0, np.float32)
    assert ctx.register_matrix(5, 16, np.zeros(66 * 4, np.uint8), 256, 4) is False  # IQ2_XXS: no kernel
    assert ctx.gemv(5, x, out) is False and np.all(out == 7.0)                      # declined, out untouched
    with pytest.raises(_lib.DnbError):                                               # wrong byte count is misuse
        ctx.register_matrix(6, orc.Q4_K, np.zeros(100, np.uint8), 256, 4)
    assert ctx.register_matrix(7, orc.Q4_K, np.zeros(144, np.uint8), 100, 1) is False  # partial block
