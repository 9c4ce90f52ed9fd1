"""GGUF container reader and expert-tensor loader (crates/denno-engine/src/gguf.rs; tests/moe_gguf.rs of
the reference writes its own sparse synthetic files the same way).  The reader needs no GPU; the test that
loads a layer into HBM and runs a block through it is marked gpu."""
import os

import numpy as np
import pytest

from helpers import SEED, gguf_moe_layer_tensors, rel_err, write_gguf


def _kvs(extra=()):
    return [("general.architecture", "str", "qwen4exp"), ("general.alignment", "u32", 64),
            ("qwen4exp.expert_count", "u32", 8), ("qwen4exp.expert_used_count", "u32", 2),
            ("qwen4exp.attention.layer_norm_rms_epsilon", "f32", 1e-6),
            ("tokenizer.ggml.tokens", "arr", ("str", ["a", "bc", "def"])), ("some.ints", "arr", ("i32", [1, -2, 3]))] + list(extra)


def test_single_file_tensor_table_and_bytes(orc, tmp_path):
    from denno_beta_b200 import gguf

    e, ff, ne = 256, 256, 8
    ts, L = gguf_moe_layer_tensors(orc, 3, orc.Q4_K, e, ff, ne, SEED, ty_down=orc.Q8_0)
    path = str(tmp_path / "m.gguf")
    offs = write_gguf(path, _kvs(), ts, alignment=64)
    with gguf.GgufFile(path) as g:
        assert g.tensor_names() == [t[0] for t in ts]
        assert g.meta("general.architecture") == "qwen4exp" and g.meta("qwen4exp.expert_count") == 8
        assert abs(g.meta("qwen4exp.attention.layer_norm_rms_epsilon") - 1e-6) < 1e-12
        assert g.meta("no.such.key") is None and g.tensor("blk.9.x") is None
        for name, ty, dims, data in ts:
            info = g.tensor(name)
            assert info["type"] == ty and info["dims"] == dims and info["part"] == 0
            assert info["offset"] == offs[name] and info["offset"] % 64 == 0 and info["nbytes"] == len(data)
            assert g.tensor_bytes(name).tobytes() == data
        # expert i of an expert-major tensor is one contiguous byte range (moe_expert.rs:49-82)
        info = g.tensor("blk.3.ffn_down_exps.weight")
        eb = info["nbytes"] // ne
        assert eb == e * orc.row_bytes(orc.Q8_0, ff)
        assert g.tensor_bytes("blk.3.ffn_down_exps.weight")[5 * eb:6 * eb].tobytes() == L.keep["down"][5 * eb:6 * eb].tobytes()


def test_split_model_merges_parts_in_split_order(orc, tmp_path):
    """tests/moe_gguf.rs: two shards merge into one table; the parts may be given in any order; metadata comes
    from part 0 first; gaps, duplicates and a wrong split.tensors.count are refused."""
    from denno_beta_b200 import _lib, gguf

    e, ff, ne = 256, 256, 8
    ts0, _ = gguf_moe_layer_tensors(orc, 0, orc.IQ3_XXS, e, ff, ne, SEED)
    ts1, _ = gguf_moe_layer_tensors(orc, 1, orc.Q4_K, e, ff, ne, SEED)
    total = len(ts0) + len(ts1)
    p0, p1 = str(tmp_path / "m-00001-of-00002.gguf"), str(tmp_path / "m-00002-of-00002.gguf")
    split = lambda no, n=total: [("split.no", "u16", no), ("split.count", "u16", 2), ("split.tensors.count", "i32", n)]
    write_gguf(p0, _kvs(split(0)), ts0, alignment=64)
    write_gguf(p1, [("general.alignment", "u32", 32), ("only.in.part1", "u32", 7)] + split(1), ts1)
    with gguf.GgufFile([p1, p0]) as g:  # any order
        assert g.tensor_names() == [t[0] for t in ts0] + [t[0] for t in ts1]
        assert g.tensor("blk.0.ffn_up_exps.weight")["part"] == 0 and g.tensor("blk.1.ffn_up_exps.weight")["part"] == 1
        assert g.meta("general.architecture") == "qwen4exp" and g.meta("only.in.part1") == 7
        assert g.meta("general.alignment") == 64  # part 0 wins
        for name, ty, dims, data in ts1:
            assert g.tensor_bytes(name).tobytes() == data
    with pytest.raises(_lib.DnbError):  # one part of two
        gguf.GgufFile([p0, p0])
    bad = str(tmp_path / "bad.gguf")
    write_gguf(bad, _kvs(split(1, total + 1)), ts1)
    with pytest.raises(_lib.DnbError):  # split.tensors.count disagrees with what the parts hold
        gguf.GgufFile([p0, bad])
    with pytest.raises(_lib.DnbError):  # two files, one without split keys
        write_gguf(bad, _kvs(), ts1)
        gguf.GgufFile([p0, bad])


def test_refuses_what_is_not_gguf(tmp_path):
    from denno_beta_b200 import _lib, gguf

    p = str(tmp_path / "x.gguf")
    open(p, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(_lib.DnbError):
        gguf.GgufFile(p)
    write_gguf(p, [], [("t", 0, [4], b"\0" * 16)], version=1)
    with pytest.raises(_lib.DnbError):
        gguf.GgufFile(p)
    write_gguf(p, [], [("t", 0, [1024], b"\0" * 16)])  # the table promises more bytes than the file holds
    with pytest.raises(_lib.DnbError):
        gguf.GgufFile(p)
    with pytest.raises(_lib.DnbError):
        gguf.GgufFile(str(tmp_path / "missing.gguf"))


@pytest.mark.gpu
def test_layer_loaded_from_a_split_gguf_runs_like_the_oracle(orc, tmp_path):
    """Two layers in two parts -> resident tables -> one decode token and a 24-token chunk per layer against the
    oracle on the same bytes; then the same with only the second half of the experts resident (a rank's shard)."""
    from denno_beta_b200 import cuda as cu, gguf
    from helpers import check_block

    e, ff, ne, k = 512, 256, 16, 3
    ts0, L0 = gguf_moe_layer_tensors(orc, 0, orc.IQ3_XXS, e, ff, ne, SEED, bias=True)
    ts1, L1 = gguf_moe_layer_tensors(orc, 1, orc.Q4_K, e, ff, ne, SEED, ty_down=orc.Q6_K, gate_row=False)
    for L in (L0, L1):
        L.k = k
        L.c.k = k
    p0, p1 = str(tmp_path / "m-00001-of-00002.gguf"), str(tmp_path / "m-00002-of-00002.gguf")
    n = len(ts0) + len(ts1)
    write_gguf(p0, [("split.no", "u16", 0), ("split.count", "u16", 2), ("split.tensors.count", "i32", n)], ts0)
    write_gguf(p1, [("split.no", "u16", 1), ("split.count", "u16", 2), ("split.tensors.count", "i32", n)], ts1)
    c = cu.CudaCtx(0)
    try:
        with gguf.GgufFile([p0, p1]) as g:
            assert c.moe_config(2, e, ff, ne, k)
            for l in (0, 1):
                assert gguf.load_layer(c, g, l, norm_name="ffn_norm.weight")
            assert gguf.load_layer(c, g, 0, gguf_layer=7) is False  # no such block: declined
        for l, L in ((0, L0), (1, L1)):
            for nt in (1, 24):
                h = orc.synth_normal(SEED, 9900 + nt, 1.0, nt * e).reshape(nt, e)
                out, sels, wts = c.moe_block(l, h, want_routing=True)
                err, _ = check_block(orc, L, h, out, sels, wts)
                assert err <= 1e-3, (l, nt, err)
        # a shard: experts 8..15 only; the bytes must be those of the full tensor's second half
        with gguf.GgufFile([p0, p1]) as g:
            assert c.moe_config(1, e, ff, ne, k)
            c.set_expert_shard(8, 8)
            assert gguf.load_layer(c, g, 0, gguf_layer=1)
            eb = L1.keep["gate"].size // ne
            assert np.array_equal(c.download_expert(0, cu.GATE, 0, eb), L1.keep["gate"][8 * eb:9 * eb])
            assert np.array_equal(c.download_expert(0, cu.GATE, 7, eb), L1.keep["gate"][15 * eb:16 * eb])
    finally:
        c.close()
