"""CPU-side checks of the boundary: the shared library builds, loads and exports every
symbol include/dnb200.h declares; the Python mirror validates its arguments; and
without a CUDA device the library refuses to run instead of falling back."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def so_path():
    from denno_beta_b200 import build

    return build.build()


def _declared():
    text = open(os.path.join(ROOT, "include", "dnb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dnb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(so_path):
    out = subprocess.check_output(["nm", "-D", "--defined-only", so_path], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    declared = _declared()
    assert len(declared) >= 25
    missing = [s for s in declared if s not in exported]
    assert not missing, "declared in dnb200.h but not exported: %s" % missing
    extra = sorted(s for s in exported if s.startswith("dnb_") and s not in declared)
    assert not extra, "exported but not declared in dnb200.h: %s" % extra


def test_binding_covers_the_header(so_path):
    from denno_beta_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared()
    _lib.load()


def test_synth_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "dnb_synth.h"\n#include "dnb200.h"\nint main(void){unsigned char b[144];'
                   'dnb_synth_fill_blocks_host(12,1,2,b,1);return b[0]==255?2:0;}\n')
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-Wno-unused-function",
                           "-I" + os.path.join(ROOT, "include"), str(src), "-lm", "-o", str(tmp_path / "t")])


def _has_gpu():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="a CUDA device is present")
def test_no_device_means_no_result(so_path):
    from denno_beta_b200 import _lib, cuda as cu

    lib = _lib.load()
    h = C.c_void_p()
    assert lib.dnb_init(0, C.byref(h)) == _lib.ERR_NO_DEVICE
    assert "no CPU path" in _lib.last_error()
    assert cu.cuda_enabled() is False
    with pytest.raises(_lib.DnbError):
        cu.maybe_gpu_gguf_gemv_into(1, cu.Q4_K, np.zeros(144, np.uint8), 256, 1, np.zeros(256, np.float32),
                                    np.zeros(1, np.float32))


def test_mirror_validates_shapes():
    from denno_beta_b200 import cuda as cu

    assert cu.row_bytes(cu.Q4_K, 4096) == 16 * 144
    assert cu.row_bytes(cu.IQ3_XXS, 2048) == 8 * 98
    with pytest.raises(ValueError):
        cu.row_bytes(cu.Q4_K, 100)
    with pytest.raises(ValueError):  # length mismatch is misuse, not "declined" (cuda.rs:8120-8126)
        cu.maybe_gpu_gguf_gemv_into(2, cu.Q4_K, np.zeros(144, np.uint8), 256, 1, np.zeros(255, np.float32),
                                    np.zeros(1, np.float32))


def test_product_never_touches_the_oracle():
    bad = []
    for dirpath, _, files in os.walk(os.path.join(ROOT, "denno_beta_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                if re.search(r"\boracle\b|dnb_oracle|orc_", text):
                    bad.append(os.path.join(dirpath, f))
    assert not bad, "library files that mention the oracle: %s" % bad
