"""GGUF files as the source of the resident expert table (crates/denno-engine/src/gguf.rs GgufFile;
model/qwen4exp.rs:1915-1963 ExpertW::load).  A thin view of the library's reader: needs no GPU."""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import check

F32, F16, BF16 = 0, 1, 30


class GgufFile:
    """One GGUF file, or all parts of a split model (paths in any order)."""

    def __init__(self, paths):
        if isinstance(paths, (str, bytes)):
            paths = [paths]
        self.lib = _lib.load()
        arr = (C.c_char_p * len(paths))(*[p.encode() if isinstance(p, str) else p for p in paths])
        h = C.c_void_p()
        check(self.lib.dnb_gguf_open(arr, len(paths), C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.lib.dnb_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def tensor_names(self):
        return [self.lib.dnb_gguf_tensor_name(self.h, i).decode() for i in range(self.lib.dnb_gguf_n_tensors(self.h))]

    def tensor(self, name):
        """dict(type, dims, part, offset, nbytes) or None (gguf.rs:402 tensor)."""
        ty, nd, part = C.c_int(), C.c_int(), C.c_int()
        dims = (C.c_uint64 * 4)()
        off, nb = C.c_uint64(), C.c_uint64()
        if not check(self.lib.dnb_gguf_tensor_info(self.h, name.encode(), C.byref(ty), C.byref(nd), dims, C.byref(part), C.byref(off),
                                                   C.byref(nb)), True):
            return None
        return dict(type=ty.value, dims=[int(dims[i]) for i in range(nd.value)], part=part.value, offset=off.value, nbytes=nb.value)

    def tensor_bytes(self, name):
        """The tensor's bytes (a copy of the file mapping), or None (gguf.rs:406 tensor_data)."""
        nb = C.c_uint64()
        p = self.lib.dnb_gguf_tensor_data(self.h, name.encode(), C.byref(nb))
        if not p:
            return None
        return np.ctypeslib.as_array((C.c_uint8 * nb.value).from_address(p)).copy()

    def meta(self, key):
        """A scalar metadata value (int, float or str), or None."""
        s = C.create_string_buffer(512)
        if check(self.lib.dnb_gguf_meta_str(self.h, key.encode(), s, len(s)), True):
            return s.value.decode("utf-8", "replace")
        u, f = C.c_uint64(), C.c_double()
        if not check(self.lib.dnb_gguf_meta_u64(self.h, key.encode(), C.byref(u)), True):
            return None
        check(self.lib.dnb_gguf_meta_f64(self.h, key.encode(), C.byref(f)))
        return f.value if f.value != float(np.int64(np.uint64(u.value))) else int(np.int64(np.uint64(u.value)))


def load_layer(ctx, gguf, layer, gguf_layer=None, norm_name=None):
    """blk.<gguf_layer>'s MoE tensors as layer `layer` of ctx's configured model; False = declined."""
    return check(ctx.lib.dnb_load_gguf_layer(ctx.h, gguf.h, layer, layer if gguf_layer is None else gguf_layer,
                                             norm_name.encode() if norm_name else None), True)
