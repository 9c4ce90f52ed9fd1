"""ctypes binding of libdnb200.so -- the declarations of include/dnb200.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "libdnb200.so")

OK, DECLINED = 0, 1
ERR_ARG, ERR_CUDA, ERR_NO_DEVICE, ERR_STATE = -1, -2, -3, -4

_vp, _i, _u64, _sz, _f = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_float
_fp, _ip, _up = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint32)

# name -> (restype, argtypes); every symbol include/dnb200.h declares
SIGNATURES = {
    "dnb_init": (_i, [_i, C.POINTER(_vp)]),
    "dnb_shutdown": (None, [_vp]),
    "dnb_last_error": (C.c_char_p, []),
    "dnb_set_stream": (_i, [_vp, _vp]),
    "dnb_sync": (_i, [_vp]),
    "dnb_launch_count": (_u64, [_vp]),
    "dnb_device_status": (_i, [_vp, C.POINTER(C.c_int)]),
    "dnb_clear_status": (_i, [_vp]),
    "dnb_set_wait_limits": (_i, [_vp, _i, _i, _i]),
    "dnb_timer_start": (_i, [_vp]),
    "dnb_timer_stop": (_i, [_vp, _fp]),
    "dnb_use_graphs": (_i, [_vp, _i]),
    "dnb_stall": (_i, [_vp, _f]),
    "dnb_profile_enable": (_i, [_vp, _i]),
    "dnb_profile_read": (_i, [_vp, C.c_char_p, _sz]),
    "dnb_dev_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "dnb_dev_free": (_i, [_vp, _vp]),
    "dnb_dev_upload": (_i, [_vp, _vp, _vp, _sz]),
    "dnb_dev_download": (_i, [_vp, _vp, _vp, _sz]),
    "dnb_dev_copy": (_i, [_vp, _vp, _vp, _sz]),
    "dnb_flush_l2": (_i, [_vp]),
    "dnb_register_matrix": (_i, [_vp, _u64, _i, _vp, _sz, _i, _i]),
    "dnb_gemv": (_i, [_vp, _u64, _vp, _vp]),
    "dnb_gemv_dev": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _i]),
    "dnb_set_gemv_impl": (_i, [_vp, _i]),
    "dnb_set_tc_min_tokens": (_i, [_vp, _i]),
    "dnb_set_router_tc": (_i, [_vp, _i]),
    "dnb_set_q4k_int": (_i, [_vp, _i]),
    "dnb_moe_config": (_i, [_vp, _i, _i, _i, _i, _i, _i, _f, _i]),
    "dnb_register_experts": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _sz]),
    "dnb_register_router": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "dnb_synth_experts": (_i, [_vp, _i, _i, _i, _i, _i, _i, _u64]),
    "dnb_download_expert": (_i, [_vp, _i, _i, _i, _vp, _sz]),
    "dnb_gguf_open": (_i, [C.POINTER(C.c_char_p), _i, C.POINTER(_vp)]),
    "dnb_gguf_close": (None, [_vp]),
    "dnb_gguf_n_tensors": (_i, [_vp]),
    "dnb_gguf_tensor_name": (C.c_char_p, [_vp, _i]),
    "dnb_gguf_tensor_info": (_i, [_vp, C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_uint64), C.POINTER(C.c_int),
                                  C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "dnb_gguf_tensor_data": (_vp, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "dnb_gguf_meta_u64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "dnb_gguf_meta_f64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "dnb_gguf_meta_str": (_i, [_vp, C.c_char_p, C.c_char_p, _sz]),
    "dnb_load_gguf_layer": (_i, [_vp, _vp, _i, _i, C.c_char_p]),
    "dnb_moe_block": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "dnb_moe_block_dev": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_moe_experts": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "dnb_router_topk": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "dnb_router_topk_static": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "dnb_grouped_gemm": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp]),
    "dnb_build_grouped_batch": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "dnb_seg_gemv": (_i, [_vp, _i, _i, _vp, _i, _vp, _sz, _vp, _sz]),
    "dnb_seg_gemv_pair": (_i, [_vp, _i, _vp, _i, _vp, _sz, _vp, _vp, _sz]),
    "dnb_router_gemv": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_moe_set_expert_shard": (_i, [_vp, _i, _i]),
    "dnb_moe_route_dev": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "dnb_expert_rows_dev": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp]),
    "dnb_moe_combine_dev": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "dnb_ep_init": (_i, [_vp, _i, _i, _i, _vp]),
    "dnb_ep_connect": (_i, [_vp, _vp]),
    "dnb_ep_block_dev": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_ep_connect_loopback": (_i, [_vp]),
    "dnb_ep_stack_dev": (_i, [_vp, _vp, _i]),
    "dnb_register_hc": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "dnb_hc_moe_block": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_hc_moe_block_dev": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_epd_init": (_i, [_vp, _i, _i, _i, _vp]),
    "dnb_epd_connect": (_i, [_vp, _vp]),
    "dnb_epd_block_dev": (_i, [_vp, _i, _vp, _i, _vp]),
    "dnb_epd_stack_dev": (_i, [_vp, _vp, _i]),
    "dnb_moe_stack": (_i, [_vp, _vp, _i, _vp]),
    "dnb_moe_stack_dev": (_i, [_vp, _vp, _i]),
}

_lib = None


class DnbError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("dnb200 error %d: %s" % (code, text))
        self.code = code


def load():
    """Load the shared library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError("%s is missing: run `python -m denno_beta_b200.build` (there is no CPU path)" % SO_PATH)
        lib = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error():
    return load().dnb_last_error().decode("utf-8", "replace")


def check(rc, allow_declined=False):
    """0 -> True, 1 (declined) -> False when allowed, otherwise raise."""
    if rc == OK:
        return True
    if rc == DECLINED and allow_declined:
        return False
    raise DnbError(rc, last_error())
