"""ctypes binding of libmoexb.so (the C ABI declared in include/moexb.h).

The library is the product: there is no Python or CPU fallback. If it is missing the import of any compute entry point
fails with instructions to build it (python -m moe_b200.build).
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmoexb.so")

FMT_SYM_F32, FMT_SYM_F16, FMT_ZP = 0, 1, 2
F32, BF16, F16 = 0, 1, 2
LAYOUT_TILED, LAYOUT_REFERENCE = 0, 1
EH, EI, EGS = 2048, 512, 64
Q_BYTES = 3 * EH * EI // 2
CHUNKS = 3 * EH * EI // 32


class MoexbError(RuntimeError):
    pass


class PairItem(C.Structure):  # moexb_pair_item, kernels.cuh:688
    _fields_ = [("slot", C.c_void_p), ("start", C.c_int), ("count", C.c_int)]


class Pair(C.Structure):  # moexb_pair, kernels.cuh:689
    _fields_ = [("t", C.c_int), ("p", C.c_int), ("w", C.c_float)]


_vp, _i, _u, _ll = C.c_void_p, C.c_int, C.c_uint, C.c_longlong

# name -> (restype, argtypes); every symbol include/moexb.h declares
SIGNATURES = {
    "moexb_last_error": (C.c_char_p, []),
    "moexb_version": (_i, []),
    "moexb_expert_bytes": (C.c_size_t, [_i]),
    "moexb_gemv_f16": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i]),
    "moexb_gemv_f32": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i]),
    "moexb_router_topk": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _i]),
    "moexb_experts_forward": (_i, [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "moexb_set_default_ctx": (_i, [_vp, _i]),
    "moexb_experts_forward_static": (_i, [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp]),
    "moexb_pairs_forward": (_i, [_i, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "moexb_pairs_forward_dev": (_i, [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "moexb_pairs_forward_tc": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _vp, _vp, _vp]),
    "moexb_ctx_set_path": (_i, [_vp, _i]),
    "moexb_ctx_set_prefill_min_tokens": (_i, [_vp, _i]),
    "moexb_ctx_set_pairs_per_pass": (_i, [_vp, _i]),
    "moexb_ctx_set_fused_decode": (_i, [_vp, _i]),
    "moexb_ctx_status": (_i, [_vp, C.POINTER(_i)]),
    "moexb_ctx_selftest_timeout": (_i, [_vp, _i, _i, C.POINTER(_i)]),
    "moexb_pairs_reduce": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "moexb_gated_add_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "moexb_shared_expert_add": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "moexb_group_pairs": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "moexb_dequant": (_i, [_i, _vp, _vp, _vp]),
    "moexb_q4k_dequant": (_i, [_vp, _ll, _vp, _vp]),
    "moexb_q4k_to_zp": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "moexb_synth_experts": (_i, [_vp, _i, _u, _i, _i, _i, _vp, _vp]),
    "moexb_synth_expert_host": (_i, [_i, _u, _i, _i, _vp]),
    "moexb_synth_q4k_host": (_i, [_u, _i, _i, _vp, _vp, _vp]),
    "moexb_ctx_create": (_i, [_i, _i, _i, _i, C.POINTER(_vp)]),
    "moexb_ctx_destroy": (_i, [_vp]),
    "moexb_layer_create": (_i, [_vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "moexb_layer_destroy": (_i, [_vp]),
    "moexb_layer_blob": (_vp, [_vp, _i]),
    "moexb_layer_slot_table": (_vp, [_vp]),
    "moexb_layer_upload_expert": (_i, [_vp, _i, _vp]),
    "moexb_layer_export_expert": (_i, [_vp, _i, _vp]),
    "moexb_layer_set_router": (_i, [_vp, _vp]),
    "moexb_layer_router": (_vp, [_vp]),
    "moexb_layer_fill_synth": (_i, [_vp, _u, _i, _vp]),
    "moexb_gguf_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "moexb_gguf_close": (_i, [_vp]),
    "moexb_gguf_tensor_count": (_i, [_vp]),
    "moexb_gguf_tensor_name": (C.c_char_p, [_vp, _i]),
    "moexb_gguf_tensor": (_i, [_vp, C.c_char_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_ll), C.POINTER(_vp), C.POINTER(_ll)]),
    "moexb_gguf_dequant_host": (_i, [_i, _vp, _ll, _vp]),
    "moexb_gguf_row_to_zp": (_i, [_i, _vp, _i, _vp, _vp, _vp]),
    "moexb_layer_load_gguf": (_i, [_vp, _vp, _i, C.POINTER(_i)]),
    "moexb_st_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "moexb_st_close": (_i, [_vp]),
    "moexb_st_tensor_count": (_i, [_vp]),
    "moexb_st_tensor_name": (C.c_char_p, [_vp, _i]),
    "moexb_st_tensor": (_i, [_vp, C.c_char_p, C.c_char_p, C.POINTER(_i), C.POINTER(_ll), C.POINTER(_vp), C.POINTER(_ll)]),
    "moexb_layer_load_st": (_i, [_vp, _vp, C.c_char_p, C.POINTER(_i)]),
    "moexb_layer_forward": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp]),
    "moexb_layer_forward_ep": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "moexb_ep_residual_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "moexb_ep_buffer_bytes": (C.c_size_t, [_i, _i, _i]),
    "moexb_ep_buffer_alloc": (_i, [C.c_size_t, C.POINTER(_vp), _vp]),
    "moexb_ep_buffer_open": (_i, [_vp, C.POINTER(_vp)]),
    "moexb_ep_buffer_close": (_i, [_vp]),
    "moexb_ep_buffer_free": (_i, [_vp]),
    "moexb_ep_create": (_i, [_vp, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_vp)]),
    "moexb_ep_destroy": (_i, [_vp]),
    "moexb_ep_own_tokens": (_i, [_vp, C.POINTER(_i), C.POINTER(_i)]),
    "moexb_ep_read_routing": (_i, [_vp, _vp, _vp, _vp]),
    "moexb_ep_begin_step": (_i, [_vp, _vp]),
    "moexb_ep_dispatch": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp]),
    "moexb_ep_experts": (_i, [_vp, _vp, _i, _vp]),
    "moexb_ep_finish": (_i, [_vp, _i, _i, _vp, _vp]),
    "moexb_ep_step": (_i, [_vp, C.POINTER(_vp), _i, _vp, _i, _i, _vp, _vp]),
    "moexb_ep_stack_create": (_i, [_vp, C.POINTER(_vp), _i, _i, _i, C.POINTER(_vp)]),
    "moexb_stack_create": (_i, [_vp, C.POINTER(_vp), _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "moexb_stack_destroy": (_i, [_vp]),
    "moexb_stack_run": (_i, [_vp, _vp, _vp, _vp]),
    "moexb_stack_run_host": (_i, [_vp, _vp, _vp, _vp]),
    "moexb_stack_kernel_count": (_i, [_vp]),
    "moexb_launch_count": (_ll, []),
    "moexb_ctx_profile": (_i, [_vp, _i]),
    "moexb_ctx_profile_read": (_i, [_vp, _vp, _vp]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MoexbError(f"{LIB_PATH} is missing: build it with `python -m moe_b200.build` (needs nvcc); "
                             "there is no fallback path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise MoexbError(f"moexb error {rc}: {lib().moexb_last_error().decode()}")
