"""Loader for the C-ABI shared library (``libtlb200.so``).

There is no fallback: if the library is missing or fails to load, importing the
ops raises.  ``check(rc)`` turns a non-zero status into ``TlbError`` carrying the
library's message.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TLB200_LIB names another build of the library (the C++ seam honours the same variable)
LIB_PATH = os.environ.get("TLB200_LIB") or os.path.join(_HERE, "libtlb200.so")

i64, f32, vp, ci = C.c_int64, C.c_float, C.c_void_p, C.c_int

# name -> (restype, argtypes); mirrors include/tlb200.h one to one
SIGNATURES = {
    "tlb_init": (ci, [ci]),
    "tlb_device_count": (ci, []),
    "tlb_last_error": (C.c_char_p, []),
    "tlb_version": (ci, []),
    "tlb_device_status": (ci, [C.POINTER(ci), ci]),
    "tlb_set_wait_limit_cycles": (ci, [i64]),
    "tlb_set_pdl": (ci, [ci]),
    "tlb_alloc": (ci, [i64, C.POINTER(vp)]),
    "tlb_free": (ci, [vp]),
    "tlb_h2d": (ci, [vp, vp, i64, vp]),
    "tlb_d2h": (ci, [vp, vp, i64, vp]),
    "tlb_memset": (ci, [vp, ci, i64, vp]),
    "tlb_sync": (ci, [vp]),
    "tlb_q4_bytes": (i64, [i64, i64]),
    "tlb_to_q4": (ci, [vp, i64, i64, vp, vp]),
    "tlb_q4_to_f32": (ci, [vp, i64, i64, vp, vp]),
    "tlb_gemv_q4": (ci, [vp, vp, vp, vp, i64, i64, i64, vp]),
    "tlb_gemm_q4": (ci, [vp, i64, i64, vp, vp, vp, i64, i64, i64, f32, f32, vp]),
    "tlb_gemm_q4_simt": (ci, [vp, i64, i64, vp, vp, vp, i64, i64, i64, f32, f32, vp]),
    "tlb_attn_decode": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, vp]),
    "tlb_attn_decode_bf16": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, vp]),
    "tlb_attn_decode_noalloc": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, vp]),
    "tlb_attn_decode_dpos": (ci, [vp, vp, vp, vp, i64, i64, vp, i64, i64, f32, vp, vp]),
    "tlb_attn_decode_dpos_bf16": (ci, [vp, vp, vp, vp, i64, i64, vp, i64, i64, f32, vp, vp]),
    "tlb_attn_partials_bytes": (i64, [i64, i64, i64, i64]),
    "tlb_rmsnorm": (ci, [vp, vp, vp, i64, f32, i64, vp]),
    "tlb_rmsnorm_res": (ci, [vp, vp, vp, vp, vp, i64, f32, i64, vp]),
    "tlb_swiglu": (ci, [vp, vp, i64, i64, vp]),
    "tlb_swiglu_split": (ci, [vp, i64, vp, i64, vp, i64, i64, vp]),
    "tlb_rope": (ci, [vp, vp, i64, i64, i64, i64, f32, vp, vp]),
    "tlb_rope_dpos": (ci, [vp, vp, i64, i64, i64, vp, f32, vp, vp]),
    "tlb_kv_append": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, vp]),
    "tlb_kv_append_bf16": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, vp]),
    "tlb_kv_append_dpos": (ci, [vp, vp, vp, vp, vp, i64, i64, i64, vp]),
    "tlb_kv_append_dpos_bf16": (ci, [vp, vp, vp, vp, vp, i64, i64, i64, vp]),
    "tlb_incr_u32": (ci, [vp, vp]),
    "tlb_argmax": (ci, [vp, i64, C.POINTER(i64), vp]),
    "tlb_argmax_dev": (ci, [vp, i64, vp, vp]),
    "tlb_gemv_bf16_row": (ci, [vp, vp, vp, i64, i64, vp]),
    "tlb_q4p_bytes": (i64, [i64, i64]),
    "tlb_q4_pack": (ci, [vp, i64, i64, vp, vp]),
    "tlb_gemv_q4p": (ci, [vp, vp, vp, i64, i64, f32, f32, vp]),
    "tlb_binary": (ci, [ci, vp, vp, vp, i64, f32, f32, vp]),
    "tlb_binary_bcast": (ci, [ci, vp, i64, i64, vp, i64, i64, vp, i64, i64, f32, f32, vp]),
    "tlb_unary": (ci, [ci, vp, vp, i64, f32, f32, vp]),
    "tlb_row_op": (ci, [ci, vp, vp, i64, i64, f32, f32, vp]),
    "tlb_gemm_f32": (ci, [vp, i64, ci, vp, i64, ci, vp, i64, i64, i64, f32, f32, vp]),
    "tlb_gemm_bf16_nt": (ci, [vp, vp, vp, i64, i64, i64, vp]),
    "tlb_gemv_f32": (ci, [vp, vp, vp, i64, i64, vp]),
    "tlb_gemv_bf16": (ci, [vp, vp, vp, i64, i64, vp]),
    "tlb_split_heads": (ci, [vp, vp, vp, i64, i64, i64, i64, i64, vp]),
    "tlb_merge_heads": (ci, [vp, vp, i64, i64, i64, vp]),
    "tlb_kv_fill": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, vp]),
    "tlb_kv_fill_bf16": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, vp]),
    "tlb_attn_prefill": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, i64, vp]),
    "tlb_attn_prefill_bf16": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, i64, vp]),
    "tlb_capture_begin": (ci, [C.POINTER(vp)]),
    "tlb_capture_end": (ci, [C.POINTER(vp)]),
    "tlb_graph_launch": (ci, [vp, vp]),
    "tlb_graph_destroy": (ci, [vp]),
    "tlb_decoder_create": (ci, [C.POINTER(i64), ci, f32, f32, C.POINTER(vp)]),
    "tlb_decoder_destroy": (ci, [vp]),
    "tlb_decoder_set_linear": (ci, [vp, i64, ci, vp, i64, i64]),
    "tlb_decoder_set_vector": (ci, [vp, i64, ci, vp]),
    "tlb_decoder_kv": (ci, [vp, i64, C.POINTER(vp), C.POINTER(vp)]),
    "tlb_decoder_logits": (ci, [vp, C.POINTER(vp)]),
    "tlb_decoder_set_pos": (ci, [vp, i64, vp]),
    "tlb_decoder_set_token": (ci, [vp, i64, vp]),
    "tlb_decoder_forward": (ci, [vp, vp]),
    "tlb_decoder_launches_per_token": (i64, [vp]),
    "tlb_decoder_capture": (ci, [vp]),
    "tlb_decoder_run": (ci, [vp, i64, vp]),
    "tlb_decoder_step": (ci, [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32), vp]),
    "tlb_decoder_prefill": (ci, [vp, C.POINTER(C.c_int32), i64, C.POINTER(C.c_int32), vp]),
    "tlb_decoder_last_token": (ci, [vp, C.POINTER(C.c_int32), vp]),
    "tlb_decoder_ipc_export": (ci, [vp, vp]),
    "tlb_decoder_ipc_open": (ci, [vp, vp]),
    "tlb_decoder_loopback_peers": (ci, [vp]),
}


class TlbError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TlbError(f"{LIB_PATH} is missing: build it with `python -m cpp_tensorlib_b200.build` "
                           "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here means the .so is stale
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise TlbError(f"tlb200 status {rc}: {lib().tlb_last_error().decode()}")
