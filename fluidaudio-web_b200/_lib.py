"""ctypes binding of libfa_cuda.so: the same entry points an N-API addon would bind."""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

P = C.c_void_p
PP = C.POINTER(C.c_void_p)
F32P = C.POINTER(C.c_float)
I = C.c_int
IP = C.POINTER(C.c_int)
ULLP = C.POINTER(C.c_ulonglong)


class ProfileEntry(C.Structure):
    _fields_ = [("label", C.c_char * 48), ("ms", C.c_float), ("count", C.c_int)]


# name -> argtypes (every function returns int except fa_last_error)
SIGNATURES = {
    "fa_ctx_create": [I, PP],
    "fa_ctx_destroy": [P],
    "fa_ctx_set_option": [P, C.c_char_p, C.c_longlong],
    "fa_ctx_stream": [P, PP],
    "fa_ctx_mark": [P],
    "fa_ctx_wait_mark": [P, P],
    "fa_sync": [P],
    "fa_launch_count": [P, ULLP],
    "fa_upload_f32": [P, P, I, I, PP],
    "fa_upload_f16": [P, P, I, I, PP],
    "fa_alloc": [P, I, I, PP],
    "fa_alloc_f16": [P, I, I, PP],
    "fa_upload_bytes": [P, P, C.c_size_t, PP],
    "fa_free_tensor": [P, P],
    "fa_free_bytes": [P, P],
    "fa_pin": [P, P, I],
    "fa_push_arena": [P, IP],
    "fa_pop_arena": [P, I],
    "fa_trim_pool": [P, C.c_size_t],
    "fa_tensor_info": [P, IP, IP, IP, PP],
    "fa_mem_stats": [P, ULLP, ULLP, ULLP, ULLP],
    "fa_host_alloc": [C.c_size_t, PP],
    "fa_host_free": [P],
    "fa_download": [P, P, P],
    "fa_download_async": [P, P, P],
    "fa_stage_download": [P, P, PP],
    "fa_staged_read": [P, P, P],
    "fa_staged_free": [P, P],
    "fa_tensor_ptr": [P, P, PP],
    "fa_rows_view": [P, P, I, PP],
    "fa_reshape_view": [P, P, I, I, PP],
    "fa_begin_batch": [P],
    "fa_end_batch": [P],
    "fa_graph_begin": [P],
    "fa_graph_end": [P, PP],
    "fa_graph_launch": [P, P],
    "fa_graph_free": [P, P],
    "fa_matmul": [P, P, P, P, I, P, PP],
    "fa_matmul_operand": [P, P, P, P, I, PP],
    "fa_matmul_int8": [P, P, P, P, I, I, P, I, PP],
    "fa_matmul_int8_operand": [P, P, P, P, I, I, P, I, P, I, PP],
    "fa_matmul_nbits": [P, P, P, P, P, I, I, PP],
    "fa_int8_gemm_i32": [P, P, I, P, I, I, P],
    "fa_matmul_int8_static": [P, P, P, P, P, I, P, I, I, I],
    "fa_layernorm": [P, P, P, P, C.c_float, PP],
    "fa_layernorm_operand": [P, P, P, P, C.c_float, PP],
    "fa_layernorm_chain": [P, P, P, P, P, P, C.c_float, PP, PP],
    "fa_softmax": [P, P, PP],
    "fa_conv1d": [P, P, P, P, I, I, I, I, I, I, I, I, PP],
    "fa_conv1d_windows": [P, P, P, P, I, I, I, I, I, I, I, I, PP],
    "fa_glu_dwconv_tm": [P, P, P, P, I, I, I, I, I, PP],
    "fa_conv2d": [P, P, P, P] + [I] * 14 + [PP],
    "fa_conv2d_windows": [P, P, P, P] + [I] * 15 + [PP],
    "fa_bmm_qk": [P, P, P, P, I, I, I, I, PP],
    "fa_bmm_pv": [P, P, P, I, I, I, PP],
    "fa_attn_fused": [P, P, P, P, P, P, P, I, I, I, PP],
    "fa_attn_fused_qkv": [P, P, P, P, P, I, I, I, PP],
    "fa_rel_shift_b": [P, P, I, PP],
    "fa_ewise": [P, P, P, I, PP],
    "fa_scale": [P, P, C.c_float, PP],
    "fa_unary": [P, P, I, PP],
    "fa_glu": [P, P, PP],
    "fa_transpose": [P, P, PP],
    "fa_slice_cols": [P, P, I, I, PP],
    "fa_set_cols": [P, P, P, I],
    "fa_slice_rows": [P, P, I, I, PP],
    "fa_copy_rows": [P, P, P, I],
    "fa_concat_rows": [P, PP, I, PP],
    "fa_sub_reshape": [P, P, I, I, I, PP],
    "fa_sub_reshape_windows": [P, P, I, I, I, I, PP],
    "fa_conv_stem_windows": [P, P, P, P, P, P, P, P, I, I, I, I, PP],
    "fa_conv_dw_pw_windows": [P, P, P, P, P, P, I, I, I, I, PP],
    "fa_argmax_rows": [P, P, I, PP],
    "fa_embed_rows": [P, P, P, P, I, PP],
    "fa_log_mel_windows": [P, P, I, C.c_double, I, PP],
    "fa_tdt_create": [P] + [P] * 13 + [PP],
    "fa_tdt_decode_proj": [P, P, P, I, I, I, P, P, P, IP],
    "fa_tdt_free": [P, P],
    "fa_unshard_cols": [P, P, I, PP],
    "fa_ipc_export": [P, P, P],
    "fa_ipc_open": [P, P, PP],
    "fa_ipc_close": [P, P],
    "fa_matmul_scatter": [P, P, P, P, I, P, I, I, I],
    "fa_profile_start": [P, I],
    "fa_profile_end": [P, C.POINTER(ProfileEntry), I, IP],
}


def library_path() -> str:
    return os.path.join(HERE, "libfa_cuda.so")


def declared_symbols(header_path: str | None = None):
    """Function names declared in include/fa_cuda.h (used by the symbol-export test)."""
    header_path = header_path or os.path.join(os.path.dirname(HERE), "include", "fa_cuda.h")
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def load_library() -> C.CDLL:
    """Load libfa_cuda.so, failing loudly when it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python fluidaudio-web_b200/build.py` "
            "(this backend has no CPU fallback)")
    lib = C.CDLL(path)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = I
    lib.fa_last_error.argtypes = [P]
    lib.fa_last_error.restype = C.c_char_p
    _LIB = lib
    return lib
