"""ctypes loader for libmycaffe_attn.so.  There is no fallback: if the library has not been
built (``python -m mycaffe_b200.build``) loading raises."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libmycaffe_attn.so"
_lib = None

LONG = C.c_int32
LONGLONG = C.c_int64
_fp = C.POINTER(C.c_float)
_vp = C.c_void_p
_i = C.c_int
_i64 = C.c_int64

# name -> (restype, argtypes); the same list the header declares
SIGNATURES = {
    "DLL_InvokeFloat": (LONG, [LONG, LONG, _fp, LONG, C.POINTER(_fp), C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeFloatEx2": (LONG, [LONG, LONG, _fp, LONG, C.POINTER(LONGLONG), LONG, C.POINTER(_fp), C.POINTER(LONG),
                                  C.c_char_p, LONG]),
    "DLL_InvokeFloatEx": (LONG, [LONG, LONG, _fp, LONG, C.c_char_p, C.POINTER(_fp), C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeDouble": (LONG, [LONG, LONG, C.POINTER(C.c_double), LONG, C.POINTER(C.POINTER(C.c_double)),
                                C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeDoubleEx2": (LONG, [LONG, LONG, C.POINTER(C.c_double), LONG, C.POINTER(LONGLONG), LONG,
                                   C.POINTER(C.POINTER(C.c_double)), C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeDoubleEx": (LONG, [LONG, LONG, C.POINTER(C.c_double), LONG, C.c_char_p, C.POINTER(C.POINTER(C.c_double)),
                                  C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_QueryString": (LONG, [LONG, LONG, C.POINTER(LONG), LONG, C.POINTER(C.c_void_p), C.c_char_p, LONG]),
    "DLL_QueryStringFloatEx": (LONG, [LONG, LONG, C.POINTER(LONG), LONG, C.c_char_p, LONG, C.c_char_p, LONG]),
    "DLL_QueryStringDoubleEx": (LONG, [LONG, LONG, C.POINTER(LONG), LONG, C.c_char_p, LONG, C.c_char_p, LONG]),
    "Internal_GetPointerDouble": (LONG, [LONG, LONG, LONG, C.POINTER(_vp)]),
    "Internal_AllocHostDouble": (LONG, [LONG, LONG, C.POINTER(C.POINTER(C.c_double)), C.POINTER(C.c_double), C.c_bool]),
    "DLL_InitFloatCustomExtension": (LONG, [_vp, LONG]),
    "DLL_InvokeFloatCustomExtension": (LONG, [LONG, _fp, LONG, C.POINTER(_fp), C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeFloatCustomExtensionEx": (LONG, [LONG, _fp, LONG, C.POINTER(_fp), C.POINTER(LONG), C.c_char_p, C.c_char_p, LONG,
                                                C.c_char_p, LONG]),
    "DLL_InitDoubleCustomExtension": (LONG, [_vp, LONG]),
    "DLL_InvokeDoubleCustomExtension": (LONG, [LONG, C.POINTER(C.c_double), LONG, C.POINTER(C.POINTER(C.c_double)),
                                               C.POINTER(LONG), C.c_char_p, LONG]),
    "DLL_InvokeDoubleCustomExtensionEx": (LONG, [LONG, C.POINTER(C.c_double), LONG, C.POINTER(C.POINTER(C.c_double)),
                                                 C.POINTER(LONG), C.c_char_p, C.c_char_p, LONG, C.c_char_p, LONG]),
    "Internal_GetPointerFloat": (LONG, [LONG, LONG, LONG, C.POINTER(_vp)]),
    "Internal_AllocHostFloat": (LONG, [LONG, LONG, C.POINTER(_fp), _fp, C.c_bool]),
    "mca_sdpa_forward_f32": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "mca_sdpa_backward_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mca_sdpa_forward_f32_layout": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "mca_sdpa_backward_f32_layout": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp,
                                          _i, _vp]),
    "mca_sdpa_forward_tc_layout": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp]),
    "mca_sdpa_forward_tc_scatter": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp), _i, _i64, _i64, _i64, _vp, _vp, _vp]),
    "mca_sdpa_backward_tc_layout": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i,
                                         _vp]),
    "mca_classify_causal_mask": (_i, [_vp, _i, _vp, _vp]),
    "mca_sdpa_forward_tc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mca_sdpa_backward_tc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "mca_sdpa_forward_f32_tc_workspace_bytes": (_i64, [_i, _i, _i]),
    "mca_sdpa_forward_f32_tc_supported": (_i, [_i]),
    "mca_sdpa_forward_f32_tc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _vp]),
    "mca_sdpa_forward_f32_tc_masked": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i, _vp, _i, _vp]),
    "mca_sdpa_forward_tc_masked": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "mca_mask_bits_row_words": (_i, [_i]),
    "mca_tc_narrow_len": (_i, [_i]),
    "mca_sdpa_forward_tc_keep": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "mca_sdpa_forward_f32_tc_workspace_bytes_d": (_i64, [_i, _i, _i, _i]),
    "mca_sdpa_backward_f32_tc_supported": (_i, [_i]),
    "mca_mask_pack": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "mca_sdpa_backward_f32_tc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _vp, _i, _vp]),
    "mca_sdpa_backward_f32_tc_masked": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _vp, _i, _vp, _vp, _i, _vp]),
    "mca_sdpa_backward_tc_masked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp]),
    "mca_wait_probe": (_i, [_vp, _i, _vp]),
    "mca_sdpa_forward_host": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i]),
    "mca_host_pipeline_chunk": (_i, [_i, _i, _i, _i]),
    "mca_host_pipeline_release": (_i, []),
    "mca_rope_f32": (_i, [_vp, _vp, _i64, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "mca_rope_tables_host": (_i, [_i, _i, C.c_float, _fp, _fp]),
    "mca_decode_plan": (_i, [_i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i64)]),
    "mca_decode_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i64,
                                  _vp, _vp]),
    "mca_decode_head_size_supported": (_i, [_i]),
    "mca_decode_status": (_i, [C.POINTER(_i)]),
    "mca_proj_tc_enable": (_i, [_i]),
    "mca_proj_tc_status": (_i, [C.POINTER(_i)]),
    "mca_decode_exchange": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp), _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "mca_decode_qkv_rmsnorm": (_i, [_vp, _vp, C.c_float, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mca_decode_out_proj": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "mca_decode_ffn": (_i, [_vp, C.c_float, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "mca_decode_logits": (_i, [_vp, _vp, C.c_float, _vp, _i, _i, _i, _i, _vp, _vp]),
    "mca_llama_workspace_floats": (_i64, [_vp, _i, _i]),
    "mca_llama_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "mca_decode_static_scratch_floats": (_i64, []),
    "mca_decode_attention_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mca_tft_attention_forward_f32": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "mca_tft_attention_backward_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mca_layernorm_forward_f32": (_i, [_vp, _vp, _vp, _i64, _i, C.c_float, _vp]),
    "mca_layernorm_backward_f32": (_i, [_vp, _vp, _vp, _vp, _i64, _i, C.c_float, _vp]),
    "mca_rmsnorm_forward_f32": (_i, [_vp, _vp, _vp, _vp, _i64, _i, C.c_float, _vp]),
    "mca_rmsnorm_backward_scratch_floats": (_i64, [_i]),
    "mca_rmsnorm_backward_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "mca_convert_f32_to_bf16": (_i, [_vp, _vp, _i64, _vp]),
    "mca_convert_bf16_to_f32": (_i, [_vp, _vp, _i64, _vp]),
    "mca_version": (C.c_char_p, []),
}


def load() -> C.CDLL:
    """Load the shared library and bind every exported entry point."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m mycaffe_b200.build` "
                               "(there is no CPU or PyTorch fallback for this path)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # raises AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
