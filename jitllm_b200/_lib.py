"""ctypes binding of libjitllm_b200.so -- the same symbols a cgo/goffi shim binds.

There is no fallback: if the shared library is missing the import fails, and if
no B200 is present jl_open fails. Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("JITLLM_B200_LIB") or os.path.join(HERE, "libjitllm_b200.so")   # the override is for A/B builds

# ggml type ids (include/jitllm_b200.h)
F32, F16, Q8_0, Q4_K, BF16, MXFP4 = 0, 1, 8, 12, 30, 39
Q4_0, Q5_0, Q5_1, Q5_K, Q6_K = 2, 6, 7, 13, 14
DT_F32, DT_F16, DT_BF16 = 0, 1, 2
K_AUTO, K_SIMT, K_MMA, K_TC5 = 0, 1, 2, 3
ACT_SILU, ACT_SWIGLU_OAI = 0, 1
# jl_opts.flags
FLAG_NO_PDL, FLAG_NO_TMA, FLAG_DECODE_CONCURRENT = 1, 2, 16
# jl_decode_form
FORM_AUTO, FORM_SPLIT, FORM_FUSED, FORM_WIDE, FORM_L1 = 0, 1, 2, 3, 4
OK, DECLINED = 0, 1
EINVAL, ECUDA, ENOMEM, EDEVICE, ETIMEDOUT, ENOTSUP, ECOMM = -1, -2, -3, -4, -5, -6, -7

BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), MXFP4: (32, 17), F32: (1, 4), F16: (1, 2), BF16: (1, 2),
         Q4_0: (32, 18), Q5_0: (32, 22), Q5_1: (32, 24), Q5_K: (256, 176), Q6_K: (256, 210)}


def row_bytes(t: int, k: int) -> int:
    be, bb = BLOCK[t]
    return k // be * bb


class Opts(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("pin_kernel", C.c_int32), ("pin_warps", C.c_int32),
                ("min_weight_bytes", C.c_uint64), ("max_resident_bytes", C.c_uint64), ("flags", C.c_uint32),
                ("decode_form", C.c_int32), ("pin_stages", C.c_int32), ("pin_row_groups", C.c_int32),
                ("wait_limit_us", C.c_uint32)]


class Choice(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("warps", C.c_int32), ("rows_per_cta", C.c_int32),
                ("split_k", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
                ("grid", C.c_int32), ("form", C.c_int32), ("stages", C.c_int32), ("launches", C.c_int32)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("served", "declined", "errors", "uploads", "upload_bytes",
                                           "resident_bytes", "forgets", "launches", "injected")]


class MoeDesc(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("type", C.c_uint32), ("n_expert", C.c_int32),
                ("top_k", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("act", C.c_int32),
                ("norm", C.c_int32), ("scale", C.c_float),
                ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("gate_bytes", C.c_size_t), ("up_bytes", C.c_size_t), ("down_bytes", C.c_size_t),
                ("gate_bias", C.c_void_p), ("up_bias", C.c_void_p), ("down_bias", C.c_void_p),
                ("router_bias", C.c_void_p), ("sel_bias", C.c_void_p), ("arm", C.c_int32)]


class Packed(C.Structure):
    _fields_ = [("qs", C.c_void_p), ("d", C.c_void_p), ("sc", C.c_void_p), ("qs_bytes", C.c_size_t), ("d_bytes", C.c_size_t),
                ("sc_bytes", C.c_size_t), ("row", C.c_int32), ("stride", C.c_int32)]


class LayersBlock(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("o", C.c_void_p), ("gate_up", C.c_void_p), ("down", C.c_void_p),
                ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class LayersDesc(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("n_layer", C.c_int32), ("hidden", C.c_int32), ("n_head", C.c_int32),
                ("n_kv", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
                ("max_len", C.c_int32), ("eps", C.c_float), ("blocks", C.POINTER(LayersBlock)), ("head", C.c_void_p),
                ("final_norm", C.c_void_p), ("emb_bf16", C.c_void_p), ("cos_t", C.c_void_p), ("sin_t", C.c_void_p),
                ("rank", C.c_int32), ("world", C.c_int32)]


# Every symbol include/jitllm_b200.h declares: (restype, argtypes).
_VP, _I, _SZ, _U32 = C.c_void_p, C.c_int, C.c_size_t, C.c_uint32
TUNE_OFF, TUNE_ON, TUNE_FORCE = 0, 1, 2
MOE_ARM_EXACT, MOE_ARM_BLOCK_SCALED, MOE_ARM_BLOCK_SCALED_X3 = 0, 1, 2
TUNE_TIMER = C.CFUNCTYPE(C.c_double, C.c_void_p, C.c_int, C.c_int)

SYMBOLS = {
    "jl_version": (C.c_char_p, []),
    "jl_abi_version": (_I, []),
    "jl_open": (_I, [_I, C.POINTER(Opts), C.POINTER(_VP)]),
    "jl_close": (None, [_VP]),
    "jl_reserve": (_I, [_VP, _I, _I, _I]),
    "jl_last_error": (C.c_char_p, [_VP]),
    "jl_stats_get": (_I, [_VP, C.POINTER(Stats)]),
    "jl_matvec": (_I, [_VP, _VP, _U32, _VP, _SZ, _VP, _I, _I]),
    "jl_forget": (_I, [_VP, _VP, _SZ]),
    "jl_matmul": (_I, [_VP, _VP, _I, _U32, _VP, _SZ, _VP, _I, _I, _I, _I]),
    "jl_packed_to_blocks": (_I, [_U32, C.POINTER(Packed), _I, _I, _VP, _SZ]),
    "jl_weight_upload_packed": (_I, [_VP, _U32, C.POINTER(Packed), _I, _I, C.POINTER(_VP)]),
    "jl_matvec_packed": (_I, [_VP, _VP, _U32, C.POINTER(Packed), _VP, _I, _I]),
    "jl_matmul_packed": (_I, [_VP, _VP, _I, _U32, C.POINTER(Packed), _VP, _I, _I, _I, _I]),
    "jl_moe": (_I, [_VP, _VP, _VP, _I, _VP, _I, C.POINTER(MoeDesc), _VP, _VP]),
    "jl_moe_route_dev": (_I, [_VP, _VP, _I, C.POINTER(MoeDesc), _VP, _VP, _VP]),
    "jl_moe_experts_dev": (_I, [_VP, _VP, _VP, _I, _VP, _I, C.POINTER(MoeDesc), _VP]),
    "jl_moe_reserve": (_I, [_VP, _I, _I, _I, _I, _I]),
    "jl_moe_bs_weights_by_tma": (_I, [_VP]),
    "jl_select": (_I, [_VP, _U32, _I, _I, _I, C.POINTER(Choice)]),
    "jl_tune_configure": (_I, [_VP, _I, C.c_char_p]),
    "jl_tune": (_I, [_VP, _VP, _I, C.POINTER(Choice)]),
    "jl_tune_stats": (_I, [_VP, C.POINTER(C.c_int64 * 4)]),
    "jl_tune_duel": (_I, [_I, _I, TUNE_TIMER, _VP, C.c_double, C.c_double, C.POINTER(_I), C.POINTER(C.c_double)]),
    "jl_tune_cache_lookup": (_I, [C.c_char_p, C.c_char_p, C.c_char_p, _SZ]),
    "jl_tune_cache_save": (_I, [C.c_char_p, C.c_char_p, C.c_char_p]),
    "jl_tune_device_key": (None, [_VP, _I, C.c_char_p, C.c_char_p]),
    "jl_build_id": (C.c_char_p, []),
    "jl_unpack": (_I, [_U32, _VP, _SZ, _VP, _VP, _VP, _VP, _VP]),
    "jl_unpack_resident": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "jl_weight_upload": (_I, [_VP, _U32, _VP, _SZ, _I, _I, C.POINTER(_VP)]),
    "jl_weight_upload_bank": (_I, [_VP, _U32, _VP, _SZ, _I, _I, _I, C.POINTER(_VP)]),
    "jl_weight_free": (None, [_VP, _VP]),
    "jl_matvec_dev": (_I, [_VP, _VP, _VP, _VP, _I, _VP]),
    "jl_matmul_dev": (_I, [_VP, _VP, _I, _VP, _VP, _I, _I, _VP]),
    "jl_moe_dev": (_I, [_VP, _VP, _VP, _I, _VP, _I, C.POINTER(MoeDesc), _VP, _VP, _VP]),
    "jl_test_fail_at": (_I, [_VP, C.POINTER(C.c_int), _I]),
    "jl_test_matvec_loop": (_I, [_VP, _VP, _U32, C.POINTER(_VP), _SZ, _VP, _I, _I, _I, _I, C.POINTER(C.c_double)]),
    "jl_layers_prep": (_I, [_VP, C.POINTER(LayersDesc), C.POINTER(_VP)]),
    "jl_layers_free": (None, [_VP, _VP]),
    "jl_layers_run": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I, _VP]),
    "jl_layers_phases": (_I, [_VP]),
    "jl_layers_profile": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I]),
    "jl_tp_slot": (_I, [_VP, _VP, C.POINTER(_VP), C.POINTER(C.c_size_t)]),
    "jl_tp_ipc_export": (_I, [_VP, _VP]),
    "jl_tp_ipc_open": (_I, [_VP, C.POINTER(_VP)]),
    "jl_tp_ipc_close": (_I, [_VP]),
    "jl_tp_attach": (_I, [_VP, _VP, C.POINTER(_VP), _I]),
    "jl_status_poll": (_I, [_VP, _VP]),
    "jl_noalloc_status": (_I, [_VP]),
    "jl_test_wait_timeout": (_I, [_VP, _U32, _VP]),
    "jl_noalloc_max_k": (_I, []),
    "jl_matvec_q4k_noalloc": (_I, [_VP, _VP, _VP, _I, _I, _VP]),
    "jl_aux_add_rmsnorm": (_I, [_VP, _VP, _VP, C.c_float, _VP, _VP, _I, _I, _VP]),
    "jl_aux_silu_mul": (_I, [_VP, _VP, _VP, _I, _I, _VP]),
    "jl_aux_argmax": (_I, [_VP, _VP, _I, _I, _VP]),
    "jl_aux_rope_kv": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP]),
    "jl_aux_attn_scratch_bytes": (C.c_size_t, [_I, _I, _I, _I]),
    "jl_aux_attn_decode": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP]),
    "jl_gemm_operand": (_I, [_VP, _VP, _I, C.POINTER(_VP), C.POINTER(_VP)]),
    "jl_matmul_dev_prepared": (_I, [_VP, _VP, _I, _VP, _I, _VP]),
    "jl_aux_add_rmsnorm_gemm": (_I, [_VP, _VP, _VP, C.c_float, _VP, _VP, _I, _I, _VP]),
    "jl_decode_operand": (_VP, [_VP, _VP, _I]),
    "jl_matvec_dev_prepared": (_I, [_VP, _VP, _VP, _I, _VP]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the library and bind every declared symbol. Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m jitllm_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
