"""ctypes binding of libleviathan_cuda.so (the C ABI in include/leviathan_cuda.h).

Loading fails loudly when the shared library is missing: there is no CPU or
PyTorch fallback for any operation of this package.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libleviathan_cuda.so")

# status codes (include/leviathan_cuda.h, enum lev_status)
OK = 0
STATUS = {
    0: "ok", 1: "badDimensions", 2: "wrongInputCount", 3: "nonFiniteInput", 4: "nonFiniteScale",
    5: "nonFiniteOutput", 6: "exceedsModelWorkload", 7: "integerOverflow", 8: "deviceUnavailable",
    9: "kernelFailed", 10: "timeout", 11: "ncclError", 12: "badArgument", 13: "outOfMemory",
    14: "badOpSpec", 15: "unsupported", 16: "badMagic", 17: "unsupportedVersion", 18: "truncated",
    19: "unknownValueType", 20: "badTensor", 21: "dataBeyondEndOfFile", 22: "missing",
    23: "unsupportedTensorType",
}
GGML_F32, GGML_Q4_0, GGML_Q4_K, GGML_Q6_K = 0, 2, 12, 14
BLOCK = {GGML_Q4_0: (32, 18), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}
FLAG_CHECK_FINITE, FLAG_HOST_IO = 1, 2
SCHEDULE_AUTO, SCHEDULE_PLAIN, SCHEDULE_STREAM = -1, 0, 1
MAX_COLUMNS = 8
NCCL_ID_BYTES = 128


class HwProfile(C.Structure):
    _fields_ = [
        ("device_name", C.c_char * 128), ("sm_count", C.c_int), ("max_threads_per_block", C.c_int),
        ("warp_width", C.c_int), ("cc_major", C.c_int), ("cc_minor", C.c_int),
        ("total_memory", C.c_size_t), ("free_memory", C.c_size_t),
        ("shared_memory_per_block_optin", C.c_size_t), ("l2_bytes", C.c_size_t),
    ]


class Evidence(C.Structure):
    _fields_ = [
        ("device_name", C.c_char * 128), ("kernel_name", C.c_char * 64), ("out_dim", C.c_int64),
        ("in_dim", C.c_int64), ("n_cols", C.c_int), ("grid", C.c_int), ("block", C.c_int),
        ("weight_bytes", C.c_size_t), ("gpu_us", C.c_float), ("status", C.c_int),
    ]


class Fusion(C.Structure):
    _fields_ = [("prologue", C.c_int), ("norm_weight", C.c_void_p), ("eps", C.c_float), ("residual", C.c_void_p),
                ("alpha", C.c_float)]


PROLOGUE_NONE, PROLOGUE_RMSNORM, PROLOGUE_GELU_UP = 0, 1, 2
MAX_CHAIN_OPS = 32


class ChainOp(C.Structure):
    _fields_ = [("w", C.c_void_p), ("row0", C.c_int64), ("rows", C.c_int64), ("x", C.c_void_p), ("y", C.c_void_p),
                ("depends", C.c_int), ("fusion", Fusion)]



class KVLayout(C.Structure):
    _fields_ = [("kv_type", C.c_int), ("page", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
                ("blocks", C.c_int64), ("max_blocks", C.c_int), ("slots", C.c_int)]


KV_F32, KV_F16 = 0, 1

# name -> (restype, argtypes); every symbol the header declares
_P, _I, _L, _Z, _U = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_uint
SIGNATURES = {
    "lev_cuda_abi_version": (_I, []),
    "lev_status_name": (C.c_char_p, [_I]),
    "lev_cuda_init": (_I, [_I, C.POINTER(_P)]),
    "lev_cuda_destroy": (_I, [_P]),
    "lev_last_error": (C.c_char_p, [_P]),
    "lev_cuda_hardware_profile": (_I, [_P, C.POINTER(HwProfile)]),
    "lev_cuda_set_stream": (_I, [_P, _P]),
    "lev_cuda_synchronize": (_I, [_P]),
    "lev_cuda_launch_count": (_L, [_P]),
    "lev_cuda_last_evidence": (_I, [_P, C.POINTER(Evidence)]),
    "lev_weights_upload": (_I, [_P, _P, _Z, _I, _L, _L, _I, C.POINTER(_P)]),
    "lev_weights_free": (_I, [_P, _P]),
    "lev_weights_release_gguf": (_I, [_P, _P]),
    "lev_weights_info": (_I, [_P, C.POINTER(_I), C.POINTER(_L), C.POINTER(_L), C.POINTER(_Z)]),
    "lev_dequantize": (_I, [_P, _P, _L, _L, _P, _U]),
    "lev_matvec": (_I, [_P, _P, _L, _L, _P, _L, _I, _P, _L, _I, _U]),
    "lev_q4_0_matvec_host": (_I, [_P, _P, _Z, _L, _L, _P, _L, _P, C.POINTER(Evidence)]),
    "lev_q4_k_matvec_host": (_I, [_P, _P, _Z, _L, _L, _P, _L, _P, C.POINTER(Evidence)]),
    "lev_q6_k_matvec_host": (_I, [_P, _P, _Z, _L, _L, _P, _L, _P, C.POINTER(Evidence)]),
    "lev_matvec_multi": (_I, [_P, _I, C.POINTER(_P), _P, _L, _I, C.POINTER(_P), C.POINTER(_L), _U]),
    "lev_matvec_static_scratch": (_I, [_P, _P, _L, _L, _P, _L, _I, _P, _L]),
    "lev_static_scratch_bytes": (_Z, []),
    "lev_rmsnorm": (_I, [_P, _P, _L, _L, _P, C.c_float, _P, _P]),
    "lev_rmsnorm_cached": (_I, [_P, _P, _L, _L, _P, _P, _P]),
    "lev_gelu_up": (_I, [_P, _P, _L, _L, _P]),
    "lev_axpy": (_I, [_P, C.c_float, _P, _P, _L, _P]),
    "lev_qkv_norm_rope": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, C.c_float, _P, _P]),
    "lev_qkv_norm_rope_append": (_I, [_P, _P, _I, _I, _I, _P, _P, C.c_float, _P, _P, C.POINTER(KVLayout), _P, _P, _P, _P]),
    "lev_qkv_norm_rope_append_split": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P, C.c_float, _P, _P, C.POINTER(KVLayout), _P, _P, _P, _P]),
    "lev_argmax": (_I, [_P, _P, _L, _L, _P, _P]),
    "lev_embed_rows": (_I, [_P, _P, _P, _L, C.c_float, _P]),
    "lev_softcap": (_I, [_P, _P, _L, C.c_float]),
    "lev_matvec_fused": (_I, [_P, _P, _L, _L, _P, _L, _I, C.POINTER(Fusion), _P, _L]),
    "lev_matvec_chain": (_I, [_P, _I, C.POINTER(ChainOp), _U]),
    "lev_matvec_multi_fused": (_I, [_P, _I, C.POINTER(_P), _P, _L, _I, C.POINTER(Fusion), C.POINTER(_P), C.POINTER(_L)]),
    "lev_kv_append": (_I, [_P, C.POINTER(KVLayout), _P, _P, _P, _P, _P, _I, _P, _P]),
    "lev_attn_decode": (_I, [_P, C.POINTER(KVLayout), _P, _P, _P, _P, _P, _I, _I, _P, _I, C.c_float, _P]),
    "lev_attn_decode_ld": (_I, [_P, C.POINTER(KVLayout), _P, _P, _P, _P, _P, _I, _I, _P, _L, _I, C.c_float, _P]),
    "lev_gemm_prefill": (_I, [_P, _P, _P, _L, _P, _U]),
    "lev_act_bf16": (_I, [_P, _P, _L, _P]),
    "lev_moe_weights_upload": (_I, [_P, _P, _P, _Z, _P, _Z, _I, _I, _I, _I, _I, _I, C.POINTER(_P)]),
    "lev_moe_weights_free": (_I, [_P, _P]),
    "lev_moe_weights_release_gguf": (_I, [_P, _P]),
    "lev_moe_route": (_I, [_P, _P, _P, _L, _I, _P, _P, _P, _U]),
    "lev_moe_group": (_I, [_P, _P, _L, _I, _I, _P, _P, _P, _U]),
    "lev_moe_experts": (_I, [_P, _P, _P, _L, _I, _P, _P, _P, _U]),
    "lev_moe_combine": (_I, [_P, _P, _P, _L, _I, _I, _P, _U]),
    "lev_moe_layer": (_I, [_P, _P, _P, _L, _I, _P, _P, _P, _U]),
    "lev_moe_layer_residual": (_I, [_P, _P, _P, _L, _I, _P, C.c_float, _P, _U]),
    "lev_op_install_json": (_I, [_P, C.c_char_p, _Z, C.POINTER(_P)]),
    "lev_op_uninstall": (_I, [_P, _P]),
    "lev_op_describe": (_I, [_P, C.c_char_p, C.POINTER(_L), C.POINTER(_L), C.POINTER(_I), C.POINTER(_I),
                             C.c_char_p, C.c_char_p]),
    "lev_op_serves": (_I, [_P, _P, _L]),
    "lev_gguf_open": (_I, [C.c_char_p, C.POINTER(_P), C.c_char_p, _Z]),
    "lev_gguf_parse": (_I, [_P, _Z, C.POINTER(_P), C.c_char_p, _Z]),
    "lev_gguf_close": (None, [_P]),
    "lev_gguf_summary": (_I, [_P, C.POINTER(C.c_uint32), C.POINTER(_L), C.POINTER(_L), C.POINTER(C.c_uint64),
                              C.POINTER(C.c_uint64)]),
    "lev_gguf_find_tensor": (_L, [_P, C.c_char_p]),
    "lev_gguf_tensor_info": (_I, [_P, _L, C.POINTER(C.c_char_p), C.POINTER(_I), C.POINTER(_I), C.POINTER(_L * 4),
                                  C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "lev_gguf_tensor_data": (_P, [_P, _L]),
    "lev_gguf_meta_u64": (_I, [_P, C.c_char_p, C.POINTER(C.c_uint64)]),
    "lev_gguf_meta_f64": (_I, [_P, C.c_char_p, C.POINTER(C.c_double)]),
    "lev_gguf_meta_string": (_I, [_P, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_Z)]),
    "lev_gguf_meta_array": (_I, [_P, C.c_char_p, C.POINTER(_I), C.POINTER(C.c_uint64)]),
    "lev_gguf_meta_array_item": (_I, [_P, C.c_char_p, C.c_uint64, C.POINTER(_P), C.POINTER(_Z)]),
    "lev_gguf_upload": (_I, [_P, _P, C.c_char_p, C.POINTER(_P)]),
    "lev_gguf_moe_upload": (_I, [_P, _P, _I, _I, _I, C.POINTER(_P), C.POINTER(_I)]),
    "lev_dist_unique_id": (_I, [_P]),
    "lev_dist_init": (_I, [_P, _I, _I, _P]),
    "lev_dist_destroy": (_I, [_P]),
    "lev_dist_peer_memory": (_I, [_P]),
    "lev_matvec_chain_rowsplit": (_I, [_P, _I, C.POINTER(ChainOp)]),
    "lev_matvec_rowsplit_allgather": (_I, [_P, _P, _P, _L, _I, _P, _L, _U]),
    "lev_gemm_prefill_rowsplit_allgather": (_I, [_P, _P, _P, _L, _P, _U]),
    "lev_moe_layer_ep": (_I, [_P, _P, _P, _L, _I, _P, _P, _P, _U]),
}

_lib = None


def load() -> C.CDLL:
    """The loaded library with typed signatures; raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m leviathan_b200.build` "
            "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
