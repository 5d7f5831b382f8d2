"""ctypes binding of libsharpmind_cuda.so (the C ABI in include/sharpmind_cuda.h).

The library is the product: if it is missing it is built with nvcc, and if that is impossible the
import fails loudly.  There is no Python or CPU compute path behind these calls.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_LIB = None

c_void_p, c_int, c_float, c_size_t, c_int64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_int64
_pp = C.POINTER(c_void_p)

# name -> (restype, argtypes); mirrors include/sharpmind_cuda.h one to one
SIGNATURES = {
    "smc_version": (c_int, []),
    "smc_device_count": (c_int, [C.POINTER(c_int)]),
    "smc_init": (c_int, [c_int, _pp]),
    "smc_destroy": (None, [c_void_p]),
    "smc_last_error": (C.c_char_p, [c_void_p]),
    "smc_set_option": (c_int, [c_void_p, C.c_char_p, c_int]),
    "smc_raw_tensor_bytes": (c_int64, [c_int, c_int64, c_int64]),
    "smc_synchronize": (c_int, [c_void_p]),
    "smc_device_status": (c_int, [c_void_p, C.POINTER(c_int)]),
    "smc_weight_register": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, _pp]),
    "smc_weight_register_dev": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, _pp]),
    "smc_weight_lookup": (c_int, [c_void_p, c_void_p, _pp]),
    "smc_weight_release": (c_int, [c_void_p, c_void_p]),
    "smc_weight_shape": (c_int, [c_void_p, C.POINTER(c_int), C.POINTER(c_int), C.POINTER(c_int)]),
    "smc_qmatmul_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "smc_host_register": (c_int, [c_void_p, c_void_p, C.c_size_t]),
    "smc_host_unregister": (c_int, [c_void_p, c_void_p]),
    "smc_qmatmul_host_w": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "smc_vecdot_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, C.POINTER(c_float)]),
    "smc_swiglu_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "smc_silu_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "smc_softmax_row_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "smc_rmsnorm_row_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float]),
    "smc_sdpa_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                              c_int, c_int, c_int, c_float]),
    "smc_qmatmul_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_q8act_create": (c_int, [c_void_p, c_int, c_int, _pp]),
    "smc_q8act_destroy": (c_int, [c_void_p, c_void_p]),
    "smc_quantize_q8_dev": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "smc_q8act_read": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_qmatmul_q8_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_qmatmul_q8_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "smc_block_isums_dev": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "smc_quantize_weights_dev": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "smc_rmsnorm_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "smc_swiglu_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "smc_silu_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "smc_softmax_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_rope_tables": (c_int, [c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "smc_rope_dev": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_void_p]),
    "smc_add_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "smc_add_bias_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_linear_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_argmax_dev": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "smc_sample_dev": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_repetition_penalty_dev": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p]),
    "smc_embed_q8_0_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "smc_sdpa_decode_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_float, c_void_p]),
    "smc_kv_create": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, _pp]),
    "smc_kv_destroy": (c_int, [c_void_p, c_void_p]),
    "smc_kv_length": (c_int, [c_void_p]),
    "smc_kv_max_seq": (c_int, [c_void_p]),
    "smc_kv_reset": (c_int, [c_void_p, c_void_p]),
    "smc_kv_truncate": (c_int, [c_void_p, c_void_p, c_int]),
    "smc_kv_trim_to_last": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "smc_kv_update_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_kv_snapshot_bytes": (c_int64, [c_void_p]),
    "smc_kv_snapshot": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, C.POINTER(c_int)]),
    "smc_kv_restore": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "smc_sdpa_kv_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "smc_model_create": (c_int, [c_void_p, c_void_p, c_int, _pp]),
    "smc_model_destroy": (c_int, [c_void_p, c_void_p]),
    "smc_model_kv": (c_int, [c_void_p, c_void_p, _pp, _pp]),
    "smc_model_kv_load": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_qmatmul_tc_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "smc_add_rmsnorm_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "smc_swiglu_quantize_q8_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "smc_add_rmsnorm_q8_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "smc_qmatmul_swiglu_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_qmatmul_addnorm_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_weight_concat_rows": (c_int, [c_void_p, c_void_p, c_int, _pp]),
    "smc_gguf_open": (c_int, [c_void_p, C.c_char_p, _pp]),
    "smc_gguf_close": (c_int, [c_void_p, c_void_p]),
    "smc_gguf_tensor_count": (c_int, [c_void_p]),
    "smc_gguf_find": (c_int, [c_void_p, C.c_char_p]),
    "smc_gguf_tensor_info": (c_int, [c_void_p, c_int, C.POINTER(C.c_char_p), C.POINTER(c_int), C.POINTER(c_int),
                                     C.POINTER(c_int64), C.POINTER(c_int64)]),
    "smc_gguf_meta_int": (c_int, [c_void_p, C.c_char_p, C.POINTER(c_int64)]),
    "smc_gguf_meta_float": (c_int, [c_void_p, C.c_char_p, C.POINTER(C.c_double)]),
    "smc_gguf_meta_string": (C.c_char_p, [c_void_p, C.c_char_p]),
    "smc_gguf_register": (c_int, [c_void_p, c_void_p, c_int, c_int, _pp]),
    "smc_gguf_read_f32": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64]),
    "smc_gather_create": (c_int, [c_void_p, c_int, c_int, c_size_t, _pp]),
    "smc_gather_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "smc_gather_connect": (c_int, [c_void_p, c_void_p, c_void_p]),
    "smc_gather_connect_local": (c_int, [c_void_p, c_void_p, c_void_p]),
    "smc_gather_set_wait_ns": (c_int, [c_void_p, c_void_p, C.c_uint64]),
    "smc_gather_buffer": (c_int, [c_void_p, c_void_p, _pp]),
    "smc_qmatmul_gather_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_gather_exchange_dev": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "smc_gather_destroy": (c_int, [c_void_p, c_void_p]),
    "smc_decode_step": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "smc_forward_last_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "smc_qmatmul_reduce_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "smc_weight_interleave_rows": (c_int, [c_void_p, c_void_p, c_void_p, _pp]),
    "smc_qmatmul_swiglu_pairs_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_dev_alloc": (c_int, [c_void_p, C.c_size_t, C.POINTER(c_void_p)]),
    "smc_dev_free": (c_int, [c_void_p, c_void_p]),
    "smc_copy_to_device": (c_int, [c_void_p, c_void_p, c_void_p, C.c_size_t, c_void_p]),
    "smc_copy_to_host": (c_int, [c_void_p, c_void_p, c_void_p, C.c_size_t, c_void_p]),
    "smc_forward_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_verify_greedy_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "smc_medusa_predict_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smc_kv_append_dev": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p]),
}


def lib_path() -> str:
    return _build.LIB


def load() -> C.CDLL:
    """Loads (building first if needed) the shared library and types every entry point."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_build.LIB):
        _build.build()
    lib = C.CDLL(_build.LIB)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib
