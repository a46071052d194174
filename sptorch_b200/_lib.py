"""ctypes binding of libsptorch_b200.so.  There is no fallback: a missing library or a missing
B200 raises, it never silently computes on the CPU."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libsptorch_b200.so")

_vp, _sz, _f, _i = C.c_void_p, C.c_size_t, C.c_float, C.c_int


class GptConfig(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("d_model", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32),
                ("d_ff", C.c_int32), ("seq_len", C.c_int32), ("dtype", C.c_int32), ("max_batch", C.c_int32),
                ("eps", C.c_float), ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("arch", C.c_int32), ("rope_base", C.c_float)]


ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p)

# name -> (restype, argtypes); the first 20 are the reference's C-ABI (include/sptorch_b200_hal.h)
HAL_SYMBOLS = {
    "sptorch_backend_init": (_i, []),
    "sptorch_backend_shutdown": (None, []),
    "sptorch_backend_name": (C.c_char_p, []),
    "sptorch_alloc": (_vp, [_sz]),
    "sptorch_free": (None, [_vp]),
    "sptorch_copy_h2d": (_i, [_vp, _vp, _sz]),
    "sptorch_copy_d2h": (_i, [_vp, _vp, _sz]),
    "sptorch_sync": (_i, []),
    "sptorch_query_runtime": (_i, [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "sptorch_add_f32": (_i, [_vp, _vp, _vp, _sz]),
    "sptorch_mul_f32": (_i, [_vp, _vp, _vp, _sz]),
    "sptorch_neg_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_exp_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_log_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_relu_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_gelu_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_scale_f32": (_i, [_vp, _f, _vp, _sz]),
    "sptorch_matmul_f32": (_i, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "sptorch_batch_matmul_f32": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz]),
    "sptorch_softmax_f32": (_i, [_vp, _vp, _sz, _sz]),
}

EXT_SYMBOLS = {
    "sptorch_ext_last_error": (C.c_char_p, []),
    "sptorch_ext_device": (_i, []),
    "sptorch_ext_sm_count": (_i, []),
    "sptorch_ext_set_stream": (_i, [_vp]),
    "sptorch_ext_alloc_bytes": (_vp, [_sz]),
    "sptorch_ext_alloc_pinned": (_vp, [_sz]),
    "sptorch_ext_free_pinned": (None, [_vp]),
    "sptorch_ext_copy_h2d_bytes": (_i, [_vp, _vp, _sz]),
    "sptorch_ext_copy_d2h_bytes": (_i, [_vp, _vp, _sz]),
    "sptorch_ext_memset": (_i, [_vp, _i, _sz]),
    "sptorch_ext_set_alloc_budget": (_i, [_sz]),
    "sptorch_ext_set_sm_reserve": (_i, [_i]),
    "sptorch_ext_timer_begin": (_i, []),
    "sptorch_ext_timer_end": (_i, [C.POINTER(C.c_float)]),
    "sptorch_ext_flush_l2": (_i, []),
    "sptorch_ext_device_status": (C.c_uint32, []),
    "sptorch_ext_prof_enable": (_i, [_i]),
    "sptorch_ext_prof_read": (_i, [C.POINTER(C.c_float), C.POINTER(C.c_uint32), _i]),
    "sptorch_ext_f32_to_bf16": (_i, [_vp, _vp, _sz]),
    "sptorch_ext_bf16_to_f32": (_i, [_vp, _vp, _sz]),
    "sptorch_ext_sum_f32": (_i, [_vp, _sz, C.POINTER(C.c_float)]),
    "sptorch_ext_masked_fill_f32": (_i, [_vp, _vp, _f, _vp, _sz]),
    "sptorch_ext_broadcast_add_f32": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "sptorch_ext_embedding_lookup_f32": (_i, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "sptorch_ext_sgd_update_f32": (_i, [_vp, _vp, _f, _sz]),
    "sptorch_ext_adam_update_f32": (_i, [_vp, _vp, _vp, _vp, _sz, _f, _f, _f, _f, _f, _f, _f]),
    "sptorch_ext_add": (_i, [_vp, _vp, _vp, _sz, _i]),
    "sptorch_ext_gelu": (_i, [_vp, _vp, _sz, _i]),
    "sptorch_ext_transpose_f32": (_i, [_vp, _vp, _sz, _sz]),
    "sptorch_ext_layernorm": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _f, _i]),
    "sptorch_ext_causal_softmax": (_i, [_vp, _vp, _sz, _sz, _f, _i]),
    "sptorch_ext_masked_softmax_f32": (_i, [_vp, _vp, _vp, _sz, _sz, _i]),
    "sptorch_ext_embedding_sum": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _i]),
    "sptorch_ext_rms_norm": (_i, [_vp, _vp, _vp, _sz, _sz, _f, _i]),
    "sptorch_ext_swiglu": (_i, [_vp, _vp, _vp, _sz, _i]),
    "sptorch_ext_rope": (_i, [_vp, _sz, _sz, _sz, _sz, _sz, _f, _sz, _i]),
    "sptorch_ext_cross_entropy": (_i, [_vp, _sz, _vp, _sz, _sz, _i, C.c_longlong, _vp, C.POINTER(C.c_float), _i]),
    "sptorch_ext_set_gemm_pair": (_i, [_i]),
    "sptorch_ext_set_matmul_mode": (_i, [_i]),
    "sptorch_ext_matmul_f32_static": (_i, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "sptorch_ext_linear": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _f, _i, _i, _i]),
    "sptorch_ext_set_attention_mode": (_i, [_i]),
    "sptorch_ext_attention_workspace": (_sz, [_sz, _sz, _sz, _sz, _i]),
    "sptorch_ext_attention_causal": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "sptorch_ext_gpt_create": (_vp, [C.POINTER(GptConfig)]),
    "sptorch_ext_gpt_destroy": (None, [_vp]),
    "sptorch_ext_gpt_set_param": (_i, [_vp, C.c_char_p, _vp, _sz]),
    "sptorch_ext_gpt_logits_ld": (_sz, [_vp]),
    "sptorch_ext_gpt_forward": (_i, [_vp, _vp, _i, _i, _vp]),
    "sptorch_ext_gpt_enable_graphs": (_i, [_vp, _i]),
    "sptorch_ext_gpt_enable_taps": (_i, [_vp, _i]),
    "sptorch_ext_gpt_tap": (_vp, [_vp, _i]),
    "sptorch_ext_gpt_forward_host": (_i, [_vp, _vp, _i, _i, _vp, _i]),
    "sptorch_ext_gpt_forward_loss": (_i, [_vp, _vp, _vp, _i, _i, _i, C.c_longlong, _vp, _vp, C.POINTER(C.c_float)]),
    "sptorch_ext_gpt_forward_loss_host": (_i, [_vp, _vp, _vp, _i, _i, _i, C.c_longlong, _vp, C.POINTER(C.c_float), _i]),
    "sptorch_ext_gpt_enable_kv_cache": (_i, [_vp, _i]),
    "sptorch_ext_gpt_cached_len": (_i, [_vp]),
    "sptorch_ext_gpt_window_start": (C.c_longlong, [_vp]),
    "sptorch_ext_gpt_prefill": (_i, [_vp, _vp, _i, _i, _vp]),
    "sptorch_ext_gpt_decode": (_i, [_vp, _vp, _i, _i, _vp]),
    "sptorch_ext_attention_last_token": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i]),
    "sptorch_ext_gpt_launches": (_i, [_vp, _i, _i]),
    "sptorch_ext_gpt_enable_ln_fold": (_i, [_vp, _i]),
    "sptorch_ext_gpt_enable_tp_overlap": (_i, [_vp, _i]),
    "sptorch_ext_sampling_candidates": (_i, [_vp, _sz, _i, _sz, _f, _sz, _f, _f, _vp, _sz, _vp, _vp, _vp, _sz, C.POINTER(_sz)]),
    "sptorch_ext_sampling_candidates_constrained": (_i, [_vp, _sz, _i, _sz, _f, _sz, _f, _f, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _sz, C.POINTER(_sz)]),
    "sptorch_ext_sample_from_candidates": (C.c_longlong, [_vp, _vp, _sz, _f]),
    "sptorch_ext_weights_open": (_vp, [C.c_char_p, _i]),
    "sptorch_ext_weights_close": (None, [_vp]),
    "sptorch_ext_weights_format": (_i, [_vp]),
    "sptorch_ext_weights_count": (_sz, [_vp]),
    "sptorch_ext_weights_name": (C.c_char_p, [_vp, _sz]),
    "sptorch_ext_weights_dtype": (C.c_char_p, [_vp, _sz]),
    "sptorch_ext_weights_ndim": (_sz, [_vp, _sz]),
    "sptorch_ext_weights_dim": (_sz, [_vp, _sz, _sz]),
    "sptorch_ext_weights_numel": (_sz, [_vp, _sz]),
    "sptorch_ext_weights_data": (C.POINTER(C.c_float), [_vp, _sz]),
    "sptorch_ext_gpt_param_count": (_sz, [_vp]),
    "sptorch_ext_gpt_param_info": (_i, [_vp, _sz, C.c_char_p, _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "sptorch_ext_gpt_load_weights": (_i, [_vp, _vp, C.POINTER(C.c_char_p), _sz]),
    "sptorch_ext_gpt_load_bundle": (_i, [_vp, C.c_char_p]),
    "sptorch_ext_gpt_set_allreduce": (_i, [_vp, ALLREDUCE_FN, _vp]),
    "sptorch_ext_tp_param_shard": (_i, [C.c_char_p, _i, _i, _sz, _sz, C.POINTER(_i), C.POINTER(_sz), C.POINTER(_sz)]),
    "sptorch_ext_tp_slice_host": (_i, [_vp, _sz, _sz, _i, _sz, _sz, _vp]),
    "sptorch_ext_tp_rank_folds_residual": (_i, [_i]),
    "sptorch_ext_nccl_unique_id": (_i, [C.c_char_p, _vp]),
    "sptorch_ext_nccl_init": (_i, [C.c_char_p, _vp, _i, _i]),
    "sptorch_ext_nccl_allreduce_sum": (_i, [_vp, _sz, _i]),
    "sptorch_ext_nccl_allreduce_avg_f32": (_i, [_vp, _sz]),
    "sptorch_ext_nccl_shutdown": (_i, []),
    "sptorch_ext_gpt_use_nccl": (_i, [_vp]),
}

_lib = None


def load(path: str | None = None) -> C.CDLL:
    """dlopen the library and bind every declared symbol; raises if the file or a symbol is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(f"{p} is missing: build it with `python -m sptorch_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(p)
    for table in (HAL_SYMBOLS, EXT_SYMBOLS):
        for name, (res, args) in table.items():
            fn = getattr(lib, name)   # AttributeError = missing symbol
            fn.restype = res
            fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


def last_error() -> str:
    return load().sptorch_ext_last_error().decode(errors="replace")
