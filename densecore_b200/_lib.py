"""ctypes loader for libdc_b200.so (the C ABI declared in include/dc_b200.h).

There is no fallback: if the shared library is missing the import of any op
fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# DC_B200_LIB points at another build of the same library (A/B timing of two builds)
LIB_PATH = os.environ.get("DC_B200_LIB") or os.path.join(PKG, "libdc_b200.so")

OK = 0
STATUS_NAMES = {
    0: "OK", -1: "INVALID_ARGUMENT", -2: "MODEL_LOAD_FAILED", -3: "OUT_OF_MEMORY",
    -5: "INTERNAL_ERROR", -6: "BACKEND_ERROR", -7: "UNSUPPORTED",
}


class DcError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"dc_b200 status {status} ({STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status
        self.message = message


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m densecore_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


class ModelConfig(C.Structure):
    """dc_model_config of include/dc_b200.h."""
    _fields_ = [
        ("n_layer", C.c_int), ("hidden", C.c_int), ("n_head", C.c_int), ("n_kv_head", C.c_int),
        ("head_dim", C.c_int), ("vocab", C.c_int), ("ffn", C.c_int), ("n_expert", C.c_int),
        ("n_expert_used", C.c_int), ("expert_ffn", C.c_int), ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("routed_scale", C.c_float), ("tie_embeddings", C.c_int), ("qk_norm", C.c_int), ("max_seqs", C.c_int),
        ("max_ctx", C.c_int), ("ep_rank", C.c_int), ("ep_size", C.c_int),
    ]


def _signatures() -> dict:
    vp, i32, i64, sz, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float
    u64, u32, cstr = C.c_uint64, C.c_uint32, C.c_char_p
    pp = C.POINTER(C.c_void_p)
    pi = C.POINTER(C.c_int)
    return {
        "dc_b200_init": (i32, [i32, pp]),
        "dc_b200_destroy": (None, [vp]),
        "dc_b200_last_error": (cstr, [vp]),
        "dc_b200_stream": (vp, [vp]),
        "dc_b200_synchronize": (i32, [vp]),
        "dc_b200_set_option": (i32, [vp, cstr, i32]),
        "dc_b200_profiler_range": (i32, [i32]),
        "dc_b200_upload_weight": (i32, [vp, i32, C.POINTER(i64), vp, pp]),
        "dc_b200_free_weight": (i32, [vp, vp]),
        "dc_b200_weight_data": (vp, [vp, C.POINTER(sz)]),
        "dc_b200_quantize_q8k": (i32, [vp, vp, i32, i32, vp]),
        "dc_b200_quantize_q8k_dev": (i32, [vp, vp, i32, i32, vp]),
        "dc_b200_mul_mat": (i32, [vp, vp, vp, i32, vp]),
        "dc_b200_mul_mat_dev": (i32, [vp, vp, vp, i32, vp]),
        "dc_b200_mul_mat_dev_noalloc": (i32, [vp, vp, vp, i32, vp]),
        "dc_b200_mul_mat_block_sums": (i32, [vp, vp, vp, i32, vp, vp]),
        "dc_b200_alloc_device": (i32, [vp, sz, pp]),
        "dc_b200_free_device": (i32, [vp, vp]),
        "dc_b200_copy_to_device": (i32, [vp, vp, vp, sz]),
        "dc_b200_copy_from_device": (i32, [vp, vp, vp, sz]),
        "dc_b200_mul_mat_id": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32, vp, vp, vp]),
        "dc_b200_mul_mat_id_dev": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32, vp, vp, vp]),
        "dc_b200_moe_forward": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32, vp, vp, vp]),
        "dc_b200_moe_route": (i32, [vp, vp, i32, i32, i32, f32, vp, vp]),
        "dc_b200_kv_create": (i32, [vp, i32, i32, i32, i32, i32, i32, pp]),
        "dc_b200_kv_destroy": (None, [vp]),
        "dc_b200_kv_seq_alloc": (i32, [vp, pi]),
        "dc_b200_kv_seq_free": (i32, [vp, i32]),
        "dc_b200_kv_seq_reserve": (i32, [vp, i32, i32]),
        "dc_b200_kv_block_table": (i32, [vp, i32, vp, i32, pi]),
        "dc_b200_kv_free_blocks": (i32, [vp]),
        "dc_b200_kv_prefix_attach": (i32, [vp, i32, vp, i32, pi]),
        "dc_b200_kv_prefix_register": (i32, [vp, i32, vp, i32]),
        "dc_b200_kv_prefix_stats": (i32, [vp, vp]),
        "dc_b200_kv_prefix_hash": (C.c_uint64, [vp, i32]),
        "dc_b200_model_prefix_stats": (i32, [vp, vp]),
        "dc_b200_sched_create": (i32, [vp, i32, i32, i32, pp]),
        "dc_b200_sched_destroy": (None, [vp]),
        "dc_b200_sched_add": (i32, [vp, vp, i32, i32, pi]),
        "dc_b200_sched_step": (i32, [vp, vp, i32, pi]),
        "dc_b200_sched_pending": (i32, [vp]),
        "dc_b200_sched_stats": (i32, [vp, vp]),
        "dc_b200_flash_attn_decode": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, f32, vp]),
        "dc_b200_flash_attn_prefill": (i32, [vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, f32, vp]),
        "dc_b200_kv_read_block": (i32, [vp, i32, i32, vp, vp]),
        "dc_b200_argmax": (i32, [vp, vp, i32, i32, vp]),
        "dc_b200_verify_accept": (i32, [vp, vp, vp, vp, vp, u64, u32, i32, i32, i32, f32, pi, pi]),
        "dc_b200_verify_uniforms": (i32, [vp, u64, u32, i32, vp]),
        "dc_b200_verify_accept_dev": (i32, [vp, vp, vp, vp, vp, u64, u32, i32, i32, i32, f32, pi, pi]),
        "dc_b200_softmax": (i32, [vp, vp, i32, i32, f32, vp]),
        "dc_b200_sample_dev": (i32, [vp, vp, i32, f32, f32, vp, pi]),
        "dc_b200_model_create": (i32, [vp, C.POINTER(ModelConfig), pp]),
        "dc_b200_model_destroy": (None, [vp]),
        "dc_b200_model_set_tensor": (i32, [vp, cstr, i32, C.POINTER(i64), vp]),
        "dc_b200_model_init_synthetic": (i32, [vp, u64, f32]),
        "dc_b200_model_get_tensor": (i32, [vp, cstr, pi, C.POINTER(i64), pp, C.POINTER(sz)]),
        "dc_b200_model_finalize": (i32, [vp]),
        "dc_b200_model_weight_bytes": (sz, [vp]),
        "dc_b200_seq_alloc": (i32, [vp, pi]),
        "dc_b200_seq_free": (i32, [vp, i32]),
        "dc_b200_seq_fork": (i32, [vp, i32, pi]),
        "dc_b200_model_free_blocks": (i32, [vp]),
        "dc_b200_kv_seq_fork": (i32, [vp, i32, pi]),
        "dc_b200_kv_block_refcount": (i32, [vp, i32]),
        "dc_b200_seq_len": (i32, [vp, i32]),
        "dc_b200_seq_truncate": (i32, [vp, i32, i32]),
        "dc_b200_prefill": (i32, [vp, i32, vp, i32, vp, pi]),
        "dc_b200_decode_step": (i32, [vp, vp, i32, vp, vp, vp]),
        "dc_b200_decode_run": (i32, [vp, vp, i32, vp, i32, vp, C.POINTER(f32)]),
        "dc_b200_forward_chunk": (i32, [vp, i32, vp, i32, vp]),
        "dc_b200_model_logits_dev": (vp, [vp]),
        "dc_b200_model_phase_timing": (i32, [vp, vp, i32]),
        "dc_b200_model_step_stats": (i32, [vp, pi, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
        "dc_b200_model_set_option": (i32, [vp, cstr, i32]),
        "dc_b200_model_profile_step": (i32, [vp, vp, i32, vp, i32, vp, vp, vp]),
        "dc_b200_kernel_class_name": (cstr, [i32]),
        "dc_b200_ep_unique_id": (i32, [vp, cstr, vp]),
        "dc_b200_model_ep_init": (i32, [vp, cstr, vp]),
        "dc_b200_model_ep_export": (i32, [vp, vp]),
        "dc_b200_model_tensor_names": (i32, [vp, vp, i32, vp]),
        "dc_b200_model_get_config": (i32, [vp, vp]),
        "dc_b200_model_from_gguf": (i32, [vp, cstr, i32, i32, i32, i32, vp]),
        "dc_b200_model_ep_import": (i32, [vp, i32, vp]),
        "dc_b200_model_read_layer_input": (i32, [vp, i32, i32, vp]),
        "dc_b200_model_read_kv": (i32, [vp, i32, i32, i32, i32, vp, vp]),
    }


def _declare(l: C.CDLL) -> None:
    for name, (res, args) in _signatures().items():
        if os.environ.get("DC_B200_LIB") and not hasattr(l, name):
            continue   # an older build named for A/B timing may lack the newest entry points
        fn = getattr(l, name)
        fn.restype = res
        fn.argtypes = args


def exported_symbols() -> list[str]:
    """Names this binding expects the library to export (checked by the CPU tests)."""
    return list(_signatures())
