"""ctypes declarations for every symbol of ``include/tensor_ash.h``.

The structs below are field-for-field the C structs of the header (and so of
the reference's ``include/tensor_ash.h:16-108``).  Loading fails loudly when
the shared library has not been built: there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def lib_path() -> str:
    return os.path.join(_HERE, "lib", "libtensor_ash.so")


class RunStatsC(C.Structure):
    _fields_ = [("has_gpu_time", C.c_uint32), ("gpu_time_ns", C.c_uint64), ("n_calls", C.c_size_t),
                ("total_flops", C.c_uint64), ("tflops", C.c_double)]


class MatmulCallC(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("alpha", C.c_float),
                ("accumulate", C.c_uint32)]


class EpilogueC(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("activation", C.c_uint32), ("binary_kind", C.c_uint32),
                ("d", C.c_void_p), ("beta", C.c_float)]


class MatmulOpC(C.Structure):
    _fields_ = [("call", MatmulCallC), ("epilogue", EpilogueC)]


class RopeDescC(C.Structure):
    _fields_ = [("heads", C.c_uint32), ("head_dim", C.c_uint32), ("rot_dim", C.c_uint32),
                ("pos_base", C.c_uint32)]


class CopyDescC(C.Structure):
    _fields_ = [("extent", C.c_uint32 * 3), ("src_offset", C.c_uint32), ("src_strides", C.c_uint32 * 3),
                ("dst_offset", C.c_uint32), ("dst_strides", C.c_uint32 * 3)]


class DispatchInfoC(C.Structure):
    _fields_ = [("kernel", C.c_char_p), ("tile", C.c_uint32 * 3), ("has_split_k2", C.c_uint32),
                ("split_k2_splits", C.c_uint32)]


class StoreDescC(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("head_dim", C.c_uint32), ("pos_base", C.c_uint32),
                ("pos_scale", C.c_uint32), ("stride_head", C.c_uint32), ("stride_dim", C.c_uint32),
                ("table", C.c_void_p), ("dst", C.c_void_p), ("pos_cell", C.c_void_p)]


class MatmulOpExC(C.Structure):
    _fields_ = [("op", MatmulOpC), ("packed_b", C.c_uint32), ("normed_weight", C.c_void_p),
                ("normed_eps", C.c_float), ("store", StoreDescC)]


class HostBatchedMatmulC(C.Structure):
    _fields_ = [("batch", C.c_uint32), ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("a", C.c_void_p), ("b", C.c_void_p), ("b_host", C.c_void_p), ("c", C.c_void_p),
                ("bias", C.c_void_p), ("bias_per_batch", C.c_uint32), ("d", C.c_void_p),
                ("activation", C.c_uint32), ("binary", C.c_uint32), ("alpha", C.c_float), ("beta", C.c_float),
                ("chunk_batch", C.c_uint32)]


class FlashDescC(C.Structure):
    _fields_ = [("kv_len", C.c_uint32), ("pos_base", C.c_uint32), ("scale", C.c_float),
                ("token_major_heads", C.c_uint32), ("out_token_major_heads", C.c_uint32), ("simt", C.c_uint32)]


class AttnDecodeDescC(C.Structure):
    _fields_ = [("kv_len", C.c_uint32), ("scale", C.c_float), ("pos_cell", C.c_void_p)]


class ExecOpC(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("mm", MatmulOpExC),
                ("in0", C.c_void_p), ("in1", C.c_void_p), ("in2", C.c_void_p), ("in3", C.c_void_p),
                ("out", C.c_void_p), ("f0", C.c_float), ("u0", C.c_uint32), ("u1", C.c_uint32),
                ("u2", C.c_uint32), ("rope", RopeDescC), ("copy", CopyDescC), ("dst_offset", C.c_uint32),
                ("dst_strides", C.c_uint32 * 3), ("pos_scale", C.c_uint32), ("flash", FlashDescC),
                ("attn", AttnDecodeDescC), ("cell", C.c_void_p), ("tokens", C.c_void_p), ("comm", C.c_void_p)]


class LlamaBreakdownRowC(C.Structure):
    _fields_ = [("op_class", C.c_char_p), ("gpu_ns", C.c_uint64), ("calls", C.c_uint32)]


class LlamaConfigC(C.Structure):
    _fields_ = [("layers", C.c_uint32), ("embd", C.c_uint32), ("heads", C.c_uint32), ("kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32), ("t_max", C.c_uint32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("weight_sigma", C.c_float),
                ("norm_jitter", C.c_float), ("seed", C.c_uint64)]


_P = C.c_void_p
_U32 = C.c_uint32
_SZ = C.c_size_t
_STATS = C.POINTER(RunStatsC)

# name -> (restype, argtypes); this table is also what the symbol-export test walks.
SIGNATURES = {
    "ta_version": (C.c_char_p, []),
    "ta_last_error": (C.c_char_p, []),
    "ta_context_create": (_P, [_U32, C.c_char_p]),
    "ta_context_destroy": (None, [_P]),
    "ta_context_supports_f16": (_U32, [_P]),
    "ta_context_supports_bda": (_U32, [_P]),
    "ta_executor_create": (_P, [_P, _SZ, _U32, C.c_char_p]),
    "ta_executor_create_v2": (_P, [_P, _SZ, _U32, C.c_char_p, _U32]),
    "ta_executor_destroy": (None, [_P]),
    "ta_tensor_create": (_P, [_P, C.POINTER(_U32), _SZ]),
    "ta_tensor_create_on_executor": (_P, [_P, C.POINTER(_U32), _SZ]),
    "ta_tensor_create_f16": (_P, [_P, C.POINTER(_U32), _SZ]),
    "ta_tensor_create_f16_on_executor": (_P, [_P, C.POINTER(_U32), _SZ]),
    "ta_tensor_destroy": (None, [_P]),
    "ta_tensor_len": (C.c_uint64, [_P]),
    "ta_tensor_size_bytes": (C.c_uint64, [_P]),
    "ta_tensor_is_f16": (_U32, [_P]),
    "ta_upload": (C.c_int, [_P, _P, _P, _SZ]),
    "ta_download": (C.c_int, [_P, _P, _P, _SZ]),
    "ta_matmul": (C.c_int, [_P, _P, _P, _P, C.c_float, _U32, _STATS]),
    "ta_matmul_batch": (C.c_int, [_P, C.POINTER(MatmulCallC), _SZ, _STATS]),
    "ta_run_ops": (C.c_int, [_P, C.POINTER(MatmulOpC), _SZ, _STATS]),
    "ta_run_matmul_host_batched": (C.c_int, [_P, C.POINTER(HostBatchedMatmulC), _STATS]),
    "ta_pinned_alloc": (C.c_void_p, [_SZ]),
    "ta_pinned_free": (None, [C.c_void_p]),
    "ta_run_op_graph": (C.c_int, [_P, C.POINTER(MatmulOpC), _SZ, _STATS]),
    "ta_softmax_rows": (C.c_int, [_P, _P, _P, C.c_float, _U32, _U32, _U32, _STATS]),
    "ta_rms_norm": (C.c_int, [_P, _P, _P, _P, C.c_float, _STATS]),
    "ta_layer_norm": (C.c_int, [_P, _P, _P, _P, _P, C.c_float, _STATS]),
    "ta_rope": (C.c_int, [_P, _P, _P, _P, C.POINTER(RopeDescC), _STATS]),
    "ta_copy_strided": (C.c_int, [_P, _P, _P, C.POINTER(CopyDescC), _STATS]),
    "ta_prepared_create": (_P, [_P, C.POINTER(MatmulOpC), _SZ, _U32]),
    "ta_prepared_run": (C.c_int, [_P, _STATS]),
    "ta_prepared_submit": (C.c_int, [_P]),
    "ta_prepared_wait": (C.c_int, [_P, _STATS]),
    "ta_prepared_destroy": (None, [_P]),
    "ta_dispatch_info_for": (C.c_int, [_P, _U32, _U32, _U32, _U32, _U32, C.POINTER(DispatchInfoC)]),
    "ta_tune_shape": (C.c_int, [_P, _U32, _U32, _U32, _U32]),
    # ---- additive entry points
    "ta_matmul_split_k2": (C.c_int, [_P, C.POINTER(MatmulCallC), _SZ, _U32, _STATS]),
    "ta_split_k2_noalloc": (C.c_int, [_P, _P, _P, _U32, _U32, _U32, _U32, C.c_float, _P]),
    "ta_run_ops_ex": (C.c_int, [_P, C.POINTER(MatmulOpExC), _SZ, _U32, _STATS]),
    "ta_swiglu_gemv": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_float, _STATS]),
    "ta_pack_f16w_row_tiles": (C.c_int, [_P, _P, _SZ, _SZ, _SZ]),
    "ta_f16w_row_tile_n": (_U32, [_U32, _U32]),
    "ta_upload_f16": (C.c_int, [_P, _P, _P, _SZ]),
    "ta_tensor_alias_with_shape": (_P, [_P, C.POINTER(_U32), _SZ]),
    "ta_flash_attention": (C.c_int, [_P, _P, _P, _P, _P, C.POINTER(FlashDescC), _STATS]),
    "ta_attn_decode_num_chunks": (_U32, [_U32]),
    "ta_attn_decode": (C.c_int, [_P, _P, _P, _P, _P, _P, C.POINTER(AttnDecodeDescC), _STATS]),
    "ta_pos_cell_create": (_P, [_P]),
    "ta_pos_cell_destroy": (None, [_P]),
    "ta_pos_cell_set": (C.c_int, [_P, _U32]),
    "ta_pos_cell_get": (C.c_int, [_P, C.POINTER(_U32)]),
    "ta_token_ids_create": (_P, [_P, _U32]),
    "ta_token_ids_destroy": (None, [_P]),
    "ta_token_ids_set": (C.c_int, [_P, _P, _U32]),
    "ta_run_exec_ops": (C.c_int, [_P, C.POINTER(ExecOpC), _SZ, _STATS]),
    "ta_prepared_create_exec": (_P, [_P, C.POINTER(ExecOpC), _SZ]),
    "ta_kernel_spec_count": (_SZ, []),
    "ta_kernel_spec_at": (C.c_int, [_SZ, C.POINTER(DispatchInfoC)]),
    "ta_kernel_selection_parse": (C.c_int, [C.c_char_p]),
    "ta_resolve_shapes": (C.c_int, [C.POINTER(_U32), _SZ, C.POINTER(_U32), _SZ, C.POINTER(_U32), _SZ,
                                    C.POINTER(_U32)]),
    "ta_default_num_k_splits": (_U32, [_U32] * 6),
    "ta_heuristic_splits": (_U32, [_U32] * 4),
    "ta_heuristic_kernel": (C.c_char_p, [_U32] * 4 + [C.c_int, C.c_int]),
    "ta_f32_to_f16_bits": (C.c_uint16, [C.c_float]),
    "ta_f16_bits_to_f32": (C.c_float, [C.c_uint16]),
    "ta_tensor_device_ptr": (_P, [_P]),
    "ta_context_device_index": (C.c_int, [_P]),
    "ta_context_device_name": (C.c_char_p, [_P]),
    "ta_kernel_launch_count": (C.c_uint64, []),
    "ta_tune_shape_f16w": (C.c_int, [_P, _U32, _U32, _U32, _U32]),
    "ta_tune_median": (C.c_int, [C.POINTER(C.c_uint64), _SZ, C.POINTER(C.c_uint64)]),
    "ta_tune_candidate_at": (_SZ, [_SZ, _U32, _SZ]),
    "ta_tune_store_path": (C.c_int, [C.c_char_p, C.c_char_p, _SZ]),
    "ta_tune_store_rewrite": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(_SZ)]),
    "ta_experiment_check": (C.c_int, [C.c_char_p]),
    "ta_selftest_bounded_wait": (C.c_int, [_P, _U32]),
    "ta_comm_unique_id": (C.c_int, [_P]),
    "ta_comm_create": (_P, [_P, _U32, _U32, _P]),
    "ta_comm_destroy": (None, [_P]),
    "ta_comm_set_wait_limit_ns": (C.c_int, [_P, C.c_uint64]),
    "ta_comm_resync": (C.c_int, [_P]),
    "ta_comm_rank": (_U32, [_P]),
    "ta_comm_world": (_U32, [_P]),
    # ---- tensor_ash_llama.h
    "ta_llama_create_random": (_P, [_P, C.POINTER(LlamaConfigC)]),
    "ta_llama_create_random_tp": (_P, [_P, C.POINTER(LlamaConfigC), _P]),
    "ta_llama_load_gguf": (_P, [_P, C.c_char_p, _U32, _P]),
    "ta_llama_get_config": (C.c_int, [_P, C.POINTER(LlamaConfigC)]),
    "ta_gguf_open": (_P, [C.c_char_p]),
    "ta_gguf_close": (None, [_P]),
    "ta_gguf_meta_kind": (C.c_int, [_P, C.c_char_p]),
    "ta_gguf_meta_u64": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64)]),
    "ta_gguf_meta_f64": (C.c_int, [_P, C.c_char_p, C.c_double, C.POINTER(C.c_double)]),
    "ta_gguf_meta_str": (C.c_int, [_P, C.c_char_p, C.c_char_p, _SZ]),
    "ta_gguf_tensor_info": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(_U32), C.POINTER(_U32),
                                      C.POINTER(C.c_uint64)]),
    "ta_gguf_read_f32": (C.c_int, [_P, C.c_char_p, _P, _SZ]),
    "ta_gguf_data_start": (C.c_uint64, [_P]),
    "ta_llama_destroy": (None, [_P]),
    "ta_llama_reset": (C.c_int, [_P]),
    "ta_llama_prefill": (C.c_int, [_P, C.POINTER(_U32), _U32, C.POINTER(_U32), _STATS]),
    "ta_llama_decode": (C.c_int, [_P, _U32, _U32, C.POINTER(_U32), _STATS]),
    "ta_llama_decode_breakdown": (C.c_int, [_P, _U32, C.POINTER(LlamaBreakdownRowC), _SZ, C.POINTER(_SZ), C.POINTER(_SZ),
                                          C.POINTER(_U32)]),
    "ta_llama_logits": (C.c_int, [_P, _P, _SZ]),
    "ta_llama_position": (_U32, [_P]),
    "ta_llama_weight_bytes_per_token": (C.c_uint64, [_P]),
}

_lib = None


def lib():
    """The loaded shared library with argtypes/restype set on every symbol."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python tensor-ash_b200/build.py` "
            "(nvcc, sm_100a).  This library has no CPU or pure-Python fallback.")
    L = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L
