"""tensor-ash GEMM hot path, B200-native: Python host mirror over the C ABI.

Everything here is a thin ctypes layer over ``lib/libtensor_ash.so`` (the
``tensor_ash.h`` symbols).  Class and method names follow the reference crate's
public API (``src/lib.rs:34-58``: ``Executor``, ``Tensor``, ``MatmulCall``,
``MatmulOp``, ``Epilogue``, ``Activation``, ``PreparedOps``, ``RunStats``,
``pack_f16w_row_tiles``, ``f16w_row_tile_n`` ...), so parity tests read like the
reference's own.  There is no CPU path: if the shared library is missing the
import of :mod:`capi` raises, and every compute call needs a CUDA device.
"""
from .api import (  # noqa: F401
    Activation,
    Binary,
    Comm,
    Context,
    DispatchInfo,
    Epilogue,
    ExecKind,
    ExecOp,
    Executor,
    TokenIdBuffer,
    MatmulCall,
    MatmulOp,
    MatmulOpEx,
    MatmulStore,
    PosCell,
    StoreKind,
    PreparedOps,
    RunStats,
    Tensor,
    TensorAshError,
    default_num_k_splits,
    f16w_row_tile_n,
    f32_to_f16_bits,
    pinned_empty,
    f16_bits_to_f32,
    heuristic_kernel,
    heuristic_splits,
    kernel_launch_count,
    kernel_selection_parse,
    kernel_specs,
    pack_f16w_row_tiles,
    resolve_shapes,
    experiment_check,
    tune_candidate_at,
    tune_median,
    tune_store_path,
    tune_store_rewrite,
    version,
)
from .capi import lib, lib_path  # noqa: F401
from .llama import GgufFile, Llama, LlamaConfig, shard_plan, write_gguf  # noqa: F401
