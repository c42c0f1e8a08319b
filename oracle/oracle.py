"""ctypes/numpy front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads ``oracle/_build/libta_oracle.so`` (built from ``ta_oracle.c`` by the
Makefile beside it) and exposes each function on numpy arrays.  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg import this module;
the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libta_oracle.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile if it is missing or stale."""
    src = os.path.join(_HERE, "ta_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


REF_C_SMOKE = os.path.join(_HERE, "_ref", "c_smoke")


def build_ref_c_smoke(reference_root: str = "/root/reference"):
    """Compiles the reference's own C acceptance program (examples/c_smoke.c), unchanged and from
    where it lies, against this repository's header and library.  Returns the binary's path, or
    None when the reference tree is not present (the prebuilt binary, if any, is left alone)."""
    src = os.path.join(reference_root, "examples", "c_smoke.c")
    if not os.path.exists(src):
        return REF_C_SMOKE if os.path.exists(REF_C_SMOKE) else None
    subprocess.run(["make", "-C", _HERE, "ref_c_smoke", f"REF={reference_root}"], check=True, capture_output=True)
    return REF_C_SMOKE


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_SO)
    L.tao_fill_det.argtypes = [_f32p, C.c_size_t, C.c_uint64]
    L.tao_fill_normal.argtypes = [_f32p, C.c_size_t, C.c_uint64, C.c_double]
    L.tao_lcg_new.argtypes = [C.c_uint64]
    L.tao_lcg_new.restype = C.c_uint64
    L.tao_lcg_next.argtypes = [C.POINTER(C.c_uint64)]
    L.tao_lcg_next.restype = C.c_uint64
    L.tao_lcg_range_u32.argtypes = [C.POINTER(C.c_uint64), C.c_uint32, C.c_uint32]
    L.tao_lcg_range_u32.restype = C.c_uint32
    L.tao_f32_to_f16_bits.argtypes = [C.c_float]
    L.tao_f32_to_f16_bits.restype = C.c_uint16
    L.tao_f16_bits_to_f32.argtypes = [C.c_uint16]
    L.tao_f16_bits_to_f32.restype = C.c_float
    L.tao_f16_bits_to_f32_reference.argtypes = [C.c_uint16]
    L.tao_f16_bits_to_f32_reference.restype = C.c_float
    L.tao_round_via_f16.argtypes = [C.c_float]
    L.tao_round_via_f16.restype = C.c_float
    L.tao_round_via_f16_array.argtypes = [_f32p, C.c_size_t]
    L.tao_f32_to_f16_array.argtypes = [_f32p, _u16p, C.c_size_t]
    L.tao_cpu_bmm.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                              C.c_float, C.c_int, C.c_int, C.c_int, C.c_int]
    L.tao_cpu_dot.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_float]
    L.tao_cpu_dot.restype = C.c_float
    L.tao_activate.argtypes = [C.c_double, C.c_int]
    L.tao_activate.restype = C.c_double
    L.tao_cpu_epilogue.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int,
                                   C.c_int, C.c_int, C.c_void_p, C.c_float]
    L.tao_tolerance.argtypes = [C.c_uint32]
    L.tao_tolerance.restype = C.c_float
    L.tao_max_abs_err.argtypes = [_f32p, _f32p, C.c_size_t, C.POINTER(C.c_size_t)]
    L.tao_max_abs_err.restype = C.c_float
    L.tao_pack_f16w_row_tiles.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t]
    L.tao_pack_f16w_row_tiles.restype = C.c_int
    L.tao_f16w_row_tile_n.argtypes = [C.c_uint32, C.c_uint32]
    L.tao_f16w_row_tile_n.restype = C.c_uint32
    L.tao_splitk_bounds.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32),
                                    C.POINTER(C.c_uint32)]
    L.tao_splitk2_f32.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_float]
    L.tao_default_num_k_splits.argtypes = [C.c_uint32] * 6
    L.tao_default_num_k_splits.restype = C.c_uint32
    L.tao_heuristic_splits.argtypes = [C.c_uint32] * 4
    L.tao_heuristic_splits.restype = C.c_uint32
    L.tao_row_gemv_f32.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32]
    L.tao_cpu_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float]
    L.tao_cpu_layernorm.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float]
    L.tao_cpu_softmax_rows.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_float, C.c_uint32,
                                       C.c_uint32, C.c_uint32]
    L.tao_cpu_rope.argtypes = [_f32p, _f32p, _f32p] + [C.c_uint32] * 5
    L.tao_cpu_argmax.argtypes = [_f32p, C.c_uint32]
    L.tao_cpu_argmax.restype = C.c_uint32
    L.tao_cpu_flash.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_uint32] * 7 + [C.c_float]
    L.tao_cpu_attn_decode.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_uint32] * 5 + [C.c_float]
    L.tao_num_threads.restype = C.c_int
    _lib = L
    return L


# ---------------------------------------------------------------- inputs
def fill_det(n: int, seed: int) -> np.ndarray:
    out = np.empty(int(n), dtype=np.float32)
    lib().tao_fill_det(out, out.size, seed)
    return out


def fill_det_shape(shape, seed: int) -> np.ndarray:
    return fill_det(int(np.prod(shape)), seed).reshape(shape)


def fill_normal(shape, seed: int, sigma: float) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), dtype=np.float32)
    lib().tao_fill_normal(out, out.size, seed, float(sigma))
    return out.reshape(shape)


class LcgRng:
    def __init__(self, seed: int):
        self._s = C.c_uint64(lib().tao_lcg_new(seed))

    def next_u64(self) -> int:
        return int(lib().tao_lcg_next(C.byref(self._s)))

    def range_u32(self, lo: int, hi: int) -> int:
        assert lo <= hi
        return int(lib().tao_lcg_range_u32(C.byref(self._s), lo, hi))


# ---------------------------------------------------------------- f16
def f32_to_f16_bits(v: float) -> int:
    return int(lib().tao_f32_to_f16_bits(np.float32(v)))


def f16_bits_to_f32(b: int) -> np.float32:
    return np.float32(lib().tao_f16_bits_to_f32(b))


def f16_bits_to_f32_reference(b: int) -> np.float32:
    """The reference's host decode, bit for bit (differs from IEEE on subnormal halves only)."""
    return np.float32(lib().tao_f16_bits_to_f32_reference(b))


def round_via_f16(x):
    if np.isscalar(x):
        return np.float32(lib().tao_round_via_f16(np.float32(x)))
    out = np.ascontiguousarray(x, dtype=np.float32).copy()
    lib().tao_round_via_f16_array(out.reshape(-1), out.size)
    return out


def f32_to_f16_array(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().tao_f32_to_f16_array(x.reshape(-1), out.reshape(-1), x.size)
    return out


# ---------------------------------------------------------------- GEMM
def cpu_bmm(a, b, batch, m, n, k, alpha=1.0, c_init=None, accumulate=False, threads=0):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    a_batched = a.size == batch * m * k
    b_batched = b.size == batch * k * n
    assert a_batched or a.size == m * k
    assert b_batched or b.size == k * n
    c = np.zeros(batch * m * n, dtype=np.float32)
    if c_init is not None:
        c[:] = np.asarray(c_init, dtype=np.float32).reshape(-1)
    lib().tao_cpu_bmm(a, b, c, batch, m, n, k, alpha, int(accumulate), int(a_batched),
                      int(b_batched), threads)
    return c


def cpu_dot(a_row: np.ndarray, b: np.ndarray, col: int, alpha: float = 1.0) -> np.float32:
    """f64-accumulated dot of one A row with column `col` of row-major B [K, N]."""
    a_row = np.ascontiguousarray(a_row, dtype=np.float32)
    assert b.dtype == np.float32 and b.flags.c_contiguous and b.ndim == 2
    k, n = b.shape
    base = b.ctypes.data + 4 * col
    return np.float32(lib().tao_cpu_dot(a_row.ctypes.data, base, k, n, alpha))


ACT = {"none": 0, "relu": 1, "silu": 2, "gelu": 3}
BIN = {"none": 0, "add_scaled": 1, "mul": 2}


def activate(x: float, act) -> float:
    return float(lib().tao_activate(float(x), ACT[act] if isinstance(act, str) else int(act)))


def cpu_epilogue(c, batch, m, n, bias=None, act=0, binary=0, d=None, beta=0.0):
    c = np.ascontiguousarray(c, dtype=np.float32).reshape(-1)
    act = ACT[act] if isinstance(act, str) else int(act)
    binary = BIN[binary] if isinstance(binary, str) else int(binary)
    bias_p, bias_batched = None, 0
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        bias_batched = int(bias.size == batch * n and batch > 1)
        bias_p = bias.ctypes.data
    d_p = None
    if d is not None:
        d = np.ascontiguousarray(d, dtype=np.float32).reshape(-1)
        assert d.size == c.size
        d_p = d.ctypes.data
    lib().tao_cpu_epilogue(c, batch, m, n, bias_p, bias_batched, act, binary, d_p, beta)
    return c


def tolerance(k: int) -> float:
    return float(lib().tao_tolerance(k))


def max_abs_err(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    assert a.size == b.size, "slice lengths differ"
    idx = C.c_size_t(0)
    e = lib().tao_max_abs_err(a, b, a.size, C.byref(idx))
    return float(e), int(idx.value)


def pack_f16w_row_tiles(src, k, n, tile_n):
    src = np.ascontiguousarray(src, dtype=np.float32).reshape(-1)
    assert src.size == k * n
    out = np.empty_like(src)
    rc = lib().tao_pack_f16w_row_tiles(src, out, k, n, tile_n)
    assert rc == 0, f"N={n} is not a multiple of tile_n={tile_n}"
    return out


def f16w_row_tile_n(k, n):
    return int(lib().tao_f16w_row_tile_n(k, n))


def splitk_bounds(k, splits, i):
    lo, hi = C.c_uint32(0), C.c_uint32(0)
    lib().tao_splitk_bounds(k, splits, i, C.byref(lo), C.byref(hi))
    return int(lo.value), int(hi.value)


def splitk2_f32(a, b, m, n, k, splits, alpha=1.0):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    c = np.empty(m * n, dtype=np.float32)
    lib().tao_splitk2_f32(a, b, c, m, n, k, splits, alpha)
    return c


def default_num_k_splits(batch, m, n, k, tile_m, tile_n):
    return int(lib().tao_default_num_k_splits(batch, m, n, k, tile_m, tile_n))


def heuristic_splits(batch, m, n, k):
    v = int(lib().tao_heuristic_splits(batch, m, n, k))
    return v or None


def row_gemv_f32(a, b, n, k, kslices):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    c = np.empty(n, dtype=np.float32)
    lib().tao_row_gemv_f32(a, b, c, n, k, kslices)
    return c


# ---------------------------------------------------------------- model ops
def cpu_rmsnorm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty_like(x)
    lib().tao_cpu_rmsnorm(x.reshape(-1), np.ascontiguousarray(w, dtype=np.float32), out.reshape(-1),
                          rows, cols, eps)
    return out


def cpu_layernorm(x, w, b, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty_like(x)
    lib().tao_cpu_layernorm(x.reshape(-1), np.ascontiguousarray(w, dtype=np.float32),
                            np.ascontiguousarray(b, dtype=np.float32), out.reshape(-1), rows, cols, eps)
    return out


def cpu_softmax_rows(x, scale=1.0, mask_kind=0, valid_or_prefix=0, rows_per_group=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty_like(x)
    lib().tao_cpu_softmax_rows(x.reshape(-1), out.reshape(-1), rows, cols, scale, mask_kind,
                               valid_or_prefix, rows_per_group)
    return out


def cpu_rope(x, table, tokens, heads, head_dim, rot_dim, pos_base):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().tao_cpu_rope(x.reshape(-1), np.ascontiguousarray(table, dtype=np.float32).reshape(-1),
                       out.reshape(-1), tokens, heads, head_dim, rot_dim, pos_base)
    return out


def cpu_argmax(x) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    return int(lib().tao_cpu_argmax(x, x.size))


def cpu_flash(q, kt, v, heads, kv_heads, t_q, dh, t_max, kv_len, pos_base, scale):
    q = np.ascontiguousarray(q, dtype=np.float32).reshape(-1)
    out = np.empty_like(q)
    lib().tao_cpu_flash(q, np.ascontiguousarray(kt, dtype=np.float32).reshape(-1),
                        np.ascontiguousarray(v, dtype=np.float32).reshape(-1), out, heads, kv_heads,
                        t_q, dh, t_max, kv_len, pos_base, scale)
    return out


def cpu_attn_decode(q, kt, v, kv_heads, group, dh, t_max, kv_len, scale):
    q = np.ascontiguousarray(q, dtype=np.float32).reshape(-1)
    out = np.empty_like(q)
    lib().tao_cpu_attn_decode(q, np.ascontiguousarray(kt, dtype=np.float32).reshape(-1),
                              np.ascontiguousarray(v, dtype=np.float32).reshape(-1), out, kv_heads,
                              group, dh, t_max, kv_len, scale)
    return out


def num_threads() -> int:
    return int(lib().tao_num_threads())
