"""Host logic of the library exercised through the C ABI on a machine with no
GPU: symbol export, null-handle rules, shape resolution, registry and aliases,
split-K heuristics, f16 conversion, packed layout.  The cases restate the
reference's host-only unit tests (file:line cited per test)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for header in ("tensor_ash.h", "tensor_ash_llama.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(ta_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(ta):
    from tensor_ash_b200 import capi
    lib = C.CDLL(capi.lib_path())
    names = declared_functions()
    assert len(names) >= 70
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/*.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"


def test_struct_layouts_match_the_c_header(ta):
    from tensor_ash_b200 import capi
    # x86-64 SysV layouts of the header's structs
    assert C.sizeof(capi.RunStatsC) == 40
    assert C.sizeof(capi.MatmulCallC) == 32
    assert C.sizeof(capi.EpilogueC) == 32
    assert C.sizeof(capi.MatmulOpC) == 64
    assert C.sizeof(capi.RopeDescC) == 16
    assert C.sizeof(capi.CopyDescC) == 44
    assert C.sizeof(capi.DispatchInfoC) == 32


def test_version(ta):
    assert ta.version() == "2.0.0"


# capi/src/api.rs:33-173
def test_null_handles(ta):
    L = ta.lib()
    err = lambda: L.ta_last_error().decode()
    assert L.ta_upload(None, None, None, 0) == -1 and "exec is null" in err()
    for destroy in (L.ta_context_destroy, L.ta_executor_destroy, L.ta_tensor_destroy,
                    L.ta_prepared_destroy, L.ta_pos_cell_destroy):
        destroy(None)
    assert L.ta_context_supports_f16(None) == 0 and L.ta_context_supports_bda(None) == 0
    assert L.ta_tensor_is_f16(None) == 0 and L.ta_tensor_len(None) == 0
    assert L.ta_run_ops(None, None, 0, None) == -1 and "ta_run_ops: exec is null" in err()
    assert L.ta_run_op_graph(None, None, 0, None) == -1 and "ta_run_op_graph: exec is null" in err()
    assert not L.ta_prepared_create(None, None, 0, 0) and "ta_prepared_create: exec is null" in err()
    assert L.ta_prepared_run(None, None) == -1 and "ta_prepared_run: prepared is null" in err()
    assert L.ta_prepared_submit(None) == -1 and "ta_prepared_submit: prepared is null" in err()
    assert L.ta_prepared_wait(None, None) == -1 and "ta_prepared_wait: prepared is null" in err()
    assert L.ta_softmax_rows(None, None, None, 1.0, 0, 0, 0, None) == -1
    assert "ta_softmax_rows: exec is null" in err()
    assert L.ta_rms_norm(None, None, None, None, 1e-5, None) == -1 and "ta_rms_norm: exec is null" in err()
    assert L.ta_layer_norm(None, None, None, None, None, 1e-5, None) == -1
    assert "ta_layer_norm: exec is null" in err()
    assert L.ta_rope(None, None, None, None, None, None) == -1 and "ta_rope: exec is null" in err()
    assert L.ta_copy_strided(None, None, None, None, None) == -1
    assert "ta_copy_strided: exec is null" in err()
    assert L.ta_dispatch_info_for(None, 1, 1, 1, 1, 0, None) == -1
    assert "ta_dispatch_info_for: exec is null" in err()
    assert L.ta_tune_shape(None, 1, 64, 64, 64) == -1 and "ta_tune_shape: exec is null" in err()
    assert L.ta_matmul_split_k2(None, None, 0, 4, None) == -1
    assert "ta_matmul_split_k2: exec is null" in err()
    # the error string is cleared at the start of the next call
    L.ta_kernel_selection_parse(b"auto")
    assert err() == ""


def test_context_creation_fails_loudly_without_a_device(ta):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(ta.TensorAshError, match="no CUDA device|CUDA"):
        ta.Context(False, "auto")
    with pytest.raises(ta.TensorAshError, match="invalid ML_DEVICE"):
        ta.Context(False, "warp-drive")


# src/matmul/tests.rs:4-155
def test_resolves_rank2_and_batched(ta):
    r = ta.resolve_shapes([2, 3], [3, 4], [2, 4])
    assert r == dict(m=2, n=4, k=3, batch=1, batch_stride_a=0, batch_stride_b=0, batch_stride_c=0,
                     total_flops=48)
    r = ta.resolve_shapes([5, 2, 3], [5, 3, 4], [5, 2, 4])
    assert (r["batch"], r["batch_stride_a"], r["batch_stride_b"], r["batch_stride_c"]) == (5, 6, 12, 8)
    assert r["total_flops"] == 240


def test_broadcasts(ta):
    a = ta.resolve_shapes([1, 2, 3], [7, 3, 4], [7, 2, 4])
    b = ta.resolve_shapes([7, 2, 3], [1, 3, 4], [7, 2, 4])
    both = ta.resolve_shapes([1, 2, 3], [1, 3, 4], [7, 2, 4])
    assert (a["batch_stride_a"], a["batch_stride_b"]) == (0, 12)
    assert (b["batch_stride_a"], b["batch_stride_b"]) == (6, 0)
    assert (both["batch_stride_a"], both["batch_stride_b"], both["batch_stride_c"]) == (0, 0, 8)
    assert both["total_flops"] == 336


def test_resolution_rejections(ta):
    E = ta.TensorAshError
    with pytest.raises(E) as e:
        ta.resolve_shapes([2, 3], [5, 4], [2, 4])
    assert "A.K=3" in str(e.value) and "B.K=5" in str(e.value)
    with pytest.raises(E) as e:
        ta.resolve_shapes([7, 2, 3], [7, 3, 4], [1, 2, 4])
    assert "incompatible batch dims" in str(e.value) and "A.B=7" in str(e.value)
    with pytest.raises(E, match="non-zero"):
        ta.resolve_shapes([0, 3], [3, 4], [1, 4])
    U = 2 ** 32 - 1
    with pytest.raises(E) as e:
        ta.resolve_shapes([2, U, U], [1, U, 1], [2, U, 1])
    assert "A batch stride" in str(e.value) and "overflows" in str(e.value)
    with pytest.raises(E, match="FLOP count overflows"):
        ta.resolve_shapes([1, U], [U, 1], [U, 1, 1])
    with pytest.raises(E, match="rank 1 not supported"):
        ta.resolve_shapes([4], [4, 4], [4, 4])


def test_u32_addressing_limits(ta):
    ta.resolve_shapes([65536, 65536], [65536, 1], [65536, 1])
    ta.resolve_shapes([2, 32768, 65536], [65536, 1], [2, 32768, 1])
    cases = [("A", [65537, 65536], [65536, 1], [65537, 1]),
             ("B", [1, 65537], [65537, 65536], [1, 65536]),
             ("C", [65537, 1], [1, 65536], [65537, 65536]),
             ("A", [3, 32768, 65536], [65536, 1], [3, 32768, 1]),
             ("B", [3, 1, 32768], [3, 32768, 65536], [3, 1, 65536]),
             ("C", [3, 32768, 1], [1, 65536], [3, 32768, 65536])]
    for label, a, b, c in cases:
        with pytest.raises(ta.TensorAshError) as e:
            ta.resolve_shapes(a, b, c)
        assert label in str(e.value) and "shader u32 indexing" in str(e.value)


# src/pipeline/catalog.rs:384-493 (registry order, aliases, parse)
def test_registry_and_aliases(ta):
    specs = ta.kernel_specs()
    names = [n for n, _ in specs]
    assert len(names) == len(set(names)) >= 12
    assert ("tf32x3_m128n256", (128, 256, 16)) in specs
    assert ta.kernel_selection_parse("") is None and ta.kernel_selection_parse(" AUTO ") is None
    for name in names:                      # every registry name resolves to itself
        assert names[ta.kernel_selection_parse(name)] == name
    # every ML_KERNEL spelling of the reference keeps resolving (to the CUDA variant that supersedes it)
    ref_aliases = ("large small m64n128 m128n64 m128n64k64 m64n32 k64 bk16 v2 m64n128k64 m128n128_t4 "
                   "m256n64 v3 large_bda m128n64k64_bda k64_bda small_bda m64n32_bda m128n64_bda "
                   "m64n128_bda large_bda_v4 m128n64k64_bda_v4 small_bda_v4 k64_bda_v4 m128n64_bda_v4 "
                   "m64n128_bda_v4 bk16_bda_v4 large_bda_v4_aligned m128n64k64_bda_v4_aligned row_bda "
                   "col_bda outer_bda f16w_large_bda_v4 f16w_small_bda_v4 f16w_k64_bda_v4 "
                   "f16w_m128n64k64_bda_v4 f16w_row_bda f16w_row_bda_k16 f16w_row_bda_k16_v2 "
                   "f16w_row_bda_k16_packed f16w_row_bda_k16_v2_packed f16w_coopmat_aligned coopmat "
                   "f16w_cm2 cm2 128 64 wide tall sota 64k").split()
    for alias in ref_aliases:
        assert ta.kernel_selection_parse(alias) is not None, alias
    assert names[ta.kernel_selection_parse("f16w_row_bda_k16_packed")] == "f16w_row_bda_k16_packed"
    with pytest.raises(ta.TensorAshError, match="invalid ML_KERNEL 'warp9'"):
        ta.kernel_selection_parse("warp9")


def test_split_heuristics_match_oracle(ta, orc):
    rng = orc.LcgRng(99)
    for _ in range(300):
        b, m, n = rng.range_u32(1, 6), rng.range_u32(1, 700), rng.range_u32(1, 700)
        k = rng.range_u32(1, 20000)
        assert ta.heuristic_splits(b, m, n, k) == orc.heuristic_splits(b, m, n, k)
        for tile in (64, 128):
            assert ta.default_num_k_splits(b, m, n, k, tile, tile) == \
                orc.default_num_k_splits(b, m, n, k, tile, tile)
    assert ta.heuristic_splits(1, 37, 41, 1088) == 16            # tests/correctness/splitk2.rs:63-70
    U = 2 ** 32 - 1
    assert ta.default_num_k_splits(U, U, U, U, 1, 1) == 1        # src/executor/splitk2.rs:506-512


def test_f16_conversion_bit_exact_vs_oracle(ta, orc):
    xs = np.concatenate([orc.fill_det(4000, 9) * s for s in (1e-9, 6e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 1 + 2.0 ** -11],
                                      np.float32)])
    for v in xs[::7]:
        assert ta.f32_to_f16_bits(float(v)) == orc.f32_to_f16_bits(v)
    for bits in list(range(0, 0x7C00, 37)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0x8001]:
        assert np.float32(ta.f16_bits_to_f32(bits)).tobytes() == np.float32(orc.f16_bits_to_f32(bits)).tobytes()
    assert np.isnan(ta.f16_bits_to_f32(ta.f32_to_f16_bits(float("nan"))))


def test_f16_decode_is_ieee_on_every_pattern(ta, orc):
    """All 65536 halves against numpy's binary16.  The reference's host decode (src/dtype.rs:93-99)
    is wrong on subnormal halves and only there; the library decodes them as the device does."""
    bits = np.arange(0x10000, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([ta.f16_bits_to_f32(int(b)) for b in bits], dtype=np.float32)
    port = np.array([orc.f16_bits_to_f32(int(b)) for b in bits], dtype=np.float32)
    ref = np.array([orc.f16_bits_to_f32_reference(int(b)) for b in bits], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.array_equal(port[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.isnan(got[~finite]).all() and np.isnan(port[~finite]).all()
    subnormal = ((bits & 0x7C00) == 0) & ((bits & 0x03FF) != 0)
    differs = ref.view(np.uint32) != want.view(np.uint32)
    assert np.array_equal(differs & finite, subnormal)
    # encode(decode(h)) == h for every non-NaN half
    back = np.array([ta.f32_to_f16_bits(float(v)) for v in want[finite]], dtype=np.uint16)
    assert np.array_equal(back, bits[finite])


def test_pack_and_tile_rule(ta, orc):
    src = np.arange(16, dtype=np.float32)
    assert ta.pack_f16w_row_tiles(src, 4, 4, 2).tolist() == \
        [0, 1, 4, 5, 8, 9, 12, 13, 2, 3, 6, 7, 10, 11, 14, 15]
    w = orc.fill_det(96 * 128, 3)
    assert (ta.pack_f16w_row_tiles(w, 96, 128, 32) == orc.pack_f16w_row_tiles(w, 96, 128, 32)).all()
    with pytest.raises(ta.TensorAshError, match="not a multiple of tile_n"):
        ta.pack_f16w_row_tiles(src, 4, 4, 3)
    for k, n in [(4096, 11008), (11008, 4096), (2048, 5632), (2048, 32000), (2048, 2048), (2048, 256),
                 (1024, 4000), (5632, 2048)]:
        assert ta.f16w_row_tile_n(k, n) == orc.f16w_row_tile_n(k, n)


def test_attn_decode_chunk_rule(ta):
    # src/executor/elementwise/mod.rs:235-237: clamp(ceil(kv_len / 32), 8, 32)
    f = ta.lib().ta_attn_decode_num_chunks
    assert [f(v) for v in (1, 256, 257, 640, 1024, 5000)] == [8, 8, 9, 20, 32, 32]


def test_c_smoke_source_compiles_against_the_header(tmp_path, ta):
    """A C program written against the reference header (examples/c_smoke.c uses
    exactly these calls) compiles and links against this library."""
    from tensor_ash_b200 import capi
    import subprocess
    src = tmp_path / "probe.c"
    src.write_text('#include "tensor_ash.h"\n#include <stdio.h>\n'
                   'int main(void){ ta_run_stats s = {0}; ta_matmul_op op = {0}; ta_copy_desc d = {0};\n'
                   ' (void)s; (void)op; (void)d; printf("%s\\n", ta_version());\n'
                   ' return ta_matmul(NULL, NULL, NULL, NULL, 1.0f, 0, &s) == -1 ? 0 : 1; }\n')
    exe = tmp_path / "probe"
    libdir = os.path.dirname(capi.lib_path())
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                    "-o", str(exe), "-L", libdir, "-ltensor_ash", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
    assert out.stdout.strip() == "2.0.0"


def test_heuristic_kernel_routing_table(ta):
    """Heuristic stage of explicit > tuned > heuristic (src/pipeline/mod.rs:259-360), on a 148-SM device:
    aligned f32 problems of 64 rows or more use the tensor-core tiles (the narrow tile when the wide one
    would leave SMs idle), 33..63 rows only over a large weight matrix, everything else the SIMT tiles;
    f16-storage weights use the row GEMV to 8 rows and the f16 tensor-core tiles from 32 rows."""
    hk = ta.heuristic_kernel
    assert hk(32, 2048, 2048, 2048) == "tf32x3_m128n256"          # the benchmark configuration
    assert hk(1, 1024, 1024, 1024) == "tf32x3_m128n128"           # 32 wide tiles would idle 116 SMs
    assert hk(1, 512, 128, 512) == "tf32x3_m128n128"              # narrow N
    assert hk(1, 64, 4096, 4096) == "tf32x3_m128n128"
    assert hk(1, 48, 4096, 4096) == "tf32x3_m128n128"             # 33..63 rows over 2^24 weights
    assert hk(1, 48, 256, 256) == "ffma_m64n64"                   # 33..63 rows over small weights
    assert hk(1, 32, 4096, 4096) == "ffma_m64n64"                 # the rows kernel lives in this family
    assert hk(1, 1023, 1025, 1027) == "ffma_m128n128"             # unaligned: no TMA
    assert hk(1, 100, 100, 100) == "tf32x3_m128n128"              # aligned and 64 or more each way
    assert hk(1, 50, 50, 50) == "ffma_m64n64"
    assert hk(1, 1, 11008, 4096, True).startswith("f16w_row_bda_k16")
    assert hk(1, 8, 4096, 11008, True).startswith("f16w_row_bda_k16")
    assert hk(1, 512, 2048, 2048, True).startswith("f16w_umma_m128n")
    assert hk(1, 16, 2048, 2048, True) == "f16w_ffma_m64n64"
    assert hk(1, 512, 2047, 2048, True) == "f16w_ffma_m128n128"   # N not a multiple of 8
    names = {name for name, _tile in ta.kernel_specs()}
    for shape in [(1, 7, 9, 11), (4, 300, 300, 300), (1, 4096, 4096, 4096)]:
        assert hk(*shape) in names and hk(*shape, True) in names
