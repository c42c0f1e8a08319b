"""Pins the CPU oracle against every known-answer vector the reference's own
host-side tests hold for this path, and against tests/golden/golden.json (an
independent pure-Python restatement of the fixture definitions)."""
import json
import math
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "golden.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


# ---- tools/test-support/src/lib.rs:168-290
def test_fill_det_deterministic_in_range_and_seeded(orc):
    a, b = orc.fill_det(8, 42), orc.fill_det(8, 42)
    assert (a == b).all()
    buf = orc.fill_det(1024, 7)
    assert ((buf >= -1.0) & (buf < 1.0)).all()
    assert not (orc.fill_det(16, 1) == orc.fill_det(16, 2)).all()


def test_fill_det_matches_independent_golden(orc, golden):
    for seed, vals in golden["fill_det"].items():
        got = orc.fill_det(len(vals), int(seed))
        assert got.tolist() == [np.float32(v) for v in vals]


def test_lcg_range(orc, golden):
    rng = orc.LcgRng(0xCAFE)
    assert all(7 <= rng.range_u32(7, 13) <= 13 for _ in range(1000))
    rng = orc.LcgRng(1)
    assert all(rng.range_u32(42, 42) == 42 for _ in range(16))
    rng = orc.LcgRng(0xC0FFEE)
    want = golden["lcg_range"]["0xC0FFEE:1:300"]
    assert [rng.range_u32(1, 300) for _ in want] == want


def test_cpu_bmm_hand_computed(orc):
    a = np.array([1, 2, 3, 4], np.float32)
    b = np.array([5, 6, 7, 8], np.float32)
    assert orc.cpu_bmm(a, b, 1, 2, 2, 2).tolist() == [19.0, 22.0, 43.0, 50.0]
    c0 = np.full(4, 100.0, np.float32)
    assert orc.cpu_bmm(a, b, 1, 2, 2, 2, c_init=c0, accumulate=True).tolist() == [119.0, 122.0, 143.0, 150.0]
    assert orc.cpu_bmm(a, b, 1, 2, 2, 2, alpha=0.5).tolist() == [9.5, 11.0, 21.5, 25.0]


def test_cpu_bmm_broadcasts(orc):
    eye = np.array([1, 0, 0, 1], np.float32)
    two = np.array([1, 2, 3, 4, 10, 20, 30, 40], np.float32)
    assert orc.cpu_bmm(eye, two, 2, 2, 2, 2).tolist() == two.tolist()   # A broadcast
    assert orc.cpu_bmm(two, eye, 2, 2, 2, 2).tolist() == two.tolist()   # B broadcast


def test_cpu_bmm_thread_count_does_not_change_bits(orc):
    a, b = orc.fill_det(37 * 53, 5), orc.fill_det(53 * 41, 6)
    one = orc.cpu_bmm(a, b, 1, 37, 41, 53, threads=1)
    many = orc.cpu_bmm(a, b, 1, 37, 41, 53, threads=0)
    assert (one == many).all()


def test_max_abs_err_and_tolerance(orc):
    e, idx = orc.max_abs_err([1.0, float("nan")], [1.0, 2.0])
    assert math.isinf(e) and idx == 1
    e, idx = orc.max_abs_err([1.0, 3.0, -5.0], [1.5, 1.0, -4.0])
    assert (e, idx) == (2.0, 1)
    with pytest.raises(AssertionError, match="slice lengths differ"):
        orc.max_abs_err([1.0], [1.0, 2.0])
    assert orc.tolerance(200) > orc.tolerance(100) and orc.tolerance(0) == 0.0
    assert orc.tolerance(1024) == pytest.approx(8 * 1024 * 2.0 ** -23)


# ---- src/dtype.rs:118-163
def test_f16_exact_roundtrip(orc):
    for v in [0.0, -0.0, 1.0, -1.0, 0.5, 2.0, 65504.0, -65504.0, 0.25, 1024.0]:
        r = orc.round_via_f16(v)
        assert np.float32(r).tobytes() == np.float32(v).tobytes()


def test_f16_known_encodings(orc):
    enc = orc.f32_to_f16_bits
    assert enc(1.0) == 0x3C00 and enc(-2.0) == 0xC000 and enc(65504.0) == 0x7BFF
    assert enc(float("inf")) == 0x7C00 and enc(65520.0) == 0x7C00
    assert enc(6.104e-5) == 0x0400 and enc(5.96e-8) == 0x0001 and enc(1e-10) == 0x0000
    assert math.isnan(orc.f16_bits_to_f32(enc(float("nan"))))


def test_f16_round_to_nearest_even(orc):
    assert orc.round_via_f16(np.float32(1.0 + 2.0 ** -11)) == 1.0
    assert orc.round_via_f16(np.float32(1.0 + 3 * 2.0 ** -11)) == np.float32(1.0 + 2.0 ** -9)
    v = np.float32(0.001)
    while v < 60000.0:
        assert abs((orc.round_via_f16(v) - v) / v) <= 2.0 ** -11
        v = np.float32(v * 1.37)


def test_f16_matches_numpy_half_everywhere(orc):
    # numpy's float16 cast is IEEE RNE too: an independent check over all exponents
    x = np.concatenate([orc.fill_det(20000, 3) * s for s in (1e-8, 1e-6, 1e-4, 1e-2, 1.0, 100.0, 7e4)])
    assert (orc.f32_to_f16_array(x) == x.astype(np.float16).view(np.uint16)).all()


# ---- src/matmul/api.rs:359-379
def test_pack_layout_golden(orc):
    src = np.arange(16, dtype=np.float32)
    want = [0, 1, 4, 5, 8, 9, 12, 13, 2, 3, 6, 7, 10, 11, 14, 15]
    assert orc.pack_f16w_row_tiles(src, 4, 4, 2).tolist() == want


# ---- src/pipeline/routing.rs:10-41 and its tests
def test_f16w_row_tile_rule(orc):
    assert orc.f16w_row_tile_n(4096, 11008) == 32     # deep K -> k16
    assert orc.f16w_row_tile_n(11008, 4096) == 32
    assert orc.f16w_row_tile_n(2048, 5632) == 64      # gate/up shaped
    assert orc.f16w_row_tile_n(2048, 32000) == 64     # lm_head
    assert orc.f16w_row_tile_n(2048, 2048) == 32
    assert orc.f16w_row_tile_n(2048, 256) == 32
    assert orc.f16w_row_tile_n(1024, 4000) == 32      # N % 64 != 0


# ---- src/executor/splitk2.rs:479-555
def test_default_num_k_splits(orc):
    d = orc.default_num_k_splits
    assert d(1, 256, 256, 4096, 128, 128) == 16
    assert d(1, 64, 64, 8192, 64, 64) == 64
    assert d(1, 512, 512, 4096, 128, 128) == 4
    assert d(1, 64, 64, 64, 64, 64) == 2
    assert d(1, 128, 128, 1024, 0, 128) == 1
    m = 2 ** 32 - 1
    assert d(m, m, m, m, 1, 1) == 1


def test_heuristic_splits_table(orc):
    cases = [((1, 64, 64, 1024), 16), ((1, 64, 64, 2048), 32), ((1, 64, 128, 8192), 64),
             ((4, 64, 64, 4096), 32), ((1, 128, 128, 1024), 16), ((1, 256, 256, 1024), None),
             ((1, 256, 256, 2048), 16), ((1, 512, 512, 2048), None), ((1, 512, 512, 4096), 4),
             ((1, 512, 512, 8192), 8), ((1, 1024, 1024, 8192), None), ((1, 1, 4096, 8192), None),
             ((0, 64, 64, 1024), None)]
    for args, want in cases:
        assert orc.heuristic_splits(*args) == want, args
    # tests/correctness/splitk2.rs:63-70: (37, 41, 1088) routes to 16 splits
    assert orc.heuristic_splits(1, 37, 41, 1088) == 16


def test_splitk_partition_covers_k_once(orc):
    for k, s in [(65536, 64), (1088, 16), (1000, 7), (5, 5)]:
        edges = [orc.splitk_bounds(k, s, i) for i in range(s)]
        assert edges[0][0] == 0 and edges[-1][1] == k
        assert all(edges[i][1] == edges[i + 1][0] for i in range(s - 1))
        sizes = [hi - lo for lo, hi in edges]
        assert max(sizes) - min(sizes) <= 1


# ---- examples/c_smoke.c:44-104
def test_c_smoke_values(orc):
    a = np.array([1, 2, 3, 4, 5, 6], np.float32)
    b = np.array([7, 8, 9, 10, 11, 12], np.float32)
    c = orc.cpu_bmm(a, b, 1, 2, 2, 3)
    assert c.tolist() == [58.0, 64.0, 139.0, 154.0]
    out = orc.cpu_epilogue(c.copy(), 1, 2, 2, bias=np.array([-58.5, 0.0], np.float32), act="silu")
    assert out[0] == pytest.approx(-0.5 / (1 + math.exp(0.5)), abs=1e-6)
    assert out[1] == pytest.approx(64.0, abs=1e-4)


# ---- epilogue + GEMM against the independent numpy golden
def test_gemm_epilogue_matches_independent_golden(orc, golden):
    for g in golden["gemm"]:
        c = g["case"]
        batch, m, n, k = c["batch"], c["m"], c["n"], c["k"]
        a = orc.fill_det(batch * m * k, c["seeds"][0])
        b = orc.fill_det((1 if c["b_shared"] else batch) * k * n, c["seeds"][1])
        out = orc.cpu_bmm(a, b, batch, m, n, k, alpha=c["alpha"])
        bias = None
        if c["bias_kind"] == "n":
            bias = orc.fill_det(n, c["seeds"][2])
        elif c["bias_kind"] == "bn":
            bias = orc.fill_det(batch * n, c["seeds"][2])
        d = orc.fill_det(batch * m * n, c["seeds"][3]) if c["binary"] != "none" else None
        out = orc.cpu_epilogue(out, batch, m, n, bias=bias, act=c["act"], binary=c["binary"], d=d,
                               beta=c["beta"])
        want = np.array(g["values"], np.float32)
        got = out[g["indices"]]
        # numpy's matmul sums in another order than the oracle's ascending-k f64 chain:
        # equal to within one f32 ulp of the f64 result
        assert np.abs(got - want).max() <= 2e-6 * max(1.0, np.abs(want).max())
        assert float(np.sum(out.astype(np.float64))) == pytest.approx(g["checksum"], rel=1e-6, abs=1e-4)


def test_activation_formulas(orc):
    assert orc.activate(-1.5, "relu") == 0.0 and orc.activate(2.0, "relu") == 2.0
    assert orc.activate(0.7, "silu") == pytest.approx(0.7 / (1 + math.exp(-0.7)))
    x = 0.9
    assert orc.activate(x, "gelu") == pytest.approx(
        0.5 * x * (1 + math.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3))))


def test_splitk2_emulation_is_close_to_f64(orc):
    m, n, k = 16, 24, 2048
    a, b = orc.fill_det(m * k, 41), orc.fill_det(k * n, 42)
    ref = orc.cpu_bmm(a, b, 1, m, n, k)
    for s in (4, 16, 64):
        got = orc.splitk2_f32(a, b, m, n, k, s)
        assert orc.max_abs_err(got, ref)[0] <= 2 * orc.tolerance(k)


def test_model_op_references(orc):
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    w = np.array([1.0, 0.5, 2.0], np.float32)
    out = orc.cpu_rmsnorm(x, w, 1e-5)
    for r in range(2):
        inv = 1.0 / math.sqrt(float((x[r] ** 2).sum()) / 3 + 1e-5)
        assert np.allclose(out[r], x[r] * w * inv, atol=1e-6)
    sm = orc.cpu_softmax_rows(x, 1.0, 1, 2, 0)
    assert (sm[:, 2] == 0.0).all() and np.allclose(sm[:, :2].sum(axis=1), 1.0)
    assert orc.cpu_argmax(np.array([1, 5, 5, 2], np.float32)) == 2   # largest index wins ties
