"""GPU parity tests for the GEMM path: the CUDA kernels, called through the C
ABI, against the CPU oracle on the same seeded inputs.  Cases, seeds and
tolerances follow the reference's integration tests (file:line per test).

Tolerances (both must hold for FP32 routes):
  * the reference's own bound, absolute: tolerance(k) = 8*k*eps
    (tools/test-support/src/lib.rs:157-162), 2*tol + 1e-4 with a transcendental
    epilogue (tests/correctness/epilogue.rs:52-54), 2*tol for split-K
    (tests/correctness/splitk2.rs:50);
  * the relative target of this build: max|err| <= 1e-5 * max(1, max|ref|).
"""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def rel_err(got, ref):
    got = np.asarray(got, np.float32).reshape(-1)
    ref = np.asarray(ref, np.float32).reshape(-1)
    assert np.isfinite(got).all(), "non-finite output"
    return float(np.abs(got - ref).max() / max(1.0, float(np.abs(ref).max())))


def check(orc, got, ref, abs_tol, label):
    e, idx = orc.max_abs_err(got, ref)
    assert e <= abs_tol, f"{label}: abs err {e:.3e} > {abs_tol:.3e} at {idx}"
    r = rel_err(got, ref)
    assert r <= REL_TOL, f"{label}: rel err {r:.3e} > {REL_TOL}"


@pytest.fixture(scope="module", params=["auto", "ffma", "tf32x3", "tf32x3_m128n128", "tf32x3_m256n256", "small"])
def setup(request, ta):
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 16, request.param, tune=False)
    yield ta, ctx, ex, request.param
    ex.close()
    ctx.close()


def shape3(batch, r, c):
    return (r, c) if batch == 1 else (batch, r, c)


def run_one(ta, ctx, ex, orc, batch, m, n, k, alpha, accumulate, seed_a, seed_b, init_c=None):
    """tests/common/mod.rs:154-213"""
    a, ha = upload_det(ta, ctx, ex, orc, shape3(batch, m, k), seed_a)
    b, hb = upload_det(ta, ctx, ex, orc, shape3(batch, k, n), seed_b)
    c = ta.Tensor.uninit_device(ctx, shape3(batch, m, n))
    if init_c is not None:
        ex.upload(init_c, c)
    ex.run_matmuls([ta.MatmulCall(a, b, c, alpha, accumulate)])
    got = ex.download(c).reshape(-1)
    ref = orc.cpu_bmm(ha, hb, batch, m, n, k, alpha=alpha, c_init=init_c, accumulate=accumulate)
    return got, ref


# tests/correctness/shapes.rs:7-47
SWEEP = [(1, 1, 1), (1, 16, 16), (16, 1, 16), (16, 16, 1), (8, 7, 5), (17, 19, 23), (31, 33, 47),
         (65, 67, 15), (65, 67, 16), (65, 67, 17), (65, 67, 31), (65, 67, 32), (65, 67, 33),
         (65, 67, 63), (65, 67, 65), (64, 64, 64), (128, 128, 128), (129, 130, 131), (256, 256, 256),
         (200, 300, 100)]


def test_shape_sweep_rank2(setup, orc):
    ta, ctx, ex, _ = setup
    for m, n, k in SWEEP:
        got, ref = run_one(ta, ctx, ex, orc, 1, m, n, k, 1.0, False, 11, 13)
        check(orc, got, ref, orc.tolerance(k), f"rank2 M={m} N={n} K={k}")


# TMA-eligible edge residues: every combination of partial M / N / K tiles
def test_edge_residues_of_the_tensor_core_tiles(setup, orc):
    ta, ctx, ex, _ = setup
    for m in (64, 127, 129, 200):
        for n in (64, 132, 260, 508):
            for k in (64, 68, 100, 144):
                got, ref = run_one(ta, ctx, ex, orc, 1, m, n, k, 1.0, False, 21, 23)
                check(orc, got, ref, orc.tolerance(k), f"edge M={m} N={n} K={k}")


# tests/correctness/property.rs:5-63
def test_property_random_shapes(setup, orc):
    ta, ctx, ex, _ = setup
    rng = orc.LcgRng(0xC0FFEE)
    for trial in range(32):
        batch, m, n, k = rng.range_u32(1, 4), rng.range_u32(1, 320), rng.range_u32(1, 320), rng.range_u32(1, 320)
        got, ref = run_one(ta, ctx, ex, orc, batch, m, n, k, 1.0, False, 1000 + trial, 2000 + trial)
        check(orc, got, ref, orc.tolerance(k), f"trial {trial}: B={batch} M={m} N={n} K={k}")


# tests/correctness/batch.rs: broadcast of either input, alpha, accumulate
def test_batched_broadcast_alpha_accumulate(setup, orc):
    ta, ctx, ex, _ = setup
    batch, m, n, k = 5, 96, 136, 72
    ha, hb = orc.fill_det(batch * m * k, 31), orc.fill_det(k * n, 32)
    hc0 = orc.fill_det(batch * m * n, 33)
    a = ta.Tensor.uninit_device(ctx, (batch, m, k))
    b = ta.Tensor.uninit_device(ctx, (k, n))
    c = ta.Tensor.uninit_device(ctx, (batch, m, n))
    for t, h in ((a, ha), (b, hb), (c, hc0)):
        ex.upload(h, t)
    ex.run_matmuls([ta.MatmulCall(a, b, c, 0.5, True)])
    ref = orc.cpu_bmm(ha, hb, batch, m, n, k, alpha=0.5, c_init=hc0, accumulate=True)
    check(orc, ex.download(c), ref, orc.tolerance(k), "B broadcast + alpha + accumulate")
    # A broadcast
    a1 = ta.Tensor.uninit_device(ctx, (m, k))
    bb = ta.Tensor.uninit_device(ctx, (batch, k, n))
    ha1, hbb = orc.fill_det(m * k, 34), orc.fill_det(batch * k * n, 35)
    ex.upload(ha1, a1)
    ex.upload(hbb, bb)
    ex.run_matmuls([ta.MatmulCall(a1, bb, c)])
    check(orc, ex.download(c), orc.cpu_bmm(ha1, hbb, batch, m, n, k), orc.tolerance(k), "A broadcast")


def epi_tol(orc, k):
    return 2.0 * orc.tolerance(k) + 1e-4


# tests/correctness/epilogue.rs:56-134
def run_epilogue_case(setup, orc, shape, alpha, accumulate, bias, act, binary):
    ta, ctx, ex, _ = setup
    m, n, k = shape
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 71)
    b, hb = upload_det(ta, ctx, ex, orc, (k, n), 72)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    hc0 = None
    if accumulate:
        hc0 = orc.fill_det(m * n, 73)
        ex.upload(hc0, c)
    bias_t = hbias = None
    if bias:
        bias_t, hbias = upload_det(ta, ctx, ex, orc, (n,), 74)
    d_t = hd = None
    kind, beta = ta.Binary.NONE, 0.0
    if binary is not None:
        d_t, hd = upload_det(ta, ctx, ex, orc, (m, n), 75)
        beta, is_mul = binary
        kind = ta.Binary.MUL if is_mul else ta.Binary.ADD_SCALED
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c, alpha, accumulate),
                            ta.Epilogue(bias_t, act, kind, d_t, beta))])
    got = ex.download(c)
    ref = orc.cpu_bmm(ha, hb, 1, m, n, k, alpha=alpha, c_init=hc0, accumulate=accumulate)
    ref = orc.cpu_epilogue(ref, 1, m, n, bias=hbias, act=int(act), binary=int(kind), d=hd, beta=beta)
    check(orc, got, ref, epi_tol(orc, k), f"epilogue {shape} alpha={alpha} acc={accumulate} bias={bias} "
                                          f"act={act!r} binary={binary}")


def test_epilogue_cases(setup, orc):
    ta = setup[0]
    A = ta.Activation
    cases = [  # tests/correctness/epilogue.rs:138-232
        ((512, 512, 512), 1.0, False, True, A.NONE, None),
        ((512, 512, 512), 1.0, False, True, A.RELU, None),
        ((256, 1024, 512), 1.0, False, False, A.SILU, (0.0, True)),
        ((512, 512, 256), 1.0, False, True, A.GELU, (0.75, False)),
        ((256, 256, 256), 0.5, True, True, A.SILU, None),
        ((255, 257, 263), 1.0, False, True, A.RELU, None),
        ((123, 517, 129), 1.0, False, False, A.SILU, (0.0, True)),
        ((1023, 129, 511), 2.0, False, True, A.NONE, (-1.5, False)),
        ((252, 260, 264), 1.0, False, True, A.GELU, (0.5, False)),   # TMA-eligible partial tiles
    ]
    for c in cases:
        run_epilogue_case(setup, orc, *c)


# tests/correctness/epilogue.rs:234-278
def test_batched_bias_uses_one_row_per_batch(setup, orc):
    ta, ctx, ex, _ = setup
    for batch, m, n, k in ((3, 2, 7, 5), (3, 130, 136, 68)):
        a, ha = upload_det(ta, ctx, ex, orc, (batch, m, k), 91)
        b, hb = upload_det(ta, ctx, ex, orc, (batch, k, n), 92)
        c = ta.Tensor.uninit_device(ctx, (batch, m, n))
        bias = ta.Tensor.uninit_device(ctx, (batch, n))
        hbias = np.array([[10.0 * bi + col for col in range(n)] for bi in range(batch)], np.float32)
        ex.upload(hbias, bias)
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(bias=bias))])
        ref = orc.cpu_bmm(ha, hb, batch, m, n, k)
        ref = orc.cpu_epilogue(ref, batch, m, n, bias=hbias)
        e, _ = orc.max_abs_err(ex.download(c), ref)
        assert e <= epi_tol(orc, k) + 1e-5 * float(np.abs(ref).max())


# tests/correctness/epilogue.rs:282-322
def test_graph_hazard_on_epilogue_d_operand(setup, orc):
    ta, ctx, ex, _ = setup
    m, h, i_ = 64, 128, 256
    x, hx = upload_det(ta, ctx, ex, orc, (m, h), 81)
    w_up, hup = upload_det(ta, ctx, ex, orc, (h, i_), 82)
    w_gate, hgate = upload_det(ta, ctx, ex, orc, (h, i_), 83)
    up = ta.Tensor.uninit_device(ctx, (m, i_))
    gated = ta.Tensor.uninit_device(ctx, (m, i_))
    ex.run_op_graph([
        ta.MatmulOp(ta.MatmulCall(x, w_up, up)),
        ta.MatmulOp(ta.MatmulCall(x, w_gate, gated),
                    ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=up)),
    ])
    up_ref = orc.cpu_bmm(hx, hup, 1, m, i_, h)
    ref = orc.cpu_epilogue(orc.cpu_bmm(hx, hgate, 1, m, i_, h), 1, m, i_, act="silu", binary="mul", d=up_ref)
    check(orc, ex.download(gated), ref, epi_tol(orc, h), "swiglu graph")


# tests/correctness/epilogue.rs:324-380 and capi/src/api/ops.rs:40-57
def test_rejections(setup, orc):
    ta, ctx, ex, _ = setup
    E = ta.TensorAshError
    a = ta.Tensor.uninit_device(ctx, (64, 64))
    b = ta.Tensor.uninit_device(ctx, (64, 64))
    c = ta.Tensor.uninit_device(ctx, (64, 64))
    bad_bias = ta.Tensor.uninit_device(ctx, (63,))
    with pytest.raises(E, match="bias"):
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(bias=bad_bias))])
    bad_d = ta.Tensor.uninit_device(ctx, (64, 32))
    with pytest.raises(E, match="D shape"):
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(binary=ta.Binary.MUL, d=bad_d))])
    with pytest.raises(E, match="epilogue.d is null"):
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(binary=ta.Binary.MUL))])
    with pytest.raises(E, match="binary_kind is 0"):
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(d=c))])
    with pytest.raises(E, match="must not alias"):
        ex.run_matmuls([ta.MatmulCall(a, b, a)])
    with pytest.raises(E, match="A.K=64"):
        ex.run_matmuls([ta.MatmulCall(a, ta.Tensor.uninit_device(ctx, (32, 64)), c)])
    c16 = ta.Tensor.uninit_device_f16(ctx, (64, 64))
    with pytest.raises(E, match="C must be f32"):
        ex.run_matmuls([ta.MatmulCall(a, b, c16)])
    with pytest.raises(E, match="exceeds max_calls_per_submit"):
        ex.run_matmuls([ta.MatmulCall(a, b, c)] * 17)
    other = ta.Context(False, "index:0")
    foreign = ta.Tensor.uninit_device(other, (64, 64))
    with pytest.raises(E, match="a belongs to a different"):
        ex.run_matmuls([ta.MatmulCall(foreign, b, c)])
    with pytest.raises(E, match="bytes > tensor capacity"):
        ex.upload(np.zeros(64 * 64 + 1, np.float32), a)
    ex.upload(np.zeros(10, np.float32), a)          # shorter than capacity is fine
    assert ex.download(a, 10).shape == (10,)


def test_f16_weight_storage(setup, orc):
    """tests/correctness/f16.rs:21-108: B stored as f16; the reference rounds B
    through f16 so that products are exact in f32."""
    ta, ctx, ex, _ = setup
    for m, n, k in ((2, 2, 3), (96, 200, 136), (130, 68, 72)):
        a, ha = upload_det(ta, ctx, ex, orc, (m, k), 51)
        hb = orc.fill_det(k * n, 52)
        b16 = ta.Tensor.uninit_device_f16(ctx, (k, n))
        assert b16.is_f16 and b16.size_bytes() == (k * n * 2 + 15) // 16 * 16
        ex.upload(hb, b16)
        assert (ex.download(b16).reshape(-1) == orc.round_via_f16(hb)).all()   # upload/download RNE round trip
        c = ta.Tensor.uninit_device(ctx, (m, n))
        ex.run_matmuls([ta.MatmulCall(a, b16, c)])
        ref = orc.cpu_bmm(ha, orc.round_via_f16(hb), 1, m, n, k)
        if ex.dispatch_info_for(1, m, n, k, b_f16=True).kernel.startswith("f16w_umma"):
            # tensor-core route: A is rounded to f16 on the way in, the f16-weight tolerance applies
            assert rel_err(ex.download(c), ref) <= 2e-3, f"f16w {m}x{n}x{k}"
        else:
            check(orc, ex.download(c), ref, orc.tolerance(k), f"f16w {m}x{n}x{k}")


def test_stats_and_dispatch_info(setup, orc):
    ta, ctx, ex, sel = setup
    a, _ = upload_det(ta, ctx, ex, orc, (256, 256), 1)
    b, _ = upload_det(ta, ctx, ex, orc, (256, 256), 2)
    c = ta.Tensor.uninit_device(ctx, (256, 256))
    before = ta.kernel_launch_count()
    st = ex.run_matmuls([ta.MatmulCall(a, b, c)])
    assert ta.kernel_launch_count() == before + 1
    assert st.n_calls == 1 and st.total_flops == 2 * 256 ** 3 and st.gpu_time_ns and st.tflops() > 0
    info = ex.dispatch_info_for(1, 256, 256, 256)
    names = [n for n, _ in ta.kernel_specs()]
    assert info.kernel in names and info.split_k2 is None
    if sel == "auto":
        assert info.kernel.startswith("tf32x3")
        assert ex.dispatch_info_for(1, 2, 2, 3).kernel == "ffma_m64n64"
        assert ex.dispatch_info_for(1, 255, 257, 263).kernel.startswith("ffma")
        # tests/correctness/splitk2.rs:63-70, 95-97
        r = ex.dispatch_info_for(1, 37, 41, 1088)
        assert r.split_k2 == 16 and r.kernel.startswith("split_k2_")
        dp = ex.dispatch_info_for(1, 37, 41, 1000)
        assert dp.split_k2 is None and not dp.kernel.startswith("split_k2_")


@pytest.mark.gpu
def test_prepared_handle_may_outlive_its_executor_for_destruction(setup, orc):
    """Handles are destroyed in any order: closing the executor first must leave the prepared
    object destroyable and no CUDA error behind for the next launch to trip over."""
    ta, ctx, ex, sel = setup
    ex2 = ta.Executor(ctx, 2, 4, sel, tune=False)
    a, _ = upload_det(ta, ctx, ex, orc, (64, 64), 71)
    b, _ = upload_det(ta, ctx, ex, orc, (64, 64), 72)
    c = ta.Tensor.uninit_device(ctx, (64, 64))
    prep = ex2.prepare_ops([ta.MatmulOp(ta.MatmulCall(a, b, c))])
    prep.run()
    want = ex.download(c)
    ex2.close()
    prep.close()
    ex.upload(np.zeros(64 * 64, np.float32), c)
    ex.run_matmuls([ta.MatmulCall(a, b, c)])      # would report a stale error if one was left
    assert (ex.download(c) == want).all()


# tests/correctness/replay.rs:13-21, prepared.rs
def test_prepared_replay_is_bitwise_equal_to_direct(setup, orc):
    ta, ctx, ex, _ = setup
    m, n, k = 192, 264, 136
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 61)
    b, hb = upload_det(ta, ctx, ex, orc, (k, n), 62)
    bias, hbias = upload_det(ta, ctx, ex, orc, (n,), 63)
    c1 = ta.Tensor.uninit_device(ctx, (m, n))
    c2 = ta.Tensor.uninit_device(ctx, (m, n))
    ep = ta.Epilogue(bias=bias, activation=ta.Activation.GELU)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c1), ep)])
    prep = ex.prepare_ops([ta.MatmulOp(ta.MatmulCall(a, b, c2), ep)])
    st = prep.run()
    assert st.gpu_time_ns and st.n_calls == 1
    direct = ex.download(c1)
    assert (ex.download(c2) == direct).all()
    ex.upload(np.zeros(m * n, np.float32), c2)
    prep.submit()
    with pytest.raises(ta.TensorAshError, match="already in flight"):
        prep.submit()
    prep.wait()
    with pytest.raises(ta.TensorAshError, match="nothing in flight"):
        prep.wait()
    assert (ex.download(c2) == direct).all()
    prep.close()


def test_config1_gelu_1024(setup, orc):
    """Single FP32 GEMM C = gelu(A@B + bias), M=N=K=1024, uniform[-1,1) from the
    documented LCG (streams 0, 1, 2), rel tol 1e-5."""
    ta, ctx, ex, _ = setup
    n = 1024
    a, ha = upload_det(ta, ctx, ex, orc, (n, n), 0)
    b, hb = upload_det(ta, ctx, ex, orc, (n, n), 1)
    bias, hbias = upload_det(ta, ctx, ex, orc, (n,), 2)
    c = ta.Tensor.uninit_device(ctx, (n, n))
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c), ta.Epilogue(bias=bias, activation=ta.Activation.GELU))])
    ref = orc.cpu_epilogue(orc.cpu_bmm(ha, hb, 1, n, n, n), 1, n, n, bias=hbias, act="gelu")
    check(orc, ex.download(c), ref, epi_tol(orc, n), "config 1")


def test_few_tile_ops_split_along_k(setup, orc):
    """Ops whose output tiles cover under half of the SMs run as K ranges over the idle SMs plus a
    reduce that applies the epilogue (3xTF32 routes; the other routes run the same cases in one
    launch): every epilogue stage, alpha, accumulate, an in-place residual, a batch with per-batch
    bias.  Twice: the planes live in slot scratch that the second run reuses."""
    ta, ctx, ex, _ = setup
    A = ta.Activation
    for case in (((512, 512, 4096), 0.5, True, True, A.SILU, (0.75, False)),     # 16 planes
                 ((1024, 512, 1024), 1.0, False, True, A.RELU, (0.0, True)),
                 ((640, 384, 2320), 2.0, False, False, A.NONE, None)):            # partial tiles, a shorter last K range
        run_epilogue_case(setup, orc, *case)
        run_epilogue_case(setup, orc, *case)
    batch, m, n, k = 2, 512, 1024, 1024
    sig = 1.0 / np.sqrt(k)
    ha, hb = orc.fill_normal((batch, m, k), 20, sig), orc.fill_normal((k, n), 21, sig)
    hbias, hr = orc.fill_normal((batch, n), 22, sig), orc.fill_normal((batch, m, n), 23, sig)
    a, b = ta.Tensor.uninit_device(ctx, (batch, m, k)), ta.Tensor.uninit_device(ctx, (k, n))
    bias, c = ta.Tensor.uninit_device(ctx, (batch, n)), ta.Tensor.uninit_device(ctx, (batch, m, n))
    for t, h in ((a, ha), (b, hb), (bias, hbias), (c, hr)):
        ex.upload(h, t)
    # the residual is C itself (read by the epilogue, then overwritten)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c),
                            ta.Epilogue(bias, A.GELU, ta.Binary.ADD_SCALED, c, 1.0))])
    ref = orc.cpu_bmm(ha, hb, batch, m, n, k)
    ref = orc.cpu_epilogue(ref, batch, m, n, bias=hbias, act="gelu", binary="add_scaled", d=hr, beta=1.0)
    check(orc, ex.download(c), ref, epi_tol(orc, k), "batched few-tile op, in-place residual")
    # planes are added in plane order: two runs on the same operands agree bit for bit
    n2 = 1024
    a2, _ = upload_det(ta, ctx, ex, orc, (n2, n2), 0)
    b2, _ = upload_det(ta, ctx, ex, orc, (n2, n2), 1)
    c2, c3 = ta.Tensor.uninit_device(ctx, (n2, n2)), ta.Tensor.uninit_device(ctx, (n2, n2))
    ex.run_matmuls([ta.MatmulCall(a2, b2, c2)])
    ex.run_matmuls([ta.MatmulCall(a2, b2, c3)])
    assert (ex.download(c2) == ex.download(c3)).all()


def test_config2_shape_family_small(setup, orc):
    """Batched GEMM with shared B, per-batch bias, SiLU and residual at a size the
    oracle finishes in seconds (the full 32 x 2048^3 case is in test_full_size.py)."""
    ta, ctx, ex, _ = setup
    batch, m, n, k = 4, 256, 512, 384
    sig = 1.0 / np.sqrt(k)
    ha, hb = orc.fill_normal((batch, m, k), 10, sig), orc.fill_normal((k, n), 11, sig)
    hbias, hr = orc.fill_normal((batch, n), 12, sig), orc.fill_normal((batch, m, n), 13, sig)
    a, b = ta.Tensor.uninit_device(ctx, (batch, m, k)), ta.Tensor.uninit_device(ctx, (k, n))
    bias, r = ta.Tensor.uninit_device(ctx, (batch, n)), ta.Tensor.uninit_device(ctx, (batch, m, n))
    c = ta.Tensor.uninit_device(ctx, (batch, m, n))
    for t, h in ((a, ha), (b, hb), (bias, hbias), (r, hr)):
        ex.upload(h, t)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c),
                            ta.Epilogue(bias, ta.Activation.SILU, ta.Binary.ADD_SCALED, r, 1.0))])
    ref = orc.cpu_bmm(ha, hb, batch, m, n, k)
    ref = orc.cpu_epilogue(ref, batch, m, n, bias=hbias, act="silu", binary="add_scaled", d=hr, beta=1.0)
    check(orc, ex.download(c), ref, epi_tol(orc, k), "config 2 (small)")


def test_golden_vectors_through_the_gpu(setup, orc):
    import json
    import os
    ta, ctx, ex, _ = setup
    with open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")) as f:
        golden = json.load(f)
    for g in golden["gemm"]:
        cs = g["case"]
        batch, m, n, k = cs["batch"], cs["m"], cs["n"], cs["k"]
        a, _ = upload_det(ta, ctx, ex, orc, (batch, m, k), cs["seeds"][0])
        b, _ = upload_det(ta, ctx, ex, orc, (k, n) if cs["b_shared"] else (batch, k, n), cs["seeds"][1])
        c = ta.Tensor.uninit_device(ctx, (batch, m, n))
        bias = d = None
        if cs["bias_kind"] == "n":
            bias, _ = upload_det(ta, ctx, ex, orc, (n,), cs["seeds"][2])
        elif cs["bias_kind"] == "bn":
            bias, _ = upload_det(ta, ctx, ex, orc, (batch, n), cs["seeds"][2])
        if cs["binary"] != "none":
            d, _ = upload_det(ta, ctx, ex, orc, (batch, m, n), cs["seeds"][3])
        ep = ta.Epilogue(bias, ta.Activation[cs["act"].upper()], ta.Binary[cs["binary"].upper()], d, cs["beta"])
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c, cs["alpha"]), ep)])
        got = ex.download(c).reshape(-1)[g["indices"]]
        want = np.array(g["values"], np.float32)
        assert np.abs(got - want).max() <= epi_tol(orc, k)
        assert rel_err(got, want) <= REL_TOL
