"""f16-weight GEMM on the tensor cores (tcgen05 kind::f16) against the f64 oracle.

Cases follow the reference's f16-weight tests (tests/correctness/f16.rs:21-241: plain,
batched with shared and per-batch B, bias + ReLU + residual, SiLU + residual) at the
prefill shapes of the llama configuration, plus every partial-tile residue of the
128 x {64,128,256} x 32 tiles.  Tolerance: 2e-3 relative to max(1, max|ref|), the
f16-weight bound; the oracle sees f32 A and f16-rounded B, so the kernel's f16
rounding of A is inside the measured error.
"""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu

F16W_TOL = 2e-3


def rel_err(got, ref):
    got = np.asarray(got, np.float32).reshape(-1)
    ref = np.asarray(ref, np.float32).reshape(-1)
    assert np.isfinite(got).all(), "non-finite output"
    return float(np.abs(got - ref).max() / max(1.0, float(np.abs(ref).max())))


@pytest.fixture(scope="module", params=["auto", "f16w_umma_m128n256", "f16w_umma_m128n128", "f16w_umma_m128n64"])
def setup(request, ta):
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 16, request.param, tune=False)
    yield ta, ctx, ex, request.param
    ex.close()
    ctx.close()


def upload_f16w(ta, ctx, ex, orc, shape, seed):
    host = orc.fill_det(int(np.prod(shape)), seed)
    t = ta.Tensor.uninit_device_f16(ctx, shape)
    ex.upload(host, t)
    return t, orc.round_via_f16(host)


def test_route_is_the_tensor_core_kernel(setup):
    ta, ctx, ex, sel = setup
    info = ex.dispatch_info_for(1, 512, 2048, 2048, b_f16=True)
    assert info.kernel.startswith("f16w_umma_m128n")
    assert info.tile[0] == 128 and info.tile[2] == 32
    if sel != "auto":
        assert info.kernel == sel
    # decode rows stay on the bandwidth GEMV; unaligned N falls back to the FFMA tiles
    if sel == "auto":
        assert ex.dispatch_info_for(1, 4, 2048, 2048, b_f16=True).kernel.startswith("f16w_row")
        assert ex.dispatch_info_for(1, 512, 2044, 2048, b_f16=True).kernel.startswith("f16w_ffma")


@pytest.mark.parametrize("m,n,k", [(512, 2048, 2048), (512, 2560, 2048), (512, 5632, 2048), (512, 2048, 5632)])
def test_prefill_shapes(setup, orc, m, n, k):
    ta, ctx, ex, _ = setup
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 71)
    b, hb = upload_f16w(ta, ctx, ex, orc, (k, n), 72)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    st = ex.run_matmuls([ta.MatmulCall(a, b, c)])
    assert st.total_flops == 2 * m * n * k
    got = ex.download(c).reshape(m, n)
    # the f64 oracle on a strided sample of rows keeps the CPU side in seconds
    rows = np.arange(0, m, 37)
    ref = orc.cpu_bmm(ha.reshape(m, k)[rows].copy(), hb, 1, len(rows), n, k).reshape(len(rows), n)
    assert rel_err(got[rows], ref) <= F16W_TOL
    # full coverage through a float32 BLAS product with a looser bound
    blas = ha.reshape(m, k) @ hb.reshape(k, n)
    assert rel_err(got, blas) <= 2 * F16W_TOL


def test_partial_tiles_in_m_n_and_k(setup, orc):
    ta, ctx, ex, _ = setup
    for m in (33, 128, 130, 257):
        for n in (64, 72, 200, 264, 520):
            for k in (64, 100, 132):
                a, ha = upload_det(ta, ctx, ex, orc, (m, k), 5 + m)
                b, hb = upload_f16w(ta, ctx, ex, orc, (k, n), 7 + n)
                c = ta.Tensor.uninit_device(ctx, (m, n))
                ex.upload(np.full(m * n, 123.0, np.float32), c)
                ex.run_matmuls([ta.MatmulCall(a, b, c)])
                ref = orc.cpu_bmm(ha, hb, 1, m, n, k)
                assert rel_err(ex.download(c), ref) <= F16W_TOL, f"M={m} N={n} K={k}"


def test_batched_shared_and_per_batch_weights_alpha_accumulate(setup, orc):
    ta, ctx, ex, _ = setup
    batch, m, n, k = 3, 140, 136, 96
    a, ha = upload_det(ta, ctx, ex, orc, (batch, m, k), 81)
    for b_shape in ((k, n), (batch, k, n)):
        b, hb = upload_f16w(ta, ctx, ex, orc, b_shape, 82)
        init = orc.fill_det(batch * m * n, 83)
        c = ta.Tensor.uninit_device(ctx, (batch, m, n))
        ex.upload(init, c)
        ex.run_matmuls([ta.MatmulCall(a, b, c, 0.5, True)])
        ref = orc.cpu_bmm(ha, hb, batch, m, n, k, alpha=0.5, c_init=init, accumulate=True)
        assert rel_err(ex.download(c), ref) <= F16W_TOL, f"B shape {b_shape}"


def test_fused_epilogues(setup, orc):
    """bias + ReLU + residual (tests/common/mod.rs:63-84) and SiLU * D, the prefill SwiGLU gate."""
    ta, ctx, ex, _ = setup
    m, n, k = 160, 264, 128
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 91)
    b, hb = upload_f16w(ta, ctx, ex, orc, (k, n), 92)
    bias, hbias = upload_det(ta, ctx, ex, orc, (n,), 93)
    d, hd = upload_det(ta, ctx, ex, orc, (m, n), 94)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    base = orc.cpu_bmm(ha, hb, 1, m, n, k).reshape(m, n).astype(np.float64)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c),
                            ta.Epilogue(bias=bias, activation=ta.Activation.RELU, binary=ta.Binary.ADD_SCALED, d=d,
                                        beta=0.75))])
    ref = np.maximum(base + hbias[None, :], 0.0) + 0.75 * hd.reshape(m, n)
    assert rel_err(ex.download(c), ref) <= F16W_TOL
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c),
                            ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=d))])
    ref = base / (1.0 + np.exp(-base)) * hd.reshape(m, n)
    assert rel_err(ex.download(c), ref) <= F16W_TOL


@pytest.mark.parametrize("m,n,k", [(300, 520, 8192), (130, 192, 4096), (512, 2048, 5632)])
def test_in_kernel_k_split_with_partial_tiles_and_fused_epilogue(setup, orc, m, n, k):
    """Deep-K shapes with few tiles take the in-kernel K split (partials in scratch, ticket, slice-wise
    reduce): partial row and column tiles, bias + SiLU + scaled residual in the reducing pass, then
    alpha with accumulation; two runs are bit-identical (fixed slice order)."""
    ta, ctx, ex, _ = setup
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 111)
    b, hb = upload_f16w(ta, ctx, ex, orc, (k, n), 112)
    bias, hbias = upload_det(ta, ctx, ex, orc, (n,), 113)
    d, hd = upload_det(ta, ctx, ex, orc, (m, n), 114)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    base = (ha.reshape(m, k).astype(np.float64) @ hb.reshape(k, n).astype(np.float64))
    op = ta.MatmulOp(ta.MatmulCall(a, b, c),
                     ta.Epilogue(bias=bias, activation=ta.Activation.SILU, binary=ta.Binary.ADD_SCALED, d=d, beta=0.5))
    ex.run_ops([op])
    z = base + hbias[None, :]
    ref = z / (1.0 + np.exp(-z)) + 0.5 * hd.reshape(m, n)
    first = ex.download(c).copy()
    assert rel_err(first, ref) <= F16W_TOL
    ex.run_ops([op])
    assert np.array_equal(first.view(np.uint32), ex.download(c).view(np.uint32))
    init = orc.fill_det(m * n, 115)
    ex.upload(init, c)
    ex.run_matmuls([ta.MatmulCall(a, b, c, 0.25, True)])
    assert rel_err(ex.download(c), 0.25 * base + init.reshape(m, n)) <= F16W_TOL


def test_prepared_replay_matches_direct_bitwise(setup, orc):
    ta, ctx, ex, _ = setup
    m, n, k = 256, 512, 256
    a, _ = upload_det(ta, ctx, ex, orc, (m, k), 101)
    b, _ = upload_f16w(ta, ctx, ex, orc, (k, n), 102)
    c1 = ta.Tensor.uninit_device(ctx, (m, n))
    c2 = ta.Tensor.uninit_device(ctx, (m, n))
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c1))])
    prep = ex.prepare_ops([ta.MatmulOp(ta.MatmulCall(a, b, c2))])
    prep.run()
    prep.run()
    assert (ex.download(c1) == ex.download(c2)).all()
