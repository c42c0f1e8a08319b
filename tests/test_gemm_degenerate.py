"""N == 1 (column), K == 1 (outer product) and M <= 32 over f32 weights (rows): the reference's
col_bda / outer_bda / row_bda routes (src/pipeline/catalog.rs:264-281, pipeline/mod.rs:530-531),
here three small kernels of the SIMT family.  Against the f64 oracle with the reference's tolerance, with every fused stage."""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,m,n,k", [(1, 300, 1, 517), (3, 64, 1, 4096), (1, 4096, 1, 4096), (1, 1, 1, 1),
                                         (2, 130, 257, 1), (1, 4096, 512, 1), (1, 7, 1, 1),
                                         # M <= 32 rows over f32 weights (row_bda, widened)
                                         (1, 1, 4096, 4096), (2, 5, 200, 333), (1, 8, 64, 64), (1, 3, 130, 70),
                                         (2, 6, 256, 512), (1, 4, 4096, 1028),
                                         # 9..32 rows: groups of 16 rows (one or two per column block)
                                         (1, 9, 128, 256), (2, 16, 200, 333), (1, 17, 96, 68), (3, 32, 160, 512),
                                         (1, 29, 70, 65)])
@pytest.mark.parametrize("fused", [False, True])
def test_column_and_outer_shapes(gpu, orc, batch, m, n, k, fused):
    ta, ctx, ex = gpu
    sh = lambda r, c: (r, c) if batch == 1 else (batch, r, c)
    a, ha = upload_det(ta, ctx, ex, orc, sh(m, k), 31)
    b, hb = upload_det(ta, ctx, ex, orc, sh(k, n), 32)
    c, hc = upload_det(ta, ctx, ex, orc, sh(m, n), 33)
    alpha, accumulate = (0.5, True) if fused else (1.0, False)
    ep, kw = ta.Epilogue(), {}
    if fused:
        bias, hbias = upload_det(ta, ctx, ex, orc, (batch, n) if batch > 1 else (n,), 34)
        d, hd = upload_det(ta, ctx, ex, orc, sh(m, n), 35)
        ep = ta.Epilogue(bias, ta.Activation.GELU, ta.Binary.ADD_SCALED, d, 0.25)
        kw = dict(bias=hbias, act=3, binary=1, d=hd, beta=0.25)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c, alpha, accumulate), ep)])
    ref = orc.cpu_bmm(ha, hb, batch, m, n, k, alpha=alpha, c_init=hc if accumulate else None, accumulate=accumulate)
    if fused:
        ref = orc.cpu_epilogue(ref, batch, m, n, **kw)
    got = ex.download(c).reshape(-1)
    tol = 2 * orc.tolerance(k) + (1e-4 if fused else 0.0)
    assert np.isfinite(got).all() and float(np.abs(got - np.asarray(ref).reshape(-1)).max()) <= tol
    assert ex.dispatch_info_for(batch, m, n, k).kernel.startswith("ffma_")


def test_column_with_f16_weights(gpu, orc):
    ta, ctx, ex = gpu
    m, k = 200, 384
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 41)
    hb = orc.round_via_f16(orc.fill_det(k, 42)).reshape(k, 1)
    b = ta.Tensor.uninit_device_f16(ctx, (k, 1))
    ex.upload(hb.ravel(), b)
    c = ta.Tensor.uninit_device(ctx, (m, 1))
    ex.run_matmuls([ta.MatmulCall(a, b, c)])
    ref = orc.cpu_bmm(ha, hb, 1, m, 1, k)
    assert float(np.abs(ex.download(c).reshape(-1) - ref).max()) <= 2 * orc.tolerance(k)
