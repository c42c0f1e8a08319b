"""a16 route: f16 A, f16 B and f16 C on the tensor cores (the reference's *_a16_* kernels,
src/matmul/resolution.rs:123-172: M, N multiples of 64, K of 32, f32 accumulation, no fused
stages).  Operands are exactly representable, so the only rounding is the f32 accumulation and the
store to f16: results must sit within one f16 ulp, plus the reference's f32 accumulation bound
8 K eps (it matters only where a sum cancels to almost nothing), of the f64 product rounded to f16.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def f16_tensor(ta, ctx, ex, orc, shape, seed, scale=1.0):
    host = orc.round_via_f16(orc.fill_det(int(np.prod(shape)), seed) * np.float32(scale))
    t = ta.Tensor.uninit_device_f16(ctx, shape)
    ex.upload(host, t)
    return t, host.reshape(shape)


def one_ulp(ref):
    """Half-precision spacing at |ref| (at least the smallest normal's)."""
    mag = np.maximum(np.abs(ref.astype(np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(mag)) - 10)


@pytest.mark.parametrize("batch,m,n,k,shared_b", [
    (1, 64, 64, 32, True), (1, 128, 192, 96, True), (1, 512, 2048, 2048, True),
    (3, 128, 64, 64, True), (2, 192, 320, 160, False), (1, 320, 576, 1056, True),
])
@pytest.mark.parametrize("alpha,accumulate", [(1.0, False), (0.5, True)])
def test_a16_matches_the_f64_product_rounded_to_f16(gpu, orc, batch, m, n, k, shared_b, alpha, accumulate):
    ta, ctx, ex = gpu
    sa = (m, k) if batch == 1 else (batch, m, k)
    sb = (k, n) if (batch == 1 or shared_b) else (batch, k, n)
    sc = (m, n) if batch == 1 else (batch, m, n)
    a, ha = f16_tensor(ta, ctx, ex, orc, sa, 3)
    b, hb = f16_tensor(ta, ctx, ex, orc, sb, 4)
    c, hc = f16_tensor(ta, ctx, ex, orc, sc, 5)
    assert c.is_f16
    st = ex.run_matmuls([ta.MatmulCall(a, b, c, alpha, accumulate)])
    assert st.total_flops == 2 * batch * m * n * k
    got = ex.download(c).reshape(batch, m, n).astype(np.float64)
    A = ha.reshape(batch, m, k).astype(np.float64)
    B = np.broadcast_to(hb.reshape((-1, k, n)).astype(np.float64), (batch, k, n))
    ref = alpha * np.einsum("bmk,bkn->bmn", A, B) + (hc.reshape(batch, m, n) if accumulate else 0.0)
    ref16 = ref.astype(np.float16).astype(np.float64)
    assert np.isfinite(got).all()
    assert (np.abs(got - ref16) <= one_ulp(ref16) + orc.tolerance(k)).all()
    # and nearly always the correctly rounded value (f32 accumulation vs f64 only moves ties)
    assert (got == ref16).mean() > 0.98


def test_a16_prepared_replay_and_rejections(gpu, orc):
    ta, ctx, ex = gpu
    a, _ = f16_tensor(ta, ctx, ex, orc, (128, 64), 7)
    b, _ = f16_tensor(ta, ctx, ex, orc, (64, 128), 8)
    c1 = ta.Tensor.uninit_device_f16(ctx, (128, 128))
    c2 = ta.Tensor.uninit_device_f16(ctx, (128, 128))
    ex.run_matmuls([ta.MatmulCall(a, b, c1)])
    prep = ex.prepare_ops([ta.MatmulOp(ta.MatmulCall(a, b, c2))])
    prep.run()
    assert np.array_equal(ex.download(c1), ex.download(c2))
    prep.close()
    cf32 = ta.Tensor.uninit_device(ctx, (128, 128))
    with pytest.raises(ta.TensorAshError, match="f16 A storage requires f16 C"):
        ex.run_matmuls([ta.MatmulCall(a, b, cf32)])
    bf32 = ta.Tensor.uninit_device(ctx, (64, 128))
    with pytest.raises(ta.TensorAshError, match="f16 A storage requires f16 B"):
        ex.run_matmuls([ta.MatmulCall(a, bf32, c1)])
    a_bad = ta.Tensor.uninit_device_f16(ctx, (96, 64))
    c_bad = ta.Tensor.uninit_device_f16(ctx, (96, 128))
    with pytest.raises(ta.TensorAshError, match=r"multiples of \(64, 64, 32\)"):
        ex.run_matmuls([ta.MatmulCall(a_bad, b, c_bad)])
    bias = ta.Tensor.uninit_device(ctx, (128,))
    with pytest.raises(ta.TensorAshError, match="cannot fuse epilogues"):
        ex.run_ops([ta.MatmulOp(ta.MatmulCall(a, b, c1), ta.Epilogue(bias=bias))])
