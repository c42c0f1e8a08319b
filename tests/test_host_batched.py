"""Host-resident batched matmul (ta_run_matmul_host_batched): the pipelined upload / GEMM /
download call against (a) the tensor path it replaces, applied chunk by chunk -- bit for bit,
since the same kernels compute every chunk -- and (b) the CPU oracle with the reference's tolerances
(tests/correctness/epilogue.rs:52-54).  Ragged tails, explicit and automatic chunking, shared
and per-plane bias, host and device B (f32 and f16), pageable and page-locked buffers.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def det(orc, shape, seed):
    return orc.fill_det(int(np.prod(shape)), seed).reshape(shape).astype(np.float32)


def tensor_path(ta, ctx, ex, a, b_t, bias, d, act, binary, alpha, beta, chunk=0):
    """upload -> run_ops -> download with device tensors, chunk by chunk: the sequence the one
    call replaces (routing may depend on the batch count, so the comparison keeps the chunking)."""
    batch = a.shape[0]
    cb = min(chunk or max(1, batch // 16), batch)
    if cb < batch:
        parts = []
        for lo in range(0, batch, cb):
            hi = min(lo + cb, batch)
            parts.append(tensor_path(ta, ctx, ex, np.ascontiguousarray(a[lo:hi]), b_t,
                                     bias if bias is None or bias.ndim == 1 else np.ascontiguousarray(bias[lo:hi]),
                                     None if d is None else np.ascontiguousarray(d[lo:hi]),
                                     act, binary, alpha, beta, hi - lo))
        return np.concatenate(parts, axis=0)
    batch, m, k = a.shape
    n = b_t.shape[-1]
    ta_a = ta.Tensor.uninit_device(ctx, (batch, m, k))
    ta_c = ta.Tensor.uninit_device(ctx, (batch, m, n))
    ex.upload(a.ravel(), ta_a)
    tb = td = None
    if bias is not None:
        tb = ta.Tensor.uninit_device(ctx, bias.shape)
        ex.upload(bias.ravel(), tb)
    if d is not None:
        td = ta.Tensor.uninit_device(ctx, (batch, m, n))
        ex.upload(d.ravel(), td)
    ep = ta.Epilogue(bias=tb, activation=act, binary=binary, d=td, beta=beta)
    ex.run_ops([ta.MatmulOp(ta.MatmulCall(ta_a, b_t, ta_c, alpha), ep)])
    return ex.download(ta_c).reshape(batch, m, n)


@pytest.mark.parametrize("batch,m,n,k,chunk", [
    (7, 160, 264, 136, 2),      # ragged tail chunk of one plane
    (5, 128, 256, 64, 0),       # library-chosen chunking
    (3, 96, 72, 40, 8),         # chunk larger than the batch: one stage
    (9, 257, 136, 100, 4),      # rows off the tile grid, K % 16 != 0
])
@pytest.mark.parametrize("per_batch_bias", [False, True])
def test_bit_identical_to_the_tensor_path_and_within_oracle_tolerance(gpu, orc, batch, m, n, k, chunk,
                                                                      per_batch_bias):
    ta, ctx, ex = gpu
    a, b = det(orc, (batch, m, k), 11), det(orc, (k, n), 12)
    bias = det(orc, (batch, n) if per_batch_bias else (n,), 13)
    d = det(orc, (batch, m, n), 14)
    c = np.full((batch, m, n), np.nan, np.float32)
    st = ex.run_matmul_host_batched(a, b, c, bias=bias, d=d, activation=ta.Activation.SILU,
                                    binary=ta.Binary.ADD_SCALED, alpha=0.75, beta=0.5, chunk_batch=chunk)
    assert st.gpu_time_ns and st.total_flops == 2 * batch * m * n * k
    tb = ta.Tensor.uninit_device(ctx, (k, n))
    ex.upload(b.ravel(), tb)
    want = tensor_path(ta, ctx, ex, a, tb, bias, d, ta.Activation.SILU, ta.Binary.ADD_SCALED, 0.75, 0.5, chunk)
    assert np.array_equal(c, want)

    acc = orc.cpu_bmm(a, b, batch, m, n, k, alpha=0.75)
    acc = np.asarray(acc, np.float64).reshape(batch, m, n)
    z = acc + (bias[:, None, :] if per_batch_bias else bias[None, None, :])
    ref = z / (1.0 + np.exp(-z)) + 0.5 * d
    tol = 2 * orc.tolerance(k) + 1e-4
    assert float(np.abs(c - ref).max()) <= tol


def test_plain_product_device_b_and_pinned_buffers(gpu, orc):
    ta, ctx, ex = gpu
    batch, m, n, k = 6, 192, 128, 96
    a = ta.pinned_empty((batch, m, k))
    a[...] = det(orc, (batch, m, k), 21)
    c = ta.pinned_empty((batch, m, n))
    c[...] = np.nan
    b = det(orc, (k, n), 22)
    tb = ta.Tensor.uninit_device(ctx, (k, n))
    ex.upload(b.ravel(), tb)
    ex.run_matmul_host_batched(a, tb, c, chunk_batch=1)
    want = tensor_path(ta, ctx, ex, np.array(a), tb, None, None, 0, 0, 1.0, 0.0, 1)
    assert np.array_equal(c, want)
    # a second call re-uses the staging ring; a different geometry re-allocates it
    c[...] = np.nan
    ex.run_matmul_host_batched(a, tb, c, chunk_batch=1)
    assert np.array_equal(c, want)
    c2 = np.empty((2, m, n), np.float32)
    ex.run_matmul_host_batched(np.ascontiguousarray(a[:2]), tb, c2, chunk_batch=2)
    assert np.array_equal(c2, tensor_path(ta, ctx, ex, np.array(a[:2]), tb, None, None, 0, 0, 1.0, 0.0, 2))


def test_f16_weights_on_the_device(gpu, orc):
    """Shared f16 B: every chunk goes through the f16-weight tensor-core GEMM (M >= 32)."""
    ta, ctx, ex = gpu
    batch, m, n, k = 4, 128, 256, 128
    a = det(orc, (batch, m, k), 31)
    b = det(orc, (k, n), 32)
    tb = ta.Tensor.uninit_device_f16(ctx, (k, n))
    ex.upload(b.ravel(), tb)
    c = np.empty((batch, m, n), np.float32)
    ex.run_matmul_host_batched(a, tb, c, chunk_batch=3)
    want = tensor_path(ta, ctx, ex, a, tb, None, None, 0, 0, 1.0, 0.0, 3)
    assert np.array_equal(c, want)


def test_invalid_descriptions_are_rejected(gpu, orc):
    ta, ctx, ex = gpu
    a, b = det(orc, (2, 32, 16), 1), det(orc, (16, 24), 2)
    c = np.empty((2, 32, 24), np.float32)
    with pytest.raises(ta.TensorAshError, match="binary epilogue needs"):
        ex.run_matmul_host_batched(a, b, c, binary=ta.Binary.MUL)
    with pytest.raises(ta.TensorAshError, match="without a binary"):
        ex.run_matmul_host_batched(a, b, c, d=np.zeros_like(c))
    with pytest.raises(ValueError):
        ex.run_matmul_host_batched(a, b, np.empty((2, 32, 25), np.float32))
    tb = ta.Tensor.uninit_device(ctx, (24, 16))
    with pytest.raises(ta.TensorAshError, match="device B must be"):
        ex.run_matmul_host_batched(a, tb, c)


def test_pinned_memory_outlives_views():
    import gc
    import __graft_entry__ as entry
    ta = entry.load_package()
    x = ta.pinned_empty((4, 8))
    x[...] = 3.0
    v = x[1:3].reshape(-1)
    del x
    gc.collect()
    assert (v == 3.0).all()
