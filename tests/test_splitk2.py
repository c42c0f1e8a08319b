"""GPU tests of the deterministic two-stage split-K route
(tests/correctness/splitk2.rs:7-175 in the reference)."""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


def run_case(gpu, orc, batch, m, n, k, splits, alpha):
    ta, ctx, ex = gpu
    sh = lambda r, c: (r, c) if batch == 1 else (batch, r, c)
    a, ha = upload_det(ta, ctx, ex, orc, sh(m, k), 101)
    b, hb = upload_det(ta, ctx, ex, orc, sh(k, n), 102)
    c = ta.Tensor.uninit_device(ctx, sh(m, n))
    ex.upload(np.full(batch * m * n, 7.0, np.float32), c)      # stale contents must be overwritten
    ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c, alpha)], splits)
    return ex.download(c).reshape(-1), orc.cpu_bmm(ha, hb, batch, m, n, k, alpha=alpha), (ha, hb)


@pytest.mark.parametrize("case", [(1, 64, 64, 8192, 0, 1.0), (1, 256, 256, 4096, 16, 1.0),
                                  (1, 101, 103, 999, 7, 1.0), (3, 64, 64, 2048, 8, 0.25)])
def test_splitk2_matches_cpu(gpu, orc, case):
    got, ref, _ = run_case(gpu, orc, *case)
    e, idx = orc.max_abs_err(got, ref)
    assert e <= 2.0 * orc.tolerance(case[3]), f"{case}: err {e} at {idx}"


def test_splitk2_simt_stage1_is_deterministic_and_matches_shader_order(gpu, orc):
    """An executor whose kernel selection names the split-K2 stage-1 kernel keeps the SIMT stage 1:
    the same per-split fma chains and the same ordered plane sum as the reference shaders, bit for bit."""
    ta, ctx, _ = gpu
    ex = ta.Executor(ctx, 2, 8, "split_k2_m128n128")
    pinned = (ta, ctx, ex)
    got1, _, (ha, hb) = run_case(pinned, orc, 1, 128, 128, 4096, 16, 1.0)
    got2, _, _ = run_case(pinned, orc, 1, 128, 128, 4096, 16, 1.0)
    assert got1.tobytes() == got2.tobytes(), "split-K2 results differ across runs"
    emu = orc.splitk2_f32(ha, hb, 128, 128, 4096, 16)
    assert got1.tobytes() == emu.tobytes()
    ex.close()


@pytest.mark.parametrize("case", [(1, 128, 128, 4096, 16, 1.0), (1, 64, 64, 65536, 64, 1.0), (1, 64, 256, 65536, 4, 0.5),
                                  (2, 96, 200, 8192, 8, 1.0), (1, 300, 72, 16384, 32, 1.0)])
def test_splitk2_tensor_stage1_is_deterministic_and_within_the_bound(gpu, orc, case):
    """The default route: stage 1 on the tensor cores (3xTF32) wherever K is a multiple of 16 * splits.
    Fixed issue order and a fixed plane order in the reduce: two runs are bit-identical; the result
    stays inside the reference's bound (tests/correctness/splitk2.rs:114-122) and inside 1e-5 of max|C|."""
    got1, ref, _ = run_case(gpu, orc, *case)
    got2, _, _ = run_case(gpu, orc, *case)
    assert got1.tobytes() == got2.tobytes(), "split-K2 results differ across runs"
    e, idx = orc.max_abs_err(got1, ref)
    assert e <= 2.0 * orc.tolerance(case[3]), f"{case}: err {e} at {idx}"
    assert e / float(np.abs(ref).max()) <= 1e-5, f"{case}: rel {e / float(np.abs(ref).max()):.3e}"


def test_deep_k_config_sweep(gpu, orc):
    """M=64, N in {64, 256}, K=65536, splits 4..64: run-to-run bit-identical and
    inside the reference bound 2*8*K*eps."""
    ta, ctx, ex = gpu
    k = 65536
    for n in (64, 256):
        a, ha = upload_det(ta, ctx, ex, orc, (64, k), 201)
        b, hb = upload_det(ta, ctx, ex, orc, (k, n), 202)
        c = ta.Tensor.uninit_device(ctx, (64, n))
        ref = orc.cpu_bmm(ha, hb, 1, 64, n, k)
        for s in (4, 8, 16, 32, 64):
            ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c)], s)
            one = ex.download(c).copy()
            ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c)], s)
            two = ex.download(c)
            assert one.tobytes() == two.tobytes()
            e, _ = orc.max_abs_err(one, ref)
            assert e <= 2.0 * orc.tolerance(k)
            rel = e / float(np.abs(ref).max())
            assert rel <= 1e-5, f"N={n} S={s}: rel {rel}"


def test_auto_route_deep_k(gpu, orc):
    ta, ctx, ex = gpu
    m, n, k = 37, 41, 1088
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 131)
    b, hb = upload_det(ta, ctx, ex, orc, (k, n), 137)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    before = ta.kernel_launch_count()
    ex.run_matmuls([ta.MatmulCall(a, b, c, 0.75)])
    assert ta.kernel_launch_count() - before == 2        # stage 1 + reduce
    e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, m, n, k, alpha=0.75))
    assert e <= 2.0 * orc.tolerance(k)


def test_rejections_and_fallback(gpu, orc):
    ta, ctx, ex = gpu
    a, ha = upload_det(ta, ctx, ex, orc, (16, 16), 211)
    b, hb = upload_det(ta, ctx, ex, orc, (16, 16), 223)
    c = ta.Tensor.uninit_device(ctx, (16, 16))
    with pytest.raises(ta.TensorAshError, match="accumulate"):
        ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c, 1.0, True)], 4)
    ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c)], 1)
    e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, 16, 16, 16))
    assert e <= orc.tolerance(16)
    with pytest.raises(ta.TensorAshError, match="exceeds K=16"):
        ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c)], 17)
