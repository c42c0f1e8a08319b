"""GPU tests of the non-GEMM model ops of the C ABI against the oracle
(examples/c_smoke.c:150-239 and tests/correctness/ops.rs in the reference)."""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


def test_rms_and_layer_norm(gpu, orc):
    ta, ctx, ex = gpu
    for rows, cols in ((2, 3), (5, 2048), (7, 1000)):
        x, hx = upload_det(ta, ctx, ex, orc, (rows, cols), 301)
        w, hw = upload_det(ta, ctx, ex, orc, (cols,), 302)
        b, hb = upload_det(ta, ctx, ex, orc, (cols,), 303)
        out = ta.Tensor.uninit_device(ctx, (rows, cols))
        ex.rms_norm(x, w, out, 1e-5)
        assert np.abs(ex.download(out) - orc.cpu_rmsnorm(hx.reshape(rows, cols), hw, 1e-5)).max() <= 1e-4
        ex.layer_norm(x, w, b, out, 1e-5)
        assert np.abs(ex.download(out) - orc.cpu_layernorm(hx.reshape(rows, cols), hw, hb, 1e-5)).max() <= 1e-4
        ex.rms_norm(x, w, x, 1e-5)            # in place
        assert np.abs(ex.download(x) - orc.cpu_rmsnorm(hx.reshape(rows, cols), hw, 1e-5)).max() <= 1e-4
    bad = ta.Tensor.uninit_device(ctx, (5,))
    with pytest.raises(ta.TensorAshError, match="weight length 5 != row length"):
        ex.rms_norm(x, bad, out, 1e-5)


def test_softmax_masks(gpu, orc):
    ta, ctx, ex = gpu
    rows, cols = 12, 333
    x, hx = upload_det(ta, ctx, ex, orc, (rows, cols), 311)
    out = ta.Tensor.uninit_device(ctx, (rows, cols))
    for kind, vp, rpg in ((0, 0, 0), (1, 100, 0), (1, 1000, 0), (2, 5, 4), (2, 0, 12)):
        ex.softmax_rows(x, out, 0.125, kind, vp, rpg)
        got = ex.download(out)
        ref = orc.cpu_softmax_rows(hx.reshape(rows, cols), 0.125, kind, vp, rpg)
        assert np.abs(got - ref).max() <= 1e-5
        assert ((ref == 0.0) <= (got == 0.0)).all()      # masked columns are exactly zero
    with pytest.raises(ta.TensorAshError, match="rows_per_group 5 must divide rows 12"):
        ex.softmax_rows(x, out, 1.0, 2, 0, 5)
    with pytest.raises(ta.TensorAshError, match="mask_kind 3 is invalid"):
        ex.softmax_rows(x, out, 1.0, 3, 0, 0)


def test_rope_full_and_partial(gpu, orc):
    ta, ctx, ex = gpu
    tokens, heads, dh, t_max = 6, 4, 64, 32
    x, hx = upload_det(ta, ctx, ex, orc, (tokens, heads, dh), 321)
    out = ta.Tensor.uninit_device(ctx, (tokens, heads, dh))
    for rot in (64, 32, 2):
        pos = np.arange(t_max, dtype=np.float64)[:, None]
        inv = 1.0 / (10000.0 ** (2.0 * np.arange(rot // 2, dtype=np.float64) / rot))
        ang = pos * inv[None, :]
        table = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)     # [T, rot/2, 2]
        tab = ta.Tensor.uninit_device(ctx, table.shape)
        ex.upload(table, tab)
        ex.rope(x, tab, out, heads, dh, rot, 3)
        ref = orc.cpu_rope(hx, table, tokens, heads, dh, rot, 3)
        assert np.abs(ex.download(out).reshape(-1) - ref.reshape(-1)).max() <= 1e-5
    with pytest.raises(ta.TensorAshError, match="rot_dim 3 must be even"):
        ex.rope(x, tab, out, heads, dh, 3, 0)
    with pytest.raises(ta.TensorAshError, match="table length"):
        ex.rope(x, tab, out, heads, dh, 2, 30)


def test_copy_strided(gpu, orc):
    ta, ctx, ex = gpu
    a = ta.Tensor.uninit_device(ctx, (2, 3))
    ex.upload(np.arange(1, 7, dtype=np.float32), a)
    t = ta.Tensor.uninit_device(ctx, (3, 2))
    ex.copy_strided(a, t, (3, 2, 1), 0, (1, 3, 0), 0, (2, 1, 0))
    assert ex.download(t).reshape(-1).tolist() == [1, 4, 2, 5, 3, 6]
    with pytest.raises(ta.TensorAshError, match="src and dst must be different"):
        ex.copy_strided(a, a, (3, 2, 1), 0, (1, 3, 0), 0, (2, 1, 0))
    with pytest.raises(ta.TensorAshError, match="zero axis"):
        ex.copy_strided(a, t, (3, 0, 1), 0, (1, 3, 0), 0, (2, 1, 0))
    with pytest.raises(ta.TensorAshError, match="source access reaches element"):
        ex.copy_strided(a, t, (3, 3, 1), 0, (1, 3, 0), 0, (2, 1, 0))
    # KV-cache style append: rows of src into a strided slot of dst
    src, hs = upload_det(ta, ctx, ex, orc, (4, 8), 331)
    dst = ta.Tensor.uninit_device(ctx, (4, 16, 8))
    ex.upload(np.zeros(4 * 16 * 8, np.float32), dst)
    ex.copy_strided(src, dst, (8, 4, 1), 0, (1, 8, 0), 5 * 8, (1, 16 * 8, 0))
    got = ex.download(dst)
    assert (got[:, 5, :] == hs.reshape(4, 8)).all() and got.sum() == pytest.approx(float(hs.sum()), rel=1e-5)


def test_alias_with_shape(gpu, orc):
    ta, ctx, ex = gpu
    t, h = upload_det(ta, ctx, ex, orc, (6, 4), 341)
    al = t.alias_with_shape((2, 12))
    assert al.device_ptr == t.device_ptr and al.len() == 24
    assert (ex.download(al).reshape(-1) == h).all()
    with pytest.raises(ta.TensorAshError, match="alias_with_shape"):
        t.alias_with_shape((5, 5))
