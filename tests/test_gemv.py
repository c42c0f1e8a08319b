"""GPU parity tests of the f16-weight decode GEMV / skinny GEMM (M <= 8) against
the f64 oracle with f16-rounded weights.  Cases follow the reference's
tests/correctness/{row,f16,fusion,store}.rs; tolerance for the f16-weight path
is rel 2e-3 (the products are exact in f32, so the measured error is far
smaller and is also held to the FP32 bound 2*8*K*eps)."""
import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


def make_weights(ta, ctx, ex, orc, k, n, seed, packed, sigma=0.02):
    """Weights ~N(0, sigma) rounded through f16, uploaded row-major or packed."""
    w = orc.round_via_f16(orc.fill_normal((k, n), seed, sigma))
    t = ta.Tensor.uninit_device_f16(ctx, (k, n))
    host = ta.pack_f16w_row_tiles(w, k, n, ta.f16w_row_tile_n(k, n)) if packed else w
    ex.upload(host, t)
    return t, w


def check(orc, got, ref, k, label):
    got, ref = np.asarray(got).reshape(-1), np.asarray(ref).reshape(-1)
    assert np.isfinite(got).all()
    scale = max(1e-6, float(np.abs(ref).max()))
    rel = float(np.abs(got - ref).max()) / scale
    assert rel <= 2e-3, f"{label}: rel {rel:.3e}"
    assert float(np.abs(got - ref).max()) <= 2 * orc.tolerance(k) * max(1.0, scale), label


@pytest.mark.parametrize("m", [1, 4, 8])
def test_config3_swiglu_then_down(gpu, orc, m):
    """x [M,4096]; Wg, Wup f16 [4096,11008] packed; h = silu(x@Wg)*(x@Wup) in one
    launch; y = h @ Wdown with Wdown f16 [11008,4096] packed."""
    ta, ctx, ex = gpu
    k, n = 4096, 11008
    x, hx = upload_det(ta, ctx, ex, orc, (m, k), 500 + m)
    wg, hwg = make_weights(ta, ctx, ex, orc, k, n, 511, True)
    wup, hwup = make_weights(ta, ctx, ex, orc, k, n, 512, True)
    wdn, hwdn = make_weights(ta, ctx, ex, orc, n, k, 513, True)
    h = ta.Tensor.uninit_device(ctx, (m, n))
    y = ta.Tensor.uninit_device(ctx, (m, k))
    before = ta.kernel_launch_count()
    st1 = ex.swiglu_gemv(x, wg, wup, h)
    assert ta.kernel_launch_count() == before + 1           # one dispatch for gate, up and gating
    st2 = ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(h, wdn, y), packed_b=True)])
    g = orc.cpu_bmm(hx, hwg, 1, m, n, k)
    u = orc.cpu_bmm(hx, hwup, 1, m, n, k)
    h_ref = orc.cpu_epilogue(g, 1, m, n, act="silu", binary="mul", d=u)
    check(orc, ex.download(h), h_ref, k, f"swiglu M={m}")
    got_h = ex.download(h).reshape(-1)
    y_ref = orc.cpu_bmm(got_h, hwdn, 1, m, k, n)
    check(orc, ex.download(y), y_ref, n, f"down M={m}")
    gb = (4 * k * n + 4 * m * (k + n)) / st1.gpu_time_ns, (2 * k * n + 4 * m * (k + n)) / st2.gpu_time_ns
    print(f"\nM={m}: swiglu {st1.gpu_time_ns / 1e3:.1f} us = {gb[0]:.0f} GB/s; down {st2.gpu_time_ns / 1e3:.1f} us = {gb[1]:.0f} GB/s")
    # deterministic: a second run is bit-identical
    first = ex.download(h).tobytes()
    ex.swiglu_gemv(x, wg, wup, h)
    assert ex.download(h).tobytes() == first


# decode shapes of the Llama configuration: q/o, k/v, gate/up (tile 64), down (row-major), lm_head
@pytest.mark.parametrize("k,n,packed", [(2048, 2048, True), (2048, 256, True), (2048, 5632, True),
                                        (5632, 2048, False), (2048, 32000, True), (2048, 2048, False),
                                        (1000, 72, False), (520, 96, True)])
def test_decode_shapes(gpu, orc, k, n, packed):
    ta, ctx, ex = gpu
    for m in (1, 3):
        x, hx = upload_det(ta, ctx, ex, orc, (m, k), 520)
        w, hw = make_weights(ta, ctx, ex, orc, k, n, 521, packed)
        c = ta.Tensor.uninit_device(ctx, (m, n))
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c), packed_b=packed)])
        check(orc, ex.download(c), orc.cpu_bmm(hx, hw, 1, m, n, k), k, f"{m}x{n}x{k} packed={packed}")
    info = ex.dispatch_info_for(1, 1, n, k, True)
    assert info.kernel.startswith("f16w_row_bda")


def test_packed_equals_row_major_bitwise(gpu, orc):
    """Same k-to-lane mapping in both layouts at tile 32: identical sums."""
    ta, ctx, ex = gpu
    k, n = 4096, 1024
    assert ta.f16w_row_tile_n(k, n) == 32
    x, hx = upload_det(ta, ctx, ex, orc, (1, k), 530)
    wp, _ = make_weights(ta, ctx, ex, orc, k, n, 531, True)
    wr, _ = make_weights(ta, ctx, ex, orc, k, n, 531, False)
    c1, c2 = ta.Tensor.uninit_device(ctx, (1, n)), ta.Tensor.uninit_device(ctx, (1, n))
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, wp, c1), packed_b=True)])
    ex.run_matmuls([ta.MatmulCall(x, wr, c2)])
    assert ex.download(c1).tobytes() == ex.download(c2).tobytes()


# tests/correctness/fusion.rs:17-24 (normed-A) with epilogue forms that remain legal
def test_normed_a_and_epilogue(gpu, orc):
    ta, ctx, ex = gpu
    k, n, eps = 2048, 5632, 1e-5
    for m in (1, 4):
        x, hx = upload_det(ta, ctx, ex, orc, (m, k), 540)
        nw = ta.Tensor.uninit_device(ctx, (k,))
        hnw = 1.0 + 0.1 * orc.fill_det(k, 541)
        ex.upload(hnw, nw)
        w, hw = make_weights(ta, ctx, ex, orc, k, n, 542, True)
        d, hd = upload_det(ta, ctx, ex, orc, (m, n), 543)
        c = ta.Tensor.uninit_device(ctx, (m, n))
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c),
                                     ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=d),
                                     packed_b=True, normed_a=(nw, eps))])
        xn = orc.cpu_rmsnorm(hx.reshape(m, k), hnw, eps)
        ref = orc.cpu_epilogue(orc.cpu_bmm(xn, hw, 1, m, n, k), 1, m, n, act="silu", binary="mul", d=hd)
        check(orc, ex.download(c), ref, k, f"normed-A silu*mul M={m}")
        # fused swiglu with normed-A equals the two-dispatch form (up, then gate with Mul d=up)
        w2, hw2 = make_weights(ta, ctx, ex, orc, k, n, 544, True)
        up, gated, fused = (ta.Tensor.uninit_device(ctx, (m, n)) for _ in range(3))
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w2, up), packed_b=True, normed_a=(nw, eps)),
                       ta.MatmulOpEx(ta.MatmulCall(x, w, gated),
                                     ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=up),
                                     packed_b=True, normed_a=(nw, eps))], as_graph=True)
        ex.swiglu_gemv(x, w, w2, fused, nw, eps)
        a, b = ex.download(gated), ex.download(fused)
        # the pair launch and the two single launches may cut K differently: same values up to f32 summation order
        assert np.abs(a - b).max() <= 1e-5 * max(1.0, float(np.abs(a).max()))
    # residual add (AddScaled) on the row-major route, as the o / down projections use it
    x, hx = upload_det(ta, ctx, ex, orc, (1, 5632), 545)
    w, hw = make_weights(ta, ctx, ex, orc, 5632, 2048, 546, False)
    r, hr = upload_det(ta, ctx, ex, orc, (1, 2048), 547)
    c = ta.Tensor.uninit_device(ctx, (1, 2048))
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c), ta.Epilogue(binary=ta.Binary.ADD_SCALED, d=r, beta=1.0))])
    ref = orc.cpu_epilogue(orc.cpu_bmm(hx, hw, 1, 1, 2048, 5632), 1, 1, 2048, binary="add_scaled", d=hr, beta=1.0)
    check(orc, ex.download(c), ref, 5632, "down + residual")


def rope_table(t_max, dh, theta=10000.0):
    pos = np.arange(t_max, dtype=np.float64)[:, None]
    inv = 1.0 / (theta ** (2.0 * np.arange(dh // 2, dtype=np.float64) / dh))
    ang = pos * inv[None, :]
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


# tests/correctness/store.rs: fused rope / scatter / rope+scatter stores equal the standalone ops
def test_fused_stores(gpu, orc):
    ta, ctx, ex = gpu
    k, heads, kv_heads, dh, t_max, pos = 2048, 32, 4, 64, 96, 37
    x, hx = upload_det(ta, ctx, ex, orc, (1, k), 550)
    table_h = rope_table(t_max, dh)
    table = ta.Tensor.uninit_device(ctx, table_h.shape)
    ex.upload(table_h, table)
    cell = ta.PosCell(ctx)
    cell.set(pos)
    assert cell.get() == pos
    # q: rope -> C
    wq, hwq = make_weights(ta, ctx, ex, orc, k, heads * dh, 551, True)
    q = ta.Tensor.uninit_device(ctx, (1, heads * dh))
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, wq, q), packed_b=True,
                                 store=ta.MatmulStore(ta.StoreKind.ROPE, head_dim=dh, table=table, pos_cell=cell))])
    plain = orc.cpu_bmm(hx, hwq, 1, 1, heads * dh, k)
    ref = orc.cpu_rope(plain, table_h, 1, heads, dh, dh, pos)
    check(orc, ex.download(q), ref, k, "rope store")
    # k: rope + scatter into Kt [H_kv, dh, T_max] (f16 cache), position from pos_base
    wk, hwk = make_weights(ta, ctx, ex, orc, k, kv_heads * dh, 552, True)
    kt = ta.Tensor.uninit_device_f16(ctx, (kv_heads, dh, t_max))
    ex.upload(np.zeros(kv_heads * dh * t_max, np.float32), kt)
    dummy = ta.Tensor.uninit_device(ctx, (1, kv_heads * dh))
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, wk, dummy), packed_b=True,
                                 store=ta.MatmulStore(ta.StoreKind.ROPE_SCATTER, head_dim=dh, pos_base=pos,
                                                      pos_scale=1, stride_head=dh * t_max, stride_dim=t_max,
                                                      table=table, dst=kt))])
    kref = orc.cpu_rope(orc.cpu_bmm(hx, hwk, 1, 1, kv_heads * dh, k), table_h, 1, kv_heads, dh, dh, pos)
    got = ex.download(kt).reshape(kv_heads, dh, t_max)
    assert (np.delete(got, pos, axis=2) == 0).all()
    want = orc.round_via_f16(kref).reshape(kv_heads, dh)
    assert np.abs(got[:, :, pos] - want).max() <= np.abs(want).max() / 1024
    # v: scatter into V [H_kv, T_max, dh] (f32 cache) with position from the cell
    wv, hwv = make_weights(ta, ctx, ex, orc, k, kv_heads * dh, 553, True)
    v = ta.Tensor.uninit_device(ctx, (kv_heads, t_max, dh))
    ex.upload(np.zeros(kv_heads * dh * t_max, np.float32), v)
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, wv, dummy), packed_b=True,
                                 store=ta.MatmulStore(ta.StoreKind.SCATTER, head_dim=dh, pos_scale=dh,
                                                      stride_head=t_max * dh, stride_dim=1, dst=v, pos_cell=cell))])
    vref = orc.cpu_bmm(hx, hwv, 1, 1, kv_heads * dh, k).reshape(kv_heads, dh)
    got = ex.download(v).reshape(kv_heads, t_max, dh)
    assert (np.delete(got, pos, axis=1) == 0).all()
    check(orc, got[:, pos, :], vref, k, "scatter store")


def test_fused_store_position_outside_the_cache_is_reported_not_written(gpu, orc):
    """A position cell beyond the scatter destination: nothing is stored, the call fails with the
    position message, and the same op with a valid position works afterwards."""
    ta, ctx, ex = gpu
    k, kv_heads, dh, t_max = 512, 2, 64, 32
    x, hx = upload_det(ta, ctx, ex, orc, (1, k), 560)
    wv, hwv = make_weights(ta, ctx, ex, orc, k, kv_heads * dh, 561, True)
    v = ta.Tensor.uninit_device(ctx, (kv_heads, t_max, dh))
    ex.upload(np.zeros(kv_heads * dh * t_max, np.float32), v)
    dummy = ta.Tensor.uninit_device(ctx, (1, kv_heads * dh))
    cell = ta.PosCell(ctx)
    op = ta.MatmulOpEx(ta.MatmulCall(x, wv, dummy), packed_b=True,
                       store=ta.MatmulStore(ta.StoreKind.SCATTER, head_dim=dh, pos_scale=dh,
                                            stride_head=t_max * dh, stride_dim=1, dst=v, pos_cell=cell))
    cell.set(t_max)                       # first position the destination does not hold
    with pytest.raises(ta.TensorAshError, match="position cell"):
        ex.run_ops_ex([op])
    assert (ex.download(v) == 0).all()
    cell.set(t_max - 1)
    ex.run_ops_ex([op])
    got = ex.download(v).reshape(kv_heads, t_max, dh)
    assert (got[:, : t_max - 1, :] == 0).all()
    check(orc, got[:, t_max - 1, :], orc.cpu_bmm(hx, hwv, 1, 1, kv_heads * dh, k).reshape(kv_heads, dh), k, "scatter at the last position")


# src/matmul/resolution.rs:176-313 validation
def test_rejections(gpu, orc):
    ta, ctx, ex = gpu
    E = ta.TensorAshError
    x = ta.Tensor.uninit_device(ctx, (1, 64))
    w32 = ta.Tensor.uninit_device(ctx, (64, 64))
    w16 = ta.Tensor.uninit_device_f16(ctx, (64, 64))
    w48 = ta.Tensor.uninit_device_f16(ctx, (64, 48))
    c = ta.Tensor.uninit_device(ctx, (1, 64))
    c48 = ta.Tensor.uninit_device(ctx, (1, 48))
    bias = ta.Tensor.uninit_device(ctx, (64,))
    nw = ta.Tensor.uninit_device(ctx, (64,))
    with pytest.raises(E, match="requires f16 weights"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w32, c), packed_b=True)])
    with pytest.raises(E, match="multiple of 32"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w48, c48), packed_b=True)])
    x16 = ta.Tensor.uninit_device(ctx, (16, 64))
    c16 = ta.Tensor.uninit_device(ctx, (16, 64))
    with pytest.raises(E, match="packed-B GEMV requires M"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x16, w16, c16), packed_b=True)])
    with pytest.raises(E, match="bias slot"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w16, c), ta.Epilogue(bias=bias), normed_a=(nw, 1e-5))])
    with pytest.raises(E, match="both use beta"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w16, c), ta.Epilogue(binary=ta.Binary.ADD_SCALED, d=ta.Tensor.uninit_device(ctx, (1, 64)), beta=1.0),
                                     normed_a=(nw, 1e-5))])
    with pytest.raises(E, match="must equal K"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w16, c), normed_a=(ta.Tensor.uninit_device(ctx, (63,)), 1e-5))])
    st = ta.MatmulStore(ta.StoreKind.SCATTER, head_dim=64, pos_base=5, pos_scale=64, stride_head=0, stride_dim=1,
                        dst=ta.Tensor.uninit_device(ctx, (4, 64)))
    with pytest.raises(E, match="out of bounds"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w16, c), store=st)])
    with pytest.raises(E, match="cannot combine with accumulate"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w16, c, 1.0, True),
                                     store=ta.MatmulStore(ta.StoreKind.SCATTER, head_dim=64, dst=c))])
    with pytest.raises(E, match="requires M == 1"):
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x16, w16, c16),
                                     store=ta.MatmulStore(ta.StoreKind.SCATTER, head_dim=64, dst=c16))])


# ---- 3..8 rows: the tensor-memory kernel (tcgen05 with the weights as the A operand)
@pytest.mark.parametrize("k,n,packed", [(2048, 2048, True), (2048, 5632, True), (5632, 2048, False), (4096, 1024, True),
                                        (1008, 200, False), (64, 32, True), (16384, 64, True), (2048, 32000, True),
                                        (11008, 4096, True), (80, 136, False)])
def test_umma_rows_match_the_oracle(gpu, orc, k, n, packed):
    """Packed tiles of 32 and 64, row-major weights, column counts that leave partial groups, K that is
    not a multiple of the ring's 64-row box, K long enough for many K slices."""
    ta, ctx, ex = gpu
    for m in (3, 5, 8):
        x, hx = upload_det(ta, ctx, ex, orc, (m, k), 560 + m)
        w, hw = make_weights(ta, ctx, ex, orc, k, n, 561, packed)
        c = ta.Tensor.uninit_device(ctx, (m, n))
        ex.upload(np.full(m * n, 9.0, np.float32), c)
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c), packed_b=packed)])
        first = ex.download(c).copy()
        check(orc, first, orc.cpu_bmm(hx, hw, 1, m, n, k), k, f"{m}x{n}x{k} packed={packed}")
        ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c), packed_b=packed)])
        assert ex.download(c).tobytes() == first.tobytes(), "two runs differ"


def test_umma_rows_full_epilogue_and_accumulate(gpu, orc):
    """alpha, accumulate, bias, GELU and AddScaled in one op; then normed-A with SiLU * Mul (the fused
    RMSNorm statistic is summed over the K slices of several CTAs)."""
    ta, ctx, ex = gpu
    m, k, n = 6, 4096, 1536
    x, hx = upload_det(ta, ctx, ex, orc, (m, k), 570)
    w, hw = make_weights(ta, ctx, ex, orc, k, n, 571, True)
    bias, hb = upload_det(ta, ctx, ex, orc, (n,), 572)
    d, hd = upload_det(ta, ctx, ex, orc, (m, n), 573)
    c, hc = upload_det(ta, ctx, ex, orc, (m, n), 574)
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c, 0.5, True),
                                 ta.Epilogue(bias, ta.Activation.GELU, ta.Binary.ADD_SCALED, d, 0.25), packed_b=True)])
    ref = orc.cpu_epilogue(orc.cpu_bmm(hx, hw, 1, m, n, k, alpha=0.5, c_init=hc, accumulate=True), 1, m, n,
                           bias=hb, act="gelu", binary="add_scaled", d=hd, beta=0.25)
    check(orc, ex.download(c), ref, k, "alpha + accumulate + bias + gelu + add_scaled")
    nw = ta.Tensor.uninit_device(ctx, (k,))
    hnw = 1.0 + 0.1 * orc.fill_det(k, 575)
    ex.upload(hnw, nw)
    ex.run_ops_ex([ta.MatmulOpEx(ta.MatmulCall(x, w, c), ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=d),
                                 packed_b=True, normed_a=(nw, 1e-5))])
    xn = orc.cpu_rmsnorm(hx.reshape(m, k), hnw, 1e-5)
    ref = orc.cpu_epilogue(orc.cpu_bmm(xn, hw, 1, m, n, k), 1, m, n, act="silu", binary="mul", d=hd)
    check(orc, ex.download(c), ref, k, "normed-A silu*mul M=6")


def test_umma_rows_take_any_activation_range(gpu, orc):
    """The f16 split of x is taken after a per-row power-of-two scaling of each K slice, so rows with
    huge, tiny and mixed magnitudes all keep about 22 bits: no activation range is excluded."""
    ta, ctx, ex = gpu
    m, k, n = 8, 2048, 256
    hx = orc.fill_det(m * k, 580).reshape(m, k).astype(np.float32)
    hx[0] *= 1.0e6          # far beyond the f16 range
    hx[1] *= 1.0e-9         # far below the f16 normal range
    hx[2, 17] = 1.0e5       # one outlier in an ordinary row
    hx[3] = 0.0
    x = ta.Tensor.uninit_device(ctx, (m, k))
    ex.upload(hx.ravel(), x)
    w, hw = make_weights(ta, ctx, ex, orc, k, n, 581, False)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    ex.run_matmuls([ta.MatmulCall(x, w, c)])
    got = ex.download(c).reshape(m, n)
    ref = orc.cpu_bmm(hx, hw, 1, m, n, k).reshape(m, n)
    for row in range(m):
        scale = max(float(np.abs(ref[row]).max()), 1e-30)
        assert np.abs(got[row] - ref[row]).max() <= 2e-3 * scale, f"row {row}"
    assert not got[3].any()
