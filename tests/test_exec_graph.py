"""Mixed graphs: the ops the llama graphs use beside matmuls (binary, argmax,
embedding gathers, RoPE + scatter, f32 -> f16 strided copies) one by one against
numpy, then a prepared mixed graph replayed with a moving position cell.
Mirrors the reference's tests/attn_decode.rs + tools/llama-ash graph tests in
structure: each op alone, then the composed graph against the composed host model.
"""
import numpy as np
import pytest


def up(ta, ctx, ex, arr):
    t = ta.Tensor.uninit_device(ctx, list(arr.shape))
    ex.upload(np.ascontiguousarray(arr, dtype=np.float32).ravel(), t)
    return t


def rope_table(t_max, half, theta=1e4):
    p = np.arange(t_max, dtype=np.float64)[:, None]
    i = np.arange(half, dtype=np.float64)[None, :]
    ang = p / np.power(theta, 2.0 * i / (2 * half))
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def rope_host(x, table, heads, dh, pos0):
    t = x.shape[0]
    xh = x.reshape(t, heads, dh // 2, 2).astype(np.float64)
    cs = table[pos0:pos0 + t].astype(np.float64)[:, None]
    a, b = xh[..., 0], xh[..., 1]
    return np.stack([a * cs[..., 0] - b * cs[..., 1], a * cs[..., 1] + b * cs[..., 0]], -1).reshape(t, heads * dh)


@pytest.mark.gpu
def test_binary_ops(gpu, orc):
    ta, ctx, ex = gpu
    a = orc.fill_det(5 * 333, 1).reshape(5, 333)
    b = orc.fill_det(5 * 333, 2).reshape(5, 333)
    ta_, tb = up(ta, ctx, ex, a), up(ta, ctx, ex, b)
    out = ta.Tensor.uninit_device(ctx, [5, 333])
    ex.run_exec_ops([ta.ExecOp.binary_add_scaled(ta_, tb, out, 0.5)])
    want = (a.astype(np.float32) + np.float32(0.5) * b.astype(np.float32))
    np.testing.assert_allclose(ex.download(out).reshape(5, 333), want, rtol=1e-6, atol=1e-7)
    ex.run_exec_ops([ta.ExecOp.binary_silu_mul(ta_, tb, out)])
    a64 = a.astype(np.float64)
    want = a64 / (1 + np.exp(-a64)) * b
    np.testing.assert_allclose(ex.download(out).reshape(5, 333), want, rtol=2e-6, atol=1e-7)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 7, 1000, 32000, 151936])
def test_argmax_ties_keep_the_largest_index(gpu, orc, n):
    ta, ctx, ex = gpu
    x = orc.fill_det(n, 40 + n % 7).copy()
    if n > 10:
        # duplicate maximum: the larger index wins (shaders/op_argmax_f32.comp:44-75)
        x[n // 3] = 5.0
        x[n - 2] = 5.0
    t = up(ta, ctx, ex, x.reshape(1, n))
    cell = ta.PosCell(ctx)
    cell.set(0xFFFFFFFF)
    ex.run_exec_ops([ta.ExecOp.argmax(t, cell)])
    want = int(np.flatnonzero(x == x.max())[-1])
    assert cell.get() == want


@pytest.mark.gpu
@pytest.mark.parametrize("embd", [160, 1030, 2048])      # 1030: rows off the 4-column vector path
def test_embed_gather_f16_and_f32_tables(gpu, orc, embd):
    ta, ctx, ex = gpu
    vocab = 97
    tab = orc.fill_det(vocab * embd, 9).reshape(vocab, embd)
    t32 = up(ta, ctx, ex, tab)
    t16 = ta.Tensor.uninit_device_f16(ctx, [vocab, embd])
    ex.upload(tab.ravel(), t16)
    tab16 = tab.astype(np.float16).astype(np.float32)
    cell = ta.PosCell(ctx)
    out = ta.Tensor.uninit_device(ctx, [1, embd])
    for tok in (0, 42, vocab - 1):
        cell.set(tok)
        ex.run_exec_ops([ta.ExecOp.embed_gather(cell, t32, out)])
        np.testing.assert_array_equal(ex.download(out).ravel(), tab[tok])
        ex.run_exec_ops([ta.ExecOp.embed_gather(cell, t16, out)])
        np.testing.assert_array_equal(ex.download(out).ravel(), tab16[tok])
    ids = ta.TokenIdBuffer(ctx, 16)
    toks = [3, 96, 0, 3, 50]
    ids.set(toks)
    rows = ta.Tensor.uninit_device(ctx, [len(toks), embd])
    ex.run_exec_ops([ta.ExecOp.embed_gather_rows(ids, t16, rows)])
    np.testing.assert_array_equal(ex.download(rows).reshape(len(toks), embd), tab16[toks])
    # an id beyond the table is clamped to the last row, so a bad id can never read out of bounds
    ids.set([1, vocab + 5])
    rows2 = ta.Tensor.uninit_device(ctx, [2, embd])
    ex.run_exec_ops([ta.ExecOp.embed_gather_rows(ids, t16, rows2)])
    np.testing.assert_array_equal(ex.download(rows2).reshape(2, embd), tab16[[1, vocab - 1]])


@pytest.mark.gpu
@pytest.mark.parametrize("dst_f16", [False, True])
def test_rope_scatter_into_transposed_cache(gpu, orc, dst_f16):
    ta, ctx, ex = gpu
    heads, dh, t_max, t, pos0 = 2, 64, 24, 5, 7
    x = orc.fill_det(t * heads * dh, 3).reshape(t, heads * dh)
    table = rope_table(t_max, dh // 2)
    tx, tt = up(ta, ctx, ex, x), up(ta, ctx, ex, table)
    mk = ta.Tensor.uninit_device_f16 if dst_f16 else ta.Tensor.uninit_device
    kt = mk(ctx, [heads, dh, t_max])
    zero = np.zeros(heads * dh * t_max, dtype=np.float32)
    ex.upload(zero, kt)
    # Kt[h, d, p]: token stride 1, head stride dh*t_max, dim stride t_max
    ex.run_exec_ops([ta.ExecOp.rope_scatter(tx, tt, kt, heads, dh, dh, pos0, pos0, [1, dh * t_max, t_max])])
    got = ex.download(kt).reshape(heads, dh, t_max)
    want = np.zeros((heads, dh, t_max))
    want[:, :, pos0:pos0 + t] = rope_host(x, table, heads, dh, pos0).reshape(t, heads, dh).transpose(1, 2, 0)
    if dst_f16:
        np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-6)
        assert np.array_equal(got[:, :, :pos0], np.zeros((heads, dh, pos0)))
    else:
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-7)


@pytest.mark.gpu
def test_copy_strided_f32_to_f16_rounds_to_nearest_even(gpu, orc):
    ta, ctx, ex = gpu
    t, kv, dh, t_max = 6, 2, 64, 16
    v = orc.fill_det(t * kv * dh, 5).reshape(t, kv * dh)
    tv = up(ta, ctx, ex, v)
    cache = ta.Tensor.uninit_device_f16(ctx, [kv, t_max, dh])
    ex.upload(np.zeros(kv * t_max * dh, dtype=np.float32), cache)
    pos0 = 3
    ex.run_exec_ops([ta.ExecOp.copy_strided(tv, cache, [dh, kv, t], 0, [1, dh, kv * dh], pos0 * dh,
                                            [1, t_max * dh, dh])])
    got = ex.download(cache).reshape(kv, t_max, dh)
    want = np.zeros((kv, t_max, dh), dtype=np.float32)
    want[:, pos0:pos0 + t] = v.astype(np.float16).astype(np.float32).reshape(t, kv, dh).transpose(1, 0, 2)
    np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("kv_f16", [False, True])
def test_prefill_qkv_pack_equals_the_composed_split_rope_and_cache_writes(gpu, orc, kv_f16):
    """One launch against the seven-op composition it replaces (three strided splits, two
    RoPE passes, two cache copies): bit-identical q and caches, and both against numpy."""
    ta, ctx, ex = gpu
    heads, kv, dh, t_max, t, pos0 = 4, 2, 64, 40, 9, 11
    q_w, kv_w = heads * dh, kv * dh
    n_qkv = q_w + 2 * kv_w
    qkv = orc.fill_det(t * n_qkv, 17).reshape(t, n_qkv)
    table = rope_table(t_max, dh // 2)
    tqkv, tt = up(ta, ctx, ex, qkv), up(ta, ctx, ex, table)
    mk = ta.Tensor.uninit_device_f16 if kv_f16 else ta.Tensor.uninit_device

    def caches():
        kt, v = mk(ctx, [kv, dh, t_max]), mk(ctx, [kv, t_max, dh])
        ex.upload(np.zeros(kv * dh * t_max, dtype=np.float32), kt)
        ex.upload(np.zeros(kv * dh * t_max, dtype=np.float32), v)
        return kt, v

    kt1, v1 = caches()
    q1 = ta.Tensor.uninit_device(ctx, [heads, t, dh])
    ex.run_exec_ops([ta.ExecOp.prefill_qkv_pack(tqkv, tt, q1, kt1, v1, heads, kv, dh, dh, pos0)])

    kt2, v2 = caches()
    q2 = ta.Tensor.uninit_device(ctx, [t, q_w])
    k2 = ta.Tensor.uninit_device(ctx, [t, kv_w])
    vv2 = ta.Tensor.uninit_device(ctx, [t, kv_w])
    E = ta.ExecOp
    ex.run_exec_ops([
        E.copy_strided(tqkv, q2, [q_w, t, 1], 0, [1, n_qkv, 0], 0, [1, q_w, 0]),
        E.copy_strided(tqkv, k2, [kv_w, t, 1], q_w, [1, n_qkv, 0], 0, [1, kv_w, 0]),
        E.copy_strided(tqkv, vv2, [kv_w, t, 1], q_w + kv_w, [1, n_qkv, 0], 0, [1, kv_w, 0]),
        E.rope(q2, tt, q2, heads, dh, dh, pos0),
        E.rope(k2, tt, k2, kv, dh, dh, pos0),
        E.copy_strided(k2, kt2, [dh, kv, t], 0, [1, dh, kv * dh], pos0, [t_max, dh * t_max, 1]),
        E.copy_strided(vv2, v2, [dh, kv, t], 0, [1, dh, kv * dh], pos0 * dh, [1, t_max * dh, dh]),
    ])
    got_q = ex.download(q1).reshape(heads, t, dh)
    np.testing.assert_array_equal(got_q, ex.download(q2).reshape(t, heads, dh).transpose(1, 0, 2))
    np.testing.assert_array_equal(ex.download(kt1).ravel(), ex.download(kt2).ravel())
    np.testing.assert_array_equal(ex.download(v1).ravel(), ex.download(v2).ravel())

    want_q = rope_host(qkv[:, :q_w], table, heads, dh, pos0).reshape(t, heads, dh).transpose(1, 0, 2)
    np.testing.assert_allclose(got_q, want_q, rtol=2e-6, atol=2e-7)
    want_k = np.zeros((kv, dh, t_max))
    want_k[:, :, pos0:pos0 + t] = rope_host(qkv[:, q_w:q_w + kv_w], table, kv, dh, pos0).reshape(t, kv, dh).transpose(1, 2, 0)
    tol = dict(rtol=1e-3, atol=1e-6) if kv_f16 else dict(rtol=2e-6, atol=2e-7)
    np.testing.assert_allclose(ex.download(kt1).reshape(kv, dh, t_max), want_k, **tol)
    want_v = np.zeros((kv, t_max, dh), dtype=np.float32)
    vsrc = qkv[:, q_w + kv_w:]
    if kv_f16:
        vsrc = vsrc.astype(np.float16).astype(np.float32)
    want_v[:, pos0:pos0 + t] = vsrc.reshape(t, kv, dh).transpose(1, 0, 2)
    np.testing.assert_array_equal(ex.download(v1).reshape(kv, t_max, dh), want_v)


@pytest.mark.gpu
def test_prefill_qkv_pack_rejects_inconsistent_shapes(gpu, orc):
    ta, ctx, ex = gpu
    heads, kv, dh, t_max, t = 4, 2, 64, 16, 4
    n_qkv = (heads + 2 * kv) * dh
    tqkv = up(ta, ctx, ex, np.zeros((t, n_qkv)))
    tt = up(ta, ctx, ex, rope_table(t_max, dh // 2))
    q = ta.Tensor.uninit_device(ctx, [heads, t, dh])
    kt, v = ta.Tensor.uninit_device(ctx, [kv, dh, t_max]), ta.Tensor.uninit_device(ctx, [kv, t_max, dh])
    with pytest.raises(ta.TensorAshError):   # positions run past the cache
        ex.run_exec_ops([ta.ExecOp.prefill_qkv_pack(tqkv, tt, q, kt, v, heads, kv, dh, dh, t_max - t + 1)])
    with pytest.raises(ta.TensorAshError):   # row width does not match the head counts
        ex.run_exec_ops([ta.ExecOp.prefill_qkv_pack(tqkv, tt, q, kt, v, heads, kv + 1, dh, dh, 0)])


@pytest.mark.gpu
def test_prepared_mixed_graph_replays_with_position_cell(gpu, orc):
    """norm -> matmul(+rope scatter store through the cell) -> argmax -> gather, replayed at
    three positions from one recording."""
    ta, ctx, ex = gpu
    embd, heads, dh, t_max, vocab = 128, 2, 64, 12, 128
    x = orc.fill_det(embd, 21).reshape(1, embd)
    w = orc.fill_det(embd * heads * dh, 22).reshape(embd, heads * dh)
    nw = 1.0 + 0.1 * orc.fill_det(embd, 23)
    table = rope_table(t_max, dh // 2)
    emb = orc.fill_det(vocab * embd, 24).reshape(vocab, embd)
    tx, tw, tnw, tt, temb = (up(ta, ctx, ex, a) for a in (x, w, nw.reshape(embd), table, emb))
    xn = ta.Tensor.uninit_device(ctx, [1, embd])
    y = ta.Tensor.uninit_device(ctx, [1, heads * dh])
    kt = ta.Tensor.uninit_device(ctx, [heads, dh, t_max])
    ex.upload(np.zeros(heads * dh * t_max, dtype=np.float32), kt)
    nxt = ta.Tensor.uninit_device(ctx, [1, embd])
    pos, tok = ta.PosCell(ctx), ta.PosCell(ctx)
    ops = [
        ta.ExecOp.rms_norm(tx, tnw, xn, 1e-5),
        ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(xn, tw, y))),
        ta.ExecOp.rope_scatter(y, tt, kt, heads, dh, dh, 0, 0, [1, dh * t_max, t_max], pos_scale=1, cell=pos),
        ta.ExecOp.argmax(y, tok),
        ta.ExecOp.embed_gather(tok, temb, nxt),
    ]
    pos.set(0)
    prepared = ex.prepare_exec_ops(ops)
    x64 = x.astype(np.float64)
    xn_h = x64 / np.sqrt((x64 * x64).mean() + 1e-5) * nw
    y_h = xn_h @ w.astype(np.float64)
    want = np.zeros((heads, dh, t_max))
    for p in (0, 4, 11):
        pos.set(p)
        st = prepared.run()
        assert st.n_calls >= 1
        want[:, :, p] = rope_host(y_h, table, heads, dh, p).reshape(heads, dh)
        assert tok.get() == int(np.argmax(y_h))
        np.testing.assert_array_equal(ex.download(nxt).ravel(), emb[tok.get()])
    got = ex.download(kt).reshape(heads, dh, t_max)
    np.testing.assert_allclose(got, want, rtol=3e-5, atol=3e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(128, 512, 256), (200, 1024, 384)])
def test_norm_then_f16w_gemm_in_one_graph_equals_the_ops_run_apart(gpu, orc, m, k, n):
    """In one submission the planner lets the RMSNorm also write its output rounded to f16 where the
    tensor-core GEMM behind it expects the f16 copy of its A (the conversion launch disappears); run
    apart, the GEMM converts for itself.  Same f32 values rounded the same way: bit-identical C."""
    ta, ctx, ex = gpu
    rng = np.random.default_rng(811)
    x = rng.standard_normal((m, k), dtype=np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    w = (rng.standard_normal((k, n), dtype=np.float32) * 0.05).astype(np.float16)
    tx, tnw = ta.Tensor.uninit_device(ctx, (m, k)), ta.Tensor.uninit_device(ctx, (k,))
    xn = ta.Tensor.uninit_device(ctx, (m, k))
    tw = ta.Tensor.uninit_device_f16(ctx, (k, n))
    c1, c2 = ta.Tensor.uninit_device(ctx, (m, n)), ta.Tensor.uninit_device(ctx, (m, n))
    ex.upload(x, tx)
    ex.upload(nw, tnw)
    ex.upload_f16(w.view(np.uint16), tw)
    before = ta.kernel_launch_count()
    ex.run_exec_ops([ta.ExecOp.rms_norm(tx, tnw, xn, 1e-5), ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(xn, tw, c1)))])
    fused_launches = ta.kernel_launch_count() - before
    xn_fused = ex.download(xn).copy()
    before = ta.kernel_launch_count()
    ex.run_exec_ops([ta.ExecOp.rms_norm(tx, tnw, xn, 1e-5)])
    ex.run_exec_ops([ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(xn, tw, c2)))])
    apart_launches = ta.kernel_launch_count() - before
    assert fused_launches == apart_launches - 1          # norm + GEMM against norm + conversion + GEMM
    assert np.array_equal(xn_fused.view(np.uint32), ex.download(xn).view(np.uint32))
    assert np.array_equal(ex.download(c1).view(np.uint32), ex.download(c2).view(np.uint32))
    ref = (xn_fused.astype(np.float64) @ w.astype(np.float64))
    assert np.abs(ex.download(c1) - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())


@pytest.mark.gpu
def test_flash_then_f16w_gemm_in_one_graph_equals_the_ops_run_apart(gpu, orc):
    """The token-major output of the tensor-core flash kernel also lands as the f16 A of the
    projection behind it; bit-identical to attention and projection run as two submissions."""
    ta, ctx, ex = gpu
    heads, kv_heads, t, t_max, dh, n = 8, 2, 96, 128, 64, 320
    rng = np.random.default_rng(812)
    q = rng.standard_normal((heads, t, dh), dtype=np.float32)
    kt = (rng.standard_normal((kv_heads, dh, t_max), dtype=np.float32)).astype(np.float16)
    v = (rng.standard_normal((kv_heads, t_max, dh), dtype=np.float32)).astype(np.float16)
    w = (rng.standard_normal((heads * dh, n), dtype=np.float32) * 0.05).astype(np.float16)
    tq = ta.Tensor.uninit_device(ctx, q.shape)
    tkt, tv = ta.Tensor.uninit_device_f16(ctx, kt.shape), ta.Tensor.uninit_device_f16(ctx, v.shape)
    tw = ta.Tensor.uninit_device_f16(ctx, w.shape)
    attn = ta.Tensor.uninit_device(ctx, (t, heads * dh))
    c1, c2 = ta.Tensor.uninit_device(ctx, (t, n)), ta.Tensor.uninit_device(ctx, (t, n))
    ex.upload(q, tq)
    ex.upload_f16(kt.view(np.uint16), tkt)
    ex.upload_f16(v.view(np.uint16), tv)
    ex.upload_f16(w.view(np.uint16), tw)
    flash = ta.ExecOp.flash_attn(tq, tkt, tv, attn, t, 0, 0.125, out_token_major_heads=heads)
    before = ta.kernel_launch_count()
    ex.run_exec_ops([flash, ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(attn, tw, c1)))])
    fused_launches = ta.kernel_launch_count() - before
    attn_fused = ex.download(attn).copy()
    before = ta.kernel_launch_count()
    ex.run_exec_ops([flash])
    ex.run_exec_ops([ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(attn, tw, c2)))])
    assert fused_launches == ta.kernel_launch_count() - before - 1
    assert np.array_equal(attn_fused.view(np.uint32), ex.download(attn).view(np.uint32))
    assert np.array_equal(ex.download(c1).view(np.uint32), ex.download(c2).view(np.uint32))
    assert np.isfinite(ex.download(c1)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(512, 2048, 5632), (200, 512, 320), (128, 256, 64)])
def test_up_then_gated_gemm_in_one_graph_equals_the_ops_run_apart(gpu, orc, m, k, n):
    """`up = A Wu` followed by `gate = silu(A Wg) * up` on the f16-weight tensor-core route becomes one
    dual-matrix launch in a graph: every output element goes through the same MMA sequence and the
    same epilogue formulas as in the two launches, so both outputs are bit-identical to the ops run
    as two submissions (incl. partial row tiles and a last partial column tile)."""
    ta, ctx, ex = gpu
    rng = np.random.default_rng(813)
    a = rng.standard_normal((m, k), dtype=np.float32)
    wu = (rng.standard_normal((k, n), dtype=np.float32) * 0.05).astype(np.float16)
    wg = (rng.standard_normal((k, n), dtype=np.float32) * 0.05).astype(np.float16)
    ta_a = ta.Tensor.uninit_device(ctx, (m, k))
    twu, twg = ta.Tensor.uninit_device_f16(ctx, (k, n)), ta.Tensor.uninit_device_f16(ctx, (k, n))
    up1, g1 = ta.Tensor.uninit_device(ctx, (m, n)), ta.Tensor.uninit_device(ctx, (m, n))
    up2, g2 = ta.Tensor.uninit_device(ctx, (m, n)), ta.Tensor.uninit_device(ctx, (m, n))
    ex.upload(a, ta_a)
    ex.upload_f16(wu.view(np.uint16), twu)
    ex.upload_f16(wg.view(np.uint16), twg)

    def ops(up, gate):
        return [ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(ta_a, twu, up))),
                ta.ExecOp.matmul(ta.MatmulOp(ta.MatmulCall(ta_a, twg, gate),
                                             ta.Epilogue(activation=ta.Activation.SILU, binary=ta.Binary.MUL, d=up)))]
    before = ta.kernel_launch_count()
    ex.run_exec_ops(ops(up1, g1))
    fused = ta.kernel_launch_count() - before
    first, second = ops(up2, g2)
    before = ta.kernel_launch_count()
    ex.run_exec_ops([first])
    ex.run_exec_ops([second])
    apart = ta.kernel_launch_count() - before
    assert fused == 2 and apart == 4                    # conversion + dual GEMM against 2 x (conversion + GEMM)
    assert np.array_equal(ex.download(up1).view(np.uint32), ex.download(up2).view(np.uint32))
    assert np.array_equal(ex.download(g1).view(np.uint32), ex.download(g2).view(np.uint32))
    u = a.astype(np.float64) @ wu.astype(np.float64)
    z = a.astype(np.float64) @ wg.astype(np.float64)
    ref = z / (1.0 + np.exp(-z)) * u
    assert np.abs(ex.download(g1) - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
