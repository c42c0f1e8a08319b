"""GPU parity tests of the fused attention kernels against the f64 oracle
(tests/correctness/flash.rs and attn_decode.rs in the reference: same cases,
cache fill, poison tails and the 1e-4 absolute tolerance)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4
# f16 caches with head dim 64 and >= 32 query rows take the tensor-core kernel, which rounds Q*scale
# and the softmax weights through f16 (the reference's coopmat2 route; its own bound is 2e-2,
# tests/correctness/flash.rs:481-485).  Measured here well inside 4e-3.
MMA_TOL = 4e-3


def takes_mma(kv16, dh, t_q, t_max):
    return kv16 and dh == 64 and t_q >= 32 and t_max % 8 == 0


def fill_kv(orc, kv_heads, t_max, dh, kv_len, poison=None, seed=5101):
    """tests/correctness/flash.rs:74-105"""
    n = kv_heads * dh * t_max
    fill = orc.fill_det(n, seed)
    kt = np.zeros((kv_heads, dh, t_max), np.float32)
    v = np.zeros((kv_heads, t_max, dh), np.float32)
    kt_idx = np.arange(n).reshape(kv_heads, dh, t_max)
    v_idx = np.arange(n).reshape(kv_heads, t_max, dh)
    kt[:] = fill[kt_idx % n]
    v[:] = fill[(v_idx * 7 + 3) % n]
    tail = np.arange(t_max) >= kv_len
    fillv = 0.0 if poison is None else poison
    kt[:, :, tail] = fillv
    v[:, tail, :] = fillv
    return kt, v


def upload(ta, ctx, ex, host, f16=False):
    t = (ta.Tensor.uninit_device_f16 if f16 else ta.Tensor.uninit_device)(ctx, host.shape)
    ex.upload(host, t)
    return t


FLASH_CASES = [  # heads, kv_heads, t_q, t_max, dh, kv_len, pos_base
    (4, 4, 64, 64, 64, 64, 0), (8, 2, 100, 160, 64, 100, 0), (32, 4, 200, 256, 64, 200, 0),
    (4, 2, 37, 128, 64, 77, 40), (2, 1, 130, 256, 128, 130, 0), (4, 4, 16, 64, 64, 10, 0),
    (8, 8, 65, 96, 128, 65, 0),
]


@pytest.mark.parametrize("case", FLASH_CASES)
@pytest.mark.parametrize("kv16", [False, True])
def test_flash_prefill(gpu, orc, case, kv16):
    ta, ctx, ex = gpu
    heads, kv_heads, t_q, t_max, dh, kv_len, pos_base = case
    scale = 1.0 / np.sqrt(dh)
    poison = 6e4 if kv16 else 1e30                      # masking must never read past kv_len
    kt_h, v_h = fill_kv(orc, kv_heads, t_max, dh, kv_len, poison)
    if kv16:
        kt_h, v_h = orc.round_via_f16(kt_h), orc.round_via_f16(v_h)
    q_h = orc.fill_det(heads * t_q * dh, 5102).reshape(heads, t_q, dh)
    q, kt, v = upload(ta, ctx, ex, q_h), upload(ta, ctx, ex, kt_h, kv16), upload(ta, ctx, ex, v_h, kv16)
    out = ta.Tensor.uninit_device(ctx, (heads, t_q, dh))
    ex.upload(np.zeros(heads * t_q * dh, np.float32), out)
    ex.run_flash_attention(q, kt, v, out, kv_len, pos_base, scale)
    ref = orc.cpu_flash(q_h, kt_h, v_h, heads, kv_heads, t_q, dh, t_max, kv_len, pos_base, scale)
    got = ex.download(out).reshape(-1)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= (MMA_TOL if takes_mma(kv16, dh, t_q, t_max) else TOL)
    if takes_mma(kv16, dh, t_q, t_max):
        # the f32-operand kernel stays available and keeps its tolerance
        out32 = ta.Tensor.uninit_device(ctx, (heads, t_q, dh))
        ex.upload(np.zeros(heads * t_q * dh, np.float32), out32)
        ex.run_flash_attention(q, kt, v, out32, kv_len, pos_base, scale, simt=True)
        assert np.abs(ex.download(out32).reshape(-1) - ref).max() <= TOL
    # token-major q and out: [T, H*dh]
    q_tm = upload(ta, ctx, ex, np.ascontiguousarray(q_h.transpose(1, 0, 2)).reshape(t_q, heads * dh))
    out_tm = ta.Tensor.uninit_device(ctx, (t_q, heads * dh))
    ex.run_flash_attention(q_tm, kt, v, out_tm, kv_len, pos_base, scale, token_major_heads=heads)
    got_tm = ex.download(out_tm).reshape(t_q, heads, dh).transpose(1, 0, 2).reshape(-1)
    assert (got_tm == got).all()                         # graph/layout variants are bitwise equal
    # head-major q, token-major out (the wide-prefill form)
    ex.upload(np.zeros(heads * t_q * dh, np.float32), out_tm)
    ex.run_flash_attention(q, kt, v, out_tm, kv_len, pos_base, scale, out_token_major_heads=heads)
    assert (ex.download(out_tm).reshape(t_q, heads, dh).transpose(1, 0, 2).reshape(-1) == got).all()


@pytest.mark.parametrize("case", [(4, 4, 64, 64, 64, 64, 0), (8, 2, 100, 160, 64, 100, 0), (4, 2, 37, 128, 64, 77, 40),
                                  (4, 4, 16, 64, 64, 10, 0), (32, 4, 512, 640, 64, 512, 0)])
def test_flash_io16_equals_the_f32_interface_rounded_to_f16(gpu, orc, case):
    """f16 q and out (the reference's kv16 io16 dh64 route, flash.rs:76-78, 193-212): with a q that
    f16 holds exactly, the kernel sees the same operands as through the f32 interface, so the f16
    output is that run's output rounded to nearest even -- and within the tensor-core tolerance of
    the oracle.  Short prefills (T_q < 32) take the tensor-core kernel too on this interface."""
    ta, ctx, ex = gpu
    heads, kv_heads, t_q, t_max, dh, kv_len, pos_base = case
    scale = 1.0 / np.sqrt(dh)
    kt_h, v_h = fill_kv(orc, kv_heads, t_max, dh, kv_len, 6e4)
    kt_h, v_h = orc.round_via_f16(kt_h), orc.round_via_f16(v_h)
    q_h = orc.round_via_f16(orc.fill_det(heads * t_q * dh, 5104)).reshape(heads, t_q, dh)
    kt, v = upload(ta, ctx, ex, kt_h, True), upload(ta, ctx, ex, v_h, True)
    q16, q32 = upload(ta, ctx, ex, q_h, True), upload(ta, ctx, ex, q_h)
    out16 = ta.Tensor.uninit_device_f16(ctx, (t_q, heads * dh))
    ex.upload(np.zeros(heads * t_q * dh, np.float32), out16)
    ex.run_flash_attention(q16, kt, v, out16, kv_len, pos_base, scale, out_token_major_heads=heads)
    got16 = ex.download(out16).reshape(t_q, heads, dh).transpose(1, 0, 2).reshape(-1)
    ref = orc.cpu_flash(q_h, kt_h, v_h, heads, kv_heads, t_q, dh, t_max, kv_len, pos_base, scale)
    assert np.isfinite(got16).all()
    assert np.abs(got16 - ref).max() <= MMA_TOL + 2.0 ** -11 * np.abs(ref).max()
    if t_q >= 32:
        out32 = ta.Tensor.uninit_device(ctx, (t_q, heads * dh))
        ex.upload(np.zeros(heads * t_q * dh, np.float32), out32)
        ex.run_flash_attention(q32, kt, v, out32, kv_len, pos_base, scale, out_token_major_heads=heads)
        want = ex.download(out32).astype(np.float16).astype(np.float32)
        assert np.array_equal(ex.download(out16), want)


def test_flash_io16_rejections(gpu, orc):
    ta, ctx, ex = gpu
    E = ta.TensorAshError
    q16 = ta.Tensor.uninit_device_f16(ctx, (4, 8, 64))
    out16 = ta.Tensor.uninit_device_f16(ctx, (4, 8, 64))
    out32 = ta.Tensor.uninit_device(ctx, (4, 8, 64))
    kt16, v16 = ta.Tensor.uninit_device_f16(ctx, (2, 64, 32)), ta.Tensor.uninit_device_f16(ctx, (2, 32, 64))
    kt32, v32 = ta.Tensor.uninit_device(ctx, (2, 64, 32)), ta.Tensor.uninit_device(ctx, (2, 32, 64))
    with pytest.raises(E, match=r"input \(f16\) and output \(f32\) must share a storage type"):
        ex.run_flash_attention(q16, kt16, v16, out32, 8, 0, 0.125)
    with pytest.raises(E, match="f16 q/out are compiled for f16 KV caches with head dimension 64"):
        ex.run_flash_attention(q16, kt32, v32, out16, 8, 0, 0.125)
    with pytest.raises(E, match="f16 q/out are compiled for f16 KV caches with head dimension 64"):
        ex.run_flash_attention(q16, kt16, v16, out16, 8, 0, 0.125, simt=True)


def test_flash_config5_shape(gpu, orc):
    """32 Q heads / 4 KV heads, dh 64, T_q = kv_len = 512, f16 KV, token-major out."""
    ta, ctx, ex = gpu
    heads, kv_heads, t_q, t_max, dh = 32, 4, 512, 640, 64
    scale = 1.0 / 8.0
    kt_h, v_h = fill_kv(orc, kv_heads, t_max, dh, t_q, 6e4)
    kt_h, v_h = orc.round_via_f16(kt_h), orc.round_via_f16(v_h)
    q_h = orc.fill_det(heads * t_q * dh, 5103).reshape(heads, t_q, dh)
    q, kt, v = upload(ta, ctx, ex, q_h), upload(ta, ctx, ex, kt_h, True), upload(ta, ctx, ex, v_h, True)
    out = ta.Tensor.uninit_device(ctx, (t_q, heads * dh))
    st = ex.run_flash_attention(q, kt, v, out, t_q, 0, scale, out_token_major_heads=heads)
    ref = orc.cpu_flash(q_h, kt_h, v_h, heads, kv_heads, t_q, dh, t_max, t_q, 0, scale)
    got = ex.download(out).reshape(t_q, heads, dh).transpose(1, 0, 2).reshape(-1)
    err = np.abs(got - ref).max()
    assert err <= MMA_TOL
    st32 = ex.run_flash_attention(q, kt, v, out, t_q, 0, scale, out_token_major_heads=heads, simt=True)
    got32 = ex.download(out).reshape(t_q, heads, dh).transpose(1, 0, 2).reshape(-1)
    assert np.abs(got32 - ref).max() <= TOL
    print(f"\nflash 32x512x64 causal: tensor cores {st.gpu_time_ns / 1e3:.1f} us (max err {err:.2e}), "
          f"f32 kernel {st32.gpu_time_ns / 1e3:.1f} us")


def test_flash_rejections(gpu, orc):
    ta, ctx, ex = gpu
    E = ta.TensorAshError
    q = ta.Tensor.uninit_device(ctx, (4, 8, 64))
    kt = ta.Tensor.uninit_device(ctx, (2, 64, 32))
    v = ta.Tensor.uninit_device(ctx, (2, 32, 64))
    out = ta.Tensor.uninit_device(ctx, (4, 8, 64))
    with pytest.raises(E, match="exceeds cache T_max"):
        ex.run_flash_attention(q, kt, v, out, 33, 0, 0.125)
    with pytest.raises(E, match="must share a storage type"):
        ex.run_flash_attention(q, kt, ta.Tensor.uninit_device_f16(ctx, (2, 32, 64)), out, 8, 0, 0.125)
    with pytest.raises(E, match="multiple of H_kv"):
        ex.run_flash_attention(ta.Tensor.uninit_device(ctx, (3, 8, 64)), kt, v, ta.Tensor.uninit_device(ctx, (3, 8, 64)), 8, 0, 0.125)
    with pytest.raises(E, match="inconsistent cache shapes"):
        ex.run_flash_attention(q, kt, ta.Tensor.uninit_device(ctx, (2, 31, 64)), out, 8, 0, 0.125)
    with pytest.raises(E, match="out shape"):
        ex.run_flash_attention(q, kt, v, ta.Tensor.uninit_device(ctx, (4, 8, 32)), 8, 0, 0.125)


DECODE_CASES = [  # kv_heads, group, t_max, kv_len
    (4, 8, 704, 640), (4, 8, 704, 513), (2, 4, 128, 1), (1, 1, 64, 33), (4, 8, 2048, 2048), (3, 5, 100, 77),
]


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("kv16", [False, True])
def test_attn_decode(gpu, orc, case, kv16):
    ta, ctx, ex = gpu
    kv_heads, group, t_max, kv_len = case
    dh, scale = 64, 0.125
    kt_h, v_h = fill_kv(orc, kv_heads, t_max, dh, kv_len, 6e4 if kv16 else 1e30, seed=5201)
    if kv16:
        kt_h, v_h = orc.round_via_f16(kt_h), orc.round_via_f16(v_h)
    q_h = orc.fill_det(kv_heads * group * dh, 5202).reshape(kv_heads, group, dh)
    q, kt, v = upload(ta, ctx, ex, q_h), upload(ta, ctx, ex, kt_h, kv16), upload(ta, ctx, ex, v_h, kv16)
    chunks = ta.lib().ta_attn_decode_num_chunks(kv_len)
    scratch = ta.Tensor.uninit_device(ctx, (kv_heads * chunks * group * (dh + 2),))
    out = ta.Tensor.uninit_device(ctx, (kv_heads, group, dh))
    before = ta.kernel_launch_count()
    ex.run_attn_decode(q, kt, v, scratch, out, kv_len, scale)
    assert ta.kernel_launch_count() == before + 1           # partials and combine in one launch
    ref = orc.cpu_attn_decode(q_h, kt_h, v_h, kv_heads, group, dh, t_max, kv_len, scale)
    got = ex.download(out).reshape(-1)
    assert np.isfinite(got).all() and np.abs(got - ref).max() <= TOL
    # position-indirect form: kv_len = 1 + *cell on the fixed 32-chunk grid gives the same answer
    cell = ta.PosCell(ctx)
    cell.set(kv_len - 1)
    scratch32 = ta.Tensor.uninit_device(ctx, (kv_heads * 32 * group * (dh + 2),))
    out2 = ta.Tensor.uninit_device(ctx, (kv_heads, group, dh))
    ex.run_attn_decode(q, kt, v, scratch32, out2, 1, scale, pos_cell=cell)
    got2 = ex.download(out2).reshape(-1)
    assert np.abs(got2 - ref).max() <= TOL


def test_attn_decode_position_outside_the_cache_is_reported_not_read(gpu, orc):
    """A position cell beyond the cache: the kernel clamps the length to t_max (no access outside the
    cache), raises its status bit, the call fails with the position message, and the next call works."""
    ta, ctx, ex = gpu
    kv_heads, group, t_max, dh, scale = 2, 4, 128, 64, 0.125
    kt_h, v_h = fill_kv(orc, kv_heads, t_max, dh, t_max, 1e30, seed=5301)
    q_h = orc.fill_det(kv_heads * group * dh, 5302).reshape(kv_heads, group, dh)
    q, kt, v = upload(ta, ctx, ex, q_h), upload(ta, ctx, ex, kt_h), upload(ta, ctx, ex, v_h)
    scratch = ta.Tensor.uninit_device(ctx, (kv_heads * 32 * group * (dh + 2),))
    out = ta.Tensor.uninit_device(ctx, (kv_heads, group, dh))
    cell = ta.PosCell(ctx)
    cell.set(t_max + 5)
    with pytest.raises(ta.TensorAshError, match="position cell"):
        ex.run_attn_decode(q, kt, v, scratch, out, 1, scale, pos_cell=cell)
    cell.set(63)
    ex.run_attn_decode(q, kt, v, scratch, out, 1, scale, pos_cell=cell)
    ref = orc.cpu_attn_decode(q_h, kt_h, v_h, kv_heads, group, dh, t_max, 64, scale)
    assert np.abs(ex.download(out).reshape(-1) - ref).max() <= TOL


def test_attn_decode_rejections(gpu, orc):
    ta, ctx, ex = gpu
    E = ta.TensorAshError
    kt = ta.Tensor.uninit_device(ctx, (2, 64, 128))
    v = ta.Tensor.uninit_device(ctx, (2, 128, 64))
    q = ta.Tensor.uninit_device(ctx, (2, 4, 64))
    out = ta.Tensor.uninit_device(ctx, (2, 4, 64))
    small = ta.Tensor.uninit_device(ctx, (16,))
    big = ta.Tensor.uninit_device(ctx, (2 * 32 * 4 * 66,))
    with pytest.raises(E, match="scratch length 16 < required"):
        ex.run_attn_decode(q, kt, v, small, out, 100, 0.125)
    with pytest.raises(E, match="out of range 1..=128"):
        ex.run_attn_decode(q, kt, v, big, out, 0, 0.125)
    with pytest.raises(E, match="out of range"):
        ex.run_attn_decode(q, kt, v, big, out, 129, 0.125)
    with pytest.raises(E, match="GQA group 9 unsupported"):
        ex.run_attn_decode(ta.Tensor.uninit_device(ctx, (2, 9, 64)), kt, v, big, ta.Tensor.uninit_device(ctx, (2, 9, 64)), 8, 0.125)
    with pytest.raises(E, match="head dimension 128 unsupported"):
        ex.run_attn_decode(ta.Tensor.uninit_device(ctx, (2, 4, 128)), ta.Tensor.uninit_device(ctx, (2, 128, 64)),
                           ta.Tensor.uninit_device(ctx, (2, 64, 128)), big, ta.Tensor.uninit_device(ctx, (2, 4, 128)), 8, 0.125)
