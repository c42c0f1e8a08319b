"""Full-size configurations through size-independent properties (the CPU oracle
cannot finish them in seconds):

* configs[1], 32 x 2048^3 batched FP32 GEMM with shared B, per-batch bias, SiLU and
  residual: sampled outputs against float64, exact power-of-two linearity, and batch
  independence (a plane computed alone is bit-identical to the same plane of the batch);
* configs[4], the llama decoder at 22L / 2048 / 32q / 4kv / 5632 / 32000: the greedy token
  stream is reproducible run to run, and the decode graph (f32 activations, GEMV) agrees
  with the prefill graph (tensor-core GEMM, f16-rounded activations) on the logits of the
  same position within the f16-weight tolerance 2e-3.

configs[2] (4096 x 11008 MLP, M in {1,4,8}) and configs[3] (K = 65536 split-K) already run
at full size against the oracle in test_gemv.py and test_splitk2.py.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

BATCH, M, N, K = 32, 2048, 2048, 2048


@pytest.fixture(scope="module")
def cfg2(ta):
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 8)
    rng = np.random.default_rng(2024)
    sig = np.float32(1.0 / np.sqrt(K))
    host = {name: rng.standard_normal(shape, dtype=np.float32) * sig
            for name, shape in (("a", (BATCH, M, K)), ("b", (K, N)), ("bias", (BATCH, N)), ("r", (BATCH, M, N)))}
    dev = {k: ta.Tensor.uninit_device(ctx, v.shape) for k, v in host.items()}
    for k, v in host.items():
        ex.upload(v, dev[k])
    dev["c"] = ta.Tensor.uninit_device(ctx, (BATCH, M, N))
    yield ta, ctx, ex, host, dev
    for t in dev.values():
        t.close()
    ex.close()
    ctx.close()


def test_config2_sampled_outputs_against_float64(cfg2):
    ta, ctx, ex, host, dev = cfg2
    op = ta.MatmulOp(ta.MatmulCall(dev["a"], dev["b"], dev["c"]),
                     ta.Epilogue(dev["bias"], ta.Activation.SILU, ta.Binary.ADD_SCALED, dev["r"], 1.0))
    st = ex.run_ops([op])
    assert st.total_flops == 2 * BATCH * M * N * K
    assert ex.dispatch_info_for(BATCH, M, N, K).kernel.startswith("tf32x3")
    out = ex.download(dev["c"]).reshape(BATCH, M, N)
    a, b, bias, r = host["a"], host["b"], host["bias"], host["r"]
    worst = 0.0
    for s in range(512):
        idx = (s * 2654435761 + 777) % (BATCH * M * N)
        bi, rem = divmod(idx, M * N)
        i, j = divmod(rem, N)
        acc = float(np.dot(a[bi, i].astype(np.float64), b[:, j].astype(np.float64)))
        x = float(np.float32(acc)) + float(bias[bi, j])
        x = x / (1.0 + np.exp(-x)) + float(r[bi, i, j])
        worst = max(worst, abs(float(out[bi, i, j]) - x) / max(1.0, abs(x)))
    assert worst <= 1e-5, f"rel err {worst:.3e}"


def test_config2_power_of_two_linearity_is_exact(cfg2):
    """C(4A) == 4 C(A) bit for bit: scaling by a power of two commutes with the hi/lo split,
    every product and every rounding of the accumulation."""
    ta, ctx, ex, host, dev = cfg2
    call = ta.MatmulCall(dev["a"], dev["b"], dev["c"])
    ex.run_matmuls([call])
    base = ex.download(dev["c"])
    ex.run_matmuls([ta.MatmulCall(dev["a"], dev["b"], dev["c"], 4.0)])       # alpha = 4 on the drain
    assert np.array_equal(ex.download(dev["c"]), base * np.float32(4.0))
    a4 = ta.Tensor.uninit_device(ctx, (BATCH, M, K))
    ex.upload(host["a"] * np.float32(4.0), a4)
    ex.run_matmuls([ta.MatmulCall(a4, dev["b"], dev["c"])])
    assert np.array_equal(ex.download(dev["c"]), base * np.float32(4.0))
    a4.close()


def test_config2_planes_are_independent(cfg2):
    ta, ctx, ex, host, dev = cfg2
    ex.run_matmuls([ta.MatmulCall(dev["a"], dev["b"], dev["c"])])
    full = ex.download(dev["c"]).reshape(BATCH, M, N)
    one_a = ta.Tensor.uninit_device(ctx, (M, K))
    one_c = ta.Tensor.uninit_device(ctx, (M, N))
    for plane in (0, 17, 31):
        ex.upload(host["a"][plane], one_a)
        ex.run_matmuls([ta.MatmulCall(one_a, dev["b"], one_c)])
        assert np.array_equal(ex.download(one_c).reshape(M, N), full[plane]), f"plane {plane}"
    one_a.close()
    one_c.close()


def test_config5_llama_full_size_reproducible_and_self_consistent(ta):
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 1024)
    cfg = ta.LlamaConfig(t_max=704, seed=5)          # 22L / 2048 / 32q / 4kv / 5632 / 32000
    model = ta.Llama(ex, cfg)
    assert model.weight_bytes_per_token == 2_068_840_448
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(512)]
    nxt, _ = model.prefill(prompt)
    logits_prefill = model.logits().astype(np.float64)
    toks, _ = model.decode(nxt, 128)
    assert model.position == 640 and all(0 <= t < cfg.vocab for t in toks)
    # the same run again gives the same stream
    model.reset()
    nxt2, _ = model.prefill(prompt)
    toks2, _ = model.decode(nxt2, 128)
    assert nxt2 == nxt and toks2 == toks
    # the last prompt position through the decode graph instead of the prefill graph
    model.reset()
    head, _ = model.prefill(prompt[:511])
    got, _ = model.decode(prompt[511], 1)
    logits_decode = model.logits().astype(np.float64)
    scale = np.abs(logits_prefill).max()
    assert np.abs(logits_decode - logits_prefill).max() <= 2e-3 * scale
    top = np.sort(logits_prefill)[-2:]
    if top[1] - top[0] > 8e-3 * scale:
        assert got[0] == nxt
    model.close()
    ex.close()
    ctx.close()
