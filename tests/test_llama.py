"""Llama runner: prefill graph and prepared decode graph against the numpy forward.

Token parity follows the reference's own criterion for greedy decoding
(tools/llama-ash/tests: tokens must agree wherever the top-2 logit margin is
larger than the accumulated rounding error); logits are compared with a
relative-to-max tolerance of 2e-4 (f32 accumulation on the device against f64
on the host, through `layers` blocks with f16 KV rounding on both sides).  Prompts
of 32 tokens and more run their projections on the f16 tensor-core GEMM, which
rounds activations to f16 on the way in: there the f16-weight bound 2e-3 applies.
"""
import numpy as np
import pytest

from llama_ref import RefLlama

LOGIT_TOL = 2e-4


def small_cfg(ta, **kw):
    base = dict(layers=2, embd=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024, t_max=96,
                weight_sigma=0.05, norm_jitter=0.25, seed=7)
    base.update(kw)
    return ta.LlamaConfig(**base)


def check_logits(got, want, tol=LOGIT_TOL):
    denom = np.abs(want).max()
    err = np.abs(got.astype(np.float64) - want).max() / denom
    assert err <= tol, f"logits rel err {err:.3e}"


def margin(logits):
    top = np.sort(logits)[-2:]
    return top[1] - top[0]


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [1, 5, 33])
def test_prefill_matches_host_forward(ta, orc, gpu, prompt_len):
    cfg = small_cfg(ta)
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    model = ta.Llama(ex, cfg)
    ref = RefLlama(orc, cfg)
    prompt = [(17 * i + 3) % cfg.vocab for i in range(prompt_len)]
    nxt, st = model.prefill(prompt)
    want = ref.forward(prompt)
    tol = 2e-3 if prompt_len >= 32 else LOGIT_TOL
    check_logits(model.logits(), want, tol)
    if margin(want) > 4 * tol * np.abs(want).max():
        assert nxt == int(np.argmax(want))
    assert model.position == prompt_len
    assert st.gpu_time_ns is not None and st.gpu_time_ns > 0


@pytest.mark.gpu
def test_decode_graph_matches_host_forward(ta, orc, gpu):
    cfg = small_cfg(ta)
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    model = ta.Llama(ex, cfg)
    ref = RefLlama(orc, cfg)
    prompt = [5, 900, 31, 64, 512, 77, 1]
    nxt, _ = model.prefill(prompt)
    want = ref.forward(prompt)
    tok = int(np.argmax(want))
    assert nxt == tok
    n = 24
    got, st = model.decode(nxt, n)
    assert st.n_calls > 0
    # teacher-forced on the device's own choices, so one near-tie cannot derail the rest
    fed = nxt
    for i in range(n):
        want = ref.forward([fed])
        if margin(want) > 1e-3 * np.abs(want).max():
            assert got[i] == int(np.argmax(want)), f"step {i}"
        fed = got[i]
    check_logits(model.logits(), want)
    assert model.position == len(prompt) + n


@pytest.mark.gpu
def test_decode_continues_across_calls_and_reset(ta, orc, gpu):
    cfg = small_cfg(ta, seed=11)
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    model = ta.Llama(ex, cfg)
    prompt = [9, 8, 7, 6]
    nxt, _ = model.prefill(prompt)
    a, _ = model.decode(nxt, 10)
    model.reset()
    nxt2, _ = model.prefill(prompt)
    assert nxt2 == nxt
    b1, _ = model.decode(nxt2, 4)
    b2, _ = model.decode(b1[-1], 6)
    assert a == b1 + b2


@pytest.mark.gpu
def test_decode_breakdown_step_equals_a_graph_step(ta, orc, gpu):
    """The instrumented step (every launch between two events, the LLAMA_ASH_BREAKDOWN table of
    tools/llama-ash/src/main.rs:161-193) computes what a replayed graph step computes: same token,
    same logits; its rows cover every launch once and name the reference's op classes."""
    cfg = small_cfg(ta, seed=13)
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    model = ta.Llama(ex, cfg)
    prompt = [3, 14, 159, 26, 535]
    nxt, _ = model.prefill(prompt)
    toks, _ = model.decode(nxt, 3)
    want_logits = model.logits().copy()
    model.reset()
    nxt2, _ = model.prefill(prompt)
    a, _ = model.decode(nxt2, 2)
    tok, launches, rows = model.decode_breakdown(a[-1])
    assert a + [tok] == toks and np.array_equal(model.logits(), want_logits)
    assert model.position == len(prompt) + 3
    classes = {name for name, _, _ in rows}
    assert {"qkv_matmul", "attn_decode", "o_proj_mm", "ffn_up_mm", "ffn_down_mm", "lm_head_mm", "argmax"} <= classes
    assert sum(calls for _, _, calls in rows) == launches == 5 * cfg.layers + 3
    assert all(ns > 0 for _, ns, _ in rows) and [ns for _, ns, _ in rows] == sorted((ns for _, ns, _ in rows), reverse=True)


@pytest.mark.gpu
def test_chunked_prefill_matches_single_prefill(ta, orc, gpu):
    cfg = small_cfg(ta, seed=3)
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    model = ta.Llama(ex, cfg)
    prompt = [(29 * i + 11) % cfg.vocab for i in range(40)]
    model.prefill(prompt)
    whole = model.logits()
    model.reset()
    model.prefill(prompt[:24])
    model.prefill(prompt[24:])
    parts = model.logits()
    # 40 and 24 rows take the tensor-core GEMM, 16 rows the f32-activation tiles
    assert np.abs(whole - parts).max() <= 2e-3 * np.abs(whole).max()


@pytest.mark.gpu
def test_kv_overflow_and_bad_config_are_errors(ta, gpu):
    ctx = ta.Context()
    ex = ta.Executor(ctx, max_calls_per_submit=256)
    with pytest.raises(ta.TensorAshError, match="heads \\* head_dim"):
        ta.Llama(ex, small_cfg(ta, heads=3))
    model = ta.Llama(ex, small_cfg(ta, t_max=8))
    with pytest.raises(ta.TensorAshError, match="KV cache overflow"):
        model.prefill(list(range(9)))
    nxt, _ = model.prefill(list(range(6)))
    with pytest.raises(ta.TensorAshError, match="KV cache overflow"):
        model.decode(nxt, 3)


def test_weight_bytes_formula_matches_config_5():
    # 22 layers, embd 2048, kv_dim 256, ffn 5632, vocab 32000: f16 bytes per decoded token
    per_layer = 2 * 2048 * 2048 + 2 * 2048 * 256 + 3 * 2048 * 5632
    assert 2 * (22 * per_layer + 2048 * 32000) == 2_068_840_448
