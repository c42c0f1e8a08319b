"""GGUF reader (host only) and the GGUF-backed llama runner.

The reader cases restate the reference's own unit tests (tools/llama-ash/src/gguf.rs:277-414):
a synthetic v3 file with scalar, string and array metadata, one f32 and one f16 tensor and
32-byte alignment; bad magic and bad version are refused.  The GPU case writes a small f16 llama
GGUF, loads it and compares prefill + greedy decode with the host forward on the same weights.
"""
import struct

import numpy as np
import pytest


def synthetic(ta, path):
    w32 = np.array([[0.5, -1.0, 2.0], [3.5, -0.25, 8.0]], np.float32)      # ne = [3, 2]
    w16 = np.array([1.0, -2.0, 0.5, 4.0], np.float16)                      # ne = [4]
    ta.write_gguf(path, {
        "general.architecture": "llama",
        "llama.block_count": 22,
        "llama.attention.layer_norm_rms_epsilon": 1e-5,
        "tokenizer.ggml.tokens": ["a", "bc"],
        "tokenizer.ggml.scores": [1.0, 2.0],
        "some.signed": -7,
        "some.wide": ("u64", 2 ** 40),
        "some.double": ("f64", 0.125),
        "some.flag": True,
    }, {"w32": w32, "w16": w16})
    return w32, w16


def test_reader_parses_the_reference_synthetic_file(ta, tmp_path):
    path = str(tmp_path / "mini.gguf")
    w32, w16 = synthetic(ta, path)
    g = ta.GgufFile(path)
    assert g.string("general.architecture") == "llama"
    assert g.require_u64("llama.block_count") == 22
    assert abs(g.f64_or("llama.attention.layer_norm_rms_epsilon", 0.0) - 1e-5) < 1e-12
    assert g.f64_or("llama.rope.freq_base", 10000.0) == 10000.0            # absent: the fallback
    assert g.kind("tokenizer.ggml.tokens") == "skipped" and g.kind("tokenizer.ggml.scores") == "skipped"
    assert g.kind("nope") is None
    assert g.kind("some.signed") == "i64" and g.f64_or("some.signed", 0.0) == -7.0
    with pytest.raises(ta.TensorAshError, match="missing integer key some.signed"):
        g.require_u64("some.signed")                                       # negative: not a u64
    assert g.require_u64("some.wide") == 2 ** 40 and g.f64_or("some.double", 0.0) == 0.125
    assert g.kind("some.flag") == "bool"
    ne, ty, off = g.info("w32")
    assert (ne, ty, off) == ([3, 2], 0, 0)
    assert np.array_equal(g.read_f32("w32"), w32.ravel())
    ne, ty, off = g.info("w16")
    assert (ne, ty, off) == ([4], 1, 32) and g.data_start % 32 == 0        # 24 payload bytes padded to 32
    assert np.array_equal(g.read_f32("w16"), w16.astype(np.float32))
    with pytest.raises(ta.TensorAshError, match="tensor nope not found"):
        g.info("nope")
    g.close()


def test_reader_honours_general_alignment_and_version_2(ta, tmp_path):
    path = str(tmp_path / "a64.gguf")
    a = np.arange(5, dtype=np.float32)
    b = np.arange(3, dtype=np.float16)
    ta.write_gguf(path, {"general.architecture": "llama"}, {"a": a, "b": b}, alignment=64, version=2)
    g = ta.GgufFile(path)
    assert g.data_start % 64 == 0 and g.info("b")[2] == 64
    assert np.array_equal(g.read_f32("a"), a) and np.array_equal(g.read_f32("b"), b.astype(np.float32))


def test_reader_rejects_bad_magic_version_types_and_truncation(ta, tmp_path):
    path = str(tmp_path / "bad.gguf")
    open(path, "wb").write(b"NOPE")
    with pytest.raises(ta.TensorAshError, match="magic"):
        ta.GgufFile(path)
    open(path, "wb").write(b"GGUF" + struct.pack("<IQQ", 7, 0, 0))
    with pytest.raises(ta.TensorAshError, match="version"):
        ta.GgufFile(path)
    open(path, "wb").write(b"GGUF" + struct.pack("<IQQ", 3, 1 << 21, 0))
    with pytest.raises(ta.TensorAshError, match="implausible"):
        ta.GgufFile(path)
    open(path, "wb").write(b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 3) + b"key" + struct.pack("<I", 13))
    with pytest.raises(ta.TensorAshError, match="unknown GGUF metadata type 13"):
        ta.GgufFile(path)
    # a quantized tensor type (2 = Q4_0) is indexed but cannot be read
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 1) + b"q" + struct.pack("<IQIQ", 1, 32, 2, 0)
    open(path, "wb").write(head + b"\0" * ((-len(head)) % 32) + b"\0" * 64)
    g = ta.GgufFile(path)
    with pytest.raises(ta.TensorAshError, match="only F32/F16 are supported"):
        g.read_f32("q")
    # payload running past the end of the file
    good = str(tmp_path / "good.gguf")
    ta.write_gguf(good, {}, {"w": np.ones(64, np.float32)})
    raw = open(good, "rb").read()
    open(path, "wb").write(raw[:-16])
    with pytest.raises(ta.TensorAshError, match="past the end of the file"):
        ta.GgufFile(path).read_f32("w")
    with pytest.raises(ta.TensorAshError, match="opening"):
        ta.GgufFile(str(tmp_path / "absent.gguf"))


# ---------------------------------------------------------------------------- model from a file
def tiny_model_file(ta, path, rng, f32_embedding=False, tied=False):
    layers, embd, heads, kv, ffn, vocab = 2, 256, 4, 2, 512, 384
    kv_dim = kv * (embd // heads)
    w = lambda n_out, n_in: (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float16)   # ggml: [n_out][n_in]
    t = {"token_embd.weight": (rng.standard_normal((vocab, embd)) * 0.05).astype(np.float32 if f32_embedding else np.float16),
         "output_norm.weight": (1 + 0.1 * rng.uniform(-1, 1, embd)).astype(np.float32)}
    if not tied:
        t["output.weight"] = w(vocab, embd)
    for i in range(layers):
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = (1 + 0.1 * rng.uniform(-1, 1, embd)).astype(np.float32)
        t[p + "ffn_norm.weight"] = (1 + 0.1 * rng.uniform(-1, 1, embd)).astype(np.float32)
        t[p + "attn_q.weight"], t[p + "attn_k.weight"], t[p + "attn_v.weight"] = w(embd, embd), w(kv_dim, embd), w(kv_dim, embd)
        t[p + "attn_output.weight"] = w(embd, embd)
        t[p + "ffn_gate.weight"], t[p + "ffn_up.weight"], t[p + "ffn_down.weight"] = w(ffn, embd), w(ffn, embd), w(embd, ffn)
    meta = {"general.architecture": "llama", "llama.block_count": layers, "llama.embedding_length": embd,
            "llama.attention.head_count": heads, "llama.attention.head_count_kv": kv,
            "llama.feed_forward_length": ffn, "llama.context_length": 96,
            "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0,
            "tokenizer.ggml.tokens": ["<s>", "a"]}
    ta.write_gguf(path, meta, t)
    return t


class FileRef:
    """Host forward (float64) on the tensors of a model file, same graph as tests/llama_ref.py."""

    def __init__(self, t, cfg):
        self.t, self.c = t, cfg
        self.kcache = [np.zeros((0, cfg.kv_heads * cfg.head_dim)) for _ in range(cfg.layers)]
        self.vcache = [np.zeros((0, cfg.kv_heads * cfg.head_dim)) for _ in range(cfg.layers)]

    def lin(self, name):                      # y = x @ W^T with W stored [n_out][n_in]
        return self.t[name].astype(np.float64).T

    def rms(self, x, w):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + self.c.rms_eps) * w.astype(np.float64)

    def rope(self, x, heads, pos0):
        n, dh = x.shape[0], self.c.head_dim
        xh = x.reshape(n, heads, dh // 2, 2)
        pos = np.arange(pos0, pos0 + n, dtype=np.float64)[:, None]
        ang = pos / np.power(float(self.c.rope_theta), 2.0 * np.arange(dh // 2) / dh)[None, :]
        cs, sn = np.cos(ang).astype(np.float32).astype(np.float64)[:, None], np.sin(ang).astype(np.float32).astype(np.float64)[:, None]
        a, b = xh[..., 0], xh[..., 1]
        return np.stack([a * cs - b * sn, a * sn + b * cs], -1).reshape(n, heads * dh)

    def forward(self, tokens):
        c = self.c
        x = self.t["token_embd.weight"].astype(np.float64)[np.asarray(tokens)]
        pos0 = self.kcache[0].shape[0]
        f16 = lambda v: v.astype(np.float16).astype(np.float64)
        for i in range(c.layers):
            p = f"blk.{i}."
            xn = self.rms(x, self.t[p + "attn_norm.weight"])
            q = self.rope(xn @ self.lin(p + "attn_q.weight"), c.heads, pos0)
            k = f16(self.rope(xn @ self.lin(p + "attn_k.weight"), c.kv_heads, pos0))
            v = f16(xn @ self.lin(p + "attn_v.weight"))
            self.kcache[i] = np.concatenate([self.kcache[i], k]); self.vcache[i] = np.concatenate([self.vcache[i], v])
            K = self.kcache[i].reshape(-1, c.kv_heads, c.head_dim); V = self.vcache[i].reshape(-1, c.kv_heads, c.head_dim)
            out = np.zeros((len(tokens), c.heads, c.head_dim))
            g = c.heads // c.kv_heads
            qh = q.reshape(len(tokens), c.heads, c.head_dim)
            for h in range(c.heads):
                s = qh[:, h] @ K[:, h // g].T / np.sqrt(c.head_dim)
                for r in range(len(tokens)):
                    s[r, pos0 + r + 1:] = -np.inf
                pr = np.exp(s - s.max(-1, keepdims=True)); pr /= pr.sum(-1, keepdims=True)
                out[:, h] = pr @ V[:, h // g]
            x = x + out.reshape(len(tokens), -1) @ self.lin(p + "attn_output.weight")
            xn = self.rms(x, self.t[p + "ffn_norm.weight"])
            gate, up = xn @ self.lin(p + "ffn_gate.weight"), xn @ self.lin(p + "ffn_up.weight")
            x = x + (gate / (1 + np.exp(-gate)) * up) @ self.lin(p + "ffn_down.weight")
        head = self.t["output.weight"] if "output.weight" in self.t else self.t["token_embd.weight"]
        return self.rms(x[-1:], self.t["output_norm.weight"])[0] @ head.astype(np.float64).T


@pytest.mark.gpu
@pytest.mark.parametrize("f32_embedding,tied", [(False, False), (True, False), (False, True)])
def test_model_loaded_from_gguf_matches_the_host_forward(gpu, tmp_path, f32_embedding, tied):
    ta, ctx, ex = gpu
    rng = np.random.default_rng(7)
    path = str(tmp_path / "tiny.gguf")
    t = tiny_model_file(ta, path, rng, f32_embedding, tied)
    m = ta.Llama.load_gguf(ex, path, t_max=4096)
    c = m.cfg
    assert (c.layers, c.embd, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab) == (2, 256, 4, 2, 64, 512, 384)
    assert c.t_max == 96                                   # clamped to llama.context_length
    ref = FileRef(t, c)
    prompt = [int(v) for v in rng.integers(0, c.vocab, 37)]
    nxt, _ = m.prefill(prompt)
    want = ref.forward(prompt)
    got = m.logits().astype(np.float64)
    assert np.abs(got - want).max() <= 2e-3 * max(1.0, np.abs(want).max())
    top2 = np.sort(want)[-2:]
    if top2[1] - top2[0] > 1e-2:
        assert nxt == int(np.argmax(want))
    toks, _ = m.decode(nxt, 6)
    cur = nxt
    for step in range(6):
        want = ref.forward([cur])
        order = np.argsort(want)
        if want[order[-1]] - want[order[-2]] > 1e-2:
            assert toks[step] == int(order[-1]), f"step {step}"
        cur = toks[step]
    m.close()


@pytest.mark.gpu
def test_gguf_model_errors(gpu, tmp_path):
    ta, ctx, ex = gpu
    path = str(tmp_path / "x.gguf")
    ta.write_gguf(path, {"general.architecture": "gpt2"}, {})
    with pytest.raises(ta.TensorAshError, match="unsupported architecture gpt2"):
        ta.Llama.load_gguf(ex, path)
    ta.write_gguf(path, {"general.architecture": "llama", "llama.block_count": 1}, {})
    with pytest.raises(ta.TensorAshError, match="missing integer key llama.embedding_length"):
        ta.Llama.load_gguf(ex, path)
    rng = np.random.default_rng(1)
    t = tiny_model_file(ta, path, rng)
    t["blk.1.attn_k.weight"] = t["blk.1.attn_k.weight"][:, :-32]
    meta = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 256,
            "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2,
            "llama.feed_forward_length": 512, "llama.context_length": 96}
    ta.write_gguf(path, meta, t)
    with pytest.raises(ta.TensorAshError, match=r"blk.1.attn_k.weight: ne \[224, 128\] != expected \[256, 128\]"):
        ta.Llama.load_gguf(ex, path)


# ---------------------------------------------------------------------------- the llama_ash tool
def llama_ash(*args):
    import os
    import subprocess
    import __graft_entry__ as entry
    exe = os.path.join(entry.PKG_DIR, "bin", "llama_ash")
    if not os.path.exists(exe):
        entry.build()
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=300)


def test_llama_ash_cli_rejects_bad_command_lines():
    """tools/llama-ash/src/main.rs:26-66: unknown flags and subcommands, missing values, missing model."""
    r = llama_ash()
    assert r.returncode != 0 and "usage:" in r.stderr
    r = llama_ash("bench")
    assert r.returncode != 0 and "missing -m <gguf>" in r.stderr
    r = llama_ash("bench", "-m", "x.gguf", "--bogus", "1")
    assert r.returncode != 0 and "unknown flag --bogus" in r.stderr
    r = llama_ash("bench", "-m")
    assert r.returncode != 0 and "flag -m needs a value" in r.stderr
    r = llama_ash("bench", "-m", "x.gguf", "--pp", "many")
    assert r.returncode != 0 and "--pp" in r.stderr
    r = llama_ash("train", "-m", "x.gguf")
    assert r.returncode != 0 and "unknown subcommand train" in r.stderr


@pytest.mark.gpu
def test_llama_ash_cli_generates_the_library_tokens_and_prints_the_bench_table(gpu, tmp_path):
    ta, ctx, ex = gpu
    rng = np.random.default_rng(11)
    path = str(tmp_path / "tiny.gguf")
    tiny_model_file(ta, path, rng)
    prompt = [1, 7, 300, 42, 5]
    m = ta.Llama.load_gguf(ex, path, t_max=96)
    first, _ = m.prefill(prompt)
    rest, _ = m.decode(first, 7)
    m.close()
    r = llama_ash("generate", "-m", path, "--ids", ", ".join(map(str, prompt)), "-n", "8", "--ctx", "96")
    assert r.returncode == 0, r.stderr
    lines = dict(l.split(":", 1) for l in r.stdout.strip().splitlines())
    assert lines["prompt_ids   "].strip() == ",".join(map(str, prompt))
    assert lines["generated_ids"].strip() == ",".join(map(str, [first] + rest))
    r = llama_ash("bench", "-m", path, "--pp", "40", "--tg", "16", "--ctx", "96")
    assert r.returncode == 0, r.stderr
    assert "| pp40 " in r.stdout and "| tg16 " in r.stdout and "tokens/s" in r.stdout
    r = llama_ash("bench", "-m", path, "--pp", "90", "--tg", "16", "--ctx", "96")
    assert r.returncode != 0 and "exceeds context 96" in r.stderr
    r = llama_ash("generate", "-m", path, "--ids", "1,99999")
    assert r.returncode != 0 and "outside the vocabulary" in r.stderr
