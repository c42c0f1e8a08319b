"""Host restatement (numpy, f64 accumulation) of the llama-architecture forward pass
the runner executes: f16-rounded weights from the documented seed streams, RMSNorm,
RoPE on interleaved pairs (2i, 2i+1) as the library's rope op defines them, GQA causal attention over an f16-rounded KV cache, SwiGLU MLP,
greedy argmax (first maximum).  Test infrastructure only.
"""
import numpy as np

CHUNK = 1 << 20


def chunk_seed(seed, tensor_id, chunk):
    return ((seed * 1000003 + tensor_id) * 4096 + chunk) & 0xFFFFFFFFFFFFFFFF


def gen_weight(orc, seed, tensor_id, rows, cols, sigma, keep_f16=False):
    """Tensor `tensor_id` of the documented seed stream, rounded to f16.  keep_f16 returns the
    float16 array itself (a quarter of the memory; every value converts to f64 exactly)."""
    n = rows * cols
    out = np.empty(n, dtype=np.float16)

    def chunk(c):
        lo, hi = c * CHUNK, min(n, (c + 1) * CHUNK)
        out[lo:hi] = orc.fill_normal((hi - lo,), chunk_seed(seed, tensor_id, c), sigma).astype(np.float16)

    chunks = range((n + CHUNK - 1) // CHUNK)
    if len(chunks) > 4:      # the C generator releases the GIL: chunks in parallel
        from concurrent.futures import ThreadPoolExecutor
        import os
        with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as pool:
            list(pool.map(chunk, chunks))
    else:
        for c in chunks:
            chunk(c)
    out = out.reshape(rows, cols)
    return out if keep_f16 else out.astype(np.float64)


def lcg_tokens(n, vocab, seed=12345):
    """Prompt ids from the reference's LcgRng stream (tools/test-support/src/lib.rs:20-55)."""
    s = (seed * 0x9E3779B97F4A7C15 | 1) & 0xFFFFFFFFFFFFFFFF
    out = []
    for _ in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out.append((s >> 33) % vocab)
    return out


def gen_norm(orc, seed, tensor_id, n, jitter):
    if jitter == 0.0:
        return np.ones(n)
    u = orc.fill_det(n, chunk_seed(seed, tensor_id, 0)).astype(np.float32)
    return (np.float32(1.0) + np.float32(jitter) * u).astype(np.float64)


class RefLlama:
    def __init__(self, orc, cfg, lean=False):
        """lean=True keeps the weights as float16 arrays and widens one matrix at a time while it is
        used: the 22-layer configuration then needs 2.2 GB instead of 8.8 GB of host memory."""
        self.cfg = c = cfg
        s, sg = c.seed, c.weight_sigma
        kv_dim = c.kv_heads * c.head_dim
        w = lambda tid, r, cc: gen_weight(orc, s, tid, r, cc, sg, keep_f16=lean)  # noqa: E731
        self.embd = w(0, c.vocab, c.embd)
        self.output_norm = gen_norm(orc, s, 1, c.embd, c.norm_jitter)
        self.lm_head = w(2, c.embd, c.vocab)
        self.layers = []
        for li in range(c.layers):
            b = 16 + 16 * li
            self.layers.append(dict(
                attn_norm=gen_norm(orc, s, b + 0, c.embd, c.norm_jitter),
                wq=w(b + 1, c.embd, c.embd),
                wk=w(b + 2, c.embd, kv_dim),
                wv=w(b + 3, c.embd, kv_dim),
                wo=w(b + 4, c.embd, c.embd),
                ffn_norm=gen_norm(orc, s, b + 5, c.embd, c.norm_jitter),
                w_gate=w(b + 6, c.embd, c.ffn),
                w_up=w(b + 7, c.embd, c.ffn),
                w_down=w(b + 8, c.ffn, c.embd),
                k=np.zeros((0, c.kv_heads, c.head_dim)), v=np.zeros((0, c.kv_heads, c.head_dim))))
        half = c.head_dim // 2
        p = np.arange(c.t_max, dtype=np.float64)[:, None]
        i = np.arange(half, dtype=np.float64)[None, :]
        theta = p / np.power(float(c.rope_theta), 2.0 * i / c.head_dim)
        # the device table is f32
        self.cos = np.cos(theta).astype(np.float32).astype(np.float64)
        self.sin = np.sin(theta).astype(np.float32).astype(np.float64)
        self.pos = 0

    def _rms(self, x, w):
        ms = np.mean(x * x, axis=-1, keepdims=True)
        return x / np.sqrt(ms + float(np.float32(self.cfg.rms_eps))) * w

    def _rope(self, x, heads, pos0):
        c = self.cfg
        t = x.shape[0]
        xh = x.reshape(t, heads, c.head_dim // 2, 2)
        cos = self.cos[pos0:pos0 + t][:, None, :]
        sin = self.sin[pos0:pos0 + t][:, None, :]
        a, b = xh[..., 0], xh[..., 1]
        return np.stack([a * cos - b * sin, a * sin + b * cos], axis=-1).reshape(t, heads * c.head_dim)

    def reset(self):
        c = self.cfg
        for L in self.layers:
            L["k"] = np.zeros((0, c.kv_heads, c.head_dim))
            L["v"] = np.zeros((0, c.kv_heads, c.head_dim))
        self.pos = 0

    def forward(self, tokens):
        """Consumes tokens at the current position; returns logits of the last one ([vocab])."""
        return self.forward_positions(tokens, 1)[0]

    def forward_positions(self, tokens, n_last):
        """Consumes tokens at the current position; returns the logits of the last n_last of them
        ([n_last, vocab]).  Attention is causal, so row i equals what a token-by-token run that was
        fed tokens[: i + 1] would have produced at that position (teacher forcing in one pass)."""
        c = self.cfg
        W = lambda a: a.astype(np.float64) if a.dtype != np.float64 else a  # noqa: E731
        t, pos0 = len(tokens), self.pos
        x = W(self.embd[np.asarray(tokens, dtype=np.int64)])
        group = c.heads // c.kv_heads
        scale = float(np.float32(1.0) / np.sqrt(np.float32(c.head_dim)))
        f16 = lambda a: a.astype(np.float32).astype(np.float16).astype(np.float64)  # noqa: E731
        for L in self.layers:
            xn = self._rms(x, L["attn_norm"])
            q = self._rope(xn @ W(L["wq"]), c.heads, pos0).reshape(t, c.heads, c.head_dim)
            k = f16(self._rope(xn @ W(L["wk"]), c.kv_heads, pos0)).reshape(t, c.kv_heads, c.head_dim)
            v = f16(xn @ W(L["wv"])).reshape(t, c.kv_heads, c.head_dim)
            L["k"] = np.concatenate([L["k"], k]); L["v"] = np.concatenate([L["v"], v])
            K, V = L["k"], L["v"]
            out = np.empty((t, c.heads, c.head_dim))
            for h in range(c.heads):
                g = h // group
                s = (q[:, h, :] @ K[:, g, :].T) * scale          # [t, kv_len]
                kpos = np.arange(K.shape[0])[None, :]
                qpos = (pos0 + np.arange(t))[:, None]
                s = np.where(kpos <= qpos, s, -np.inf)
                s = s - s.max(axis=1, keepdims=True)
                p = np.exp(s)
                out[:, h, :] = (p @ V[:, g, :]) / p.sum(axis=1, keepdims=True)
            o = out.reshape(t, c.embd) @ W(L["wo"]) + x
            on = self._rms(o, L["ffn_norm"])
            up = on @ W(L["w_up"])
            gate = on @ W(L["w_gate"])
            act = gate / (1.0 + np.exp(-gate)) * up
            x = act @ W(L["w_down"]) + o
        self.pos += t
        last = self._rms(x[-n_last:], self.output_norm)
        return last @ W(self.lm_head)
