"""Host restatement (numpy, f64 accumulation) of the llama-architecture forward pass
the runner executes: f16-rounded weights from the documented seed streams, RMSNorm,
RoPE on interleaved pairs (2i, 2i+1) as the library's rope op defines them, GQA causal attention over an f16-rounded KV cache, SwiGLU MLP,
greedy argmax (first maximum).  Test infrastructure only.
"""
import numpy as np

CHUNK = 1 << 20


def chunk_seed(seed, tensor_id, chunk):
    return ((seed * 1000003 + tensor_id) * 4096 + chunk) & 0xFFFFFFFFFFFFFFFF


def gen_weight(orc, seed, tensor_id, rows, cols, sigma):
    n = rows * cols
    out = np.empty(n, dtype=np.float32)
    for c in range((n + CHUNK - 1) // CHUNK):
        lo, hi = c * CHUNK, min(n, (c + 1) * CHUNK)
        out[lo:hi] = orc.fill_normal((hi - lo,), chunk_seed(seed, tensor_id, c), sigma)
    return out.astype(np.float16).astype(np.float64).reshape(rows, cols)


def gen_norm(orc, seed, tensor_id, n, jitter):
    if jitter == 0.0:
        return np.ones(n)
    u = orc.fill_det(n, chunk_seed(seed, tensor_id, 0)).astype(np.float32)
    return (np.float32(1.0) + np.float32(jitter) * u).astype(np.float64)


class RefLlama:
    def __init__(self, orc, cfg):
        self.cfg = c = cfg
        s, sg = c.seed, c.weight_sigma
        kv_dim = c.kv_heads * c.head_dim
        self.embd = gen_weight(orc, s, 0, c.vocab, c.embd, sg)
        self.output_norm = gen_norm(orc, s, 1, c.embd, c.norm_jitter)
        self.lm_head = gen_weight(orc, s, 2, c.embd, c.vocab, sg)
        self.layers = []
        for li in range(c.layers):
            b = 16 + 16 * li
            self.layers.append(dict(
                attn_norm=gen_norm(orc, s, b + 0, c.embd, c.norm_jitter),
                wq=gen_weight(orc, s, b + 1, c.embd, c.embd, sg),
                wk=gen_weight(orc, s, b + 2, c.embd, kv_dim, sg),
                wv=gen_weight(orc, s, b + 3, c.embd, kv_dim, sg),
                wo=gen_weight(orc, s, b + 4, c.embd, c.embd, sg),
                ffn_norm=gen_norm(orc, s, b + 5, c.embd, c.norm_jitter),
                w_gate=gen_weight(orc, s, b + 6, c.embd, c.ffn, sg),
                w_up=gen_weight(orc, s, b + 7, c.embd, c.ffn, sg),
                w_down=gen_weight(orc, s, b + 8, c.ffn, c.embd, sg),
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

    def forward(self, tokens):
        """Consumes tokens at the current position; returns logits of the last one ([vocab])."""
        c = self.cfg
        t, pos0 = len(tokens), self.pos
        x = self.embd[np.asarray(tokens, dtype=np.int64)]
        group = c.heads // c.kv_heads
        scale = float(np.float32(1.0) / np.sqrt(np.float32(c.head_dim)))
        f16 = lambda a: a.astype(np.float32).astype(np.float16).astype(np.float64)  # noqa: E731
        for L in self.layers:
            xn = self._rms(x, L["attn_norm"])
            q = self._rope(xn @ L["wq"], c.heads, pos0).reshape(t, c.heads, c.head_dim)
            k = f16(self._rope(xn @ L["wk"], c.kv_heads, pos0)).reshape(t, c.kv_heads, c.head_dim)
            v = f16(xn @ L["wv"]).reshape(t, c.kv_heads, c.head_dim)
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
            o = out.reshape(t, c.embd) @ L["wo"] + x
            on = self._rms(o, L["ffn_norm"])
            up = on @ L["w_up"]
            gate = on @ L["w_gate"]
            act = gate / (1.0 + np.exp(-gate)) * up
            x = act @ L["w_down"] + o
        self.pos += t
        last = self._rms(x[-1:], self.output_norm)
        return (last @ self.lm_head)[0]
