"""Generates tests/golden/golden.json.

The reference is Rust + GLSL and cannot be run here, so these vectors are not
reference outputs: they are computed by an INDEPENDENT pure-Python/numpy
restatement of the reference's fixture definitions (big-integer LCG, float64
GEMM + epilogue), separate from oracle/ta_oracle.c.  The C oracle and the CUDA
path are both checked against them.  Definitions followed:
  fill_det        tools/test-support/src/lib.rs:9-18
  LcgRng          tools/test-support/src/lib.rs:26-55
  cpu_bmm         tools/test-support/src/lib.rs:57-135
  epilogue        tests/correctness/epilogue.rs:9-47
Run:  python tests/golden/make_golden.py
"""
import json
import math
import os

import numpy as np

MASK = (1 << 64) - 1


def lcg_seed(seed):
    return ((seed * 0x9E3779B97F4A7C15) & MASK) | 1


def lcg_step(s):
    return (s * 6364136223846793005 + 1442695040888963407) & MASK


def fill_det(n, seed):
    s = lcg_seed(seed)
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = lcg_step(s)
        bits = s >> 40
        out[i] = np.float32(np.float32(np.float32(bits) / np.float32(1 << 24)) * np.float32(2.0)) - np.float32(1.0)
    return out


def lcg_ranges(seed, lo, hi, count):
    s = lcg_seed(seed)
    vals = []
    for _ in range(count):
        s = lcg_step(s)
        vals.append(lo + (s % (hi - lo + 1)))
    return vals


def act64(x, act):
    if act == "relu":
        return max(x, 0.0)
    if act == "silu":
        return x / (1.0 + math.exp(-x))
    if act == "gelu":
        return 0.5 * x * (1.0 + math.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))
    return x


def gemm_case(batch, m, n, k, seeds, alpha, act, bias_kind, binary, beta, b_shared):
    a = fill_det(batch * m * k, seeds[0]).reshape(batch, m, k)
    b = fill_det((1 if b_shared else batch) * k * n, seeds[1]).reshape(-1, k, n)
    out = np.empty((batch, m, n), dtype=np.float32)
    bias = None
    if bias_kind == "n":
        bias = fill_det(n, seeds[2]).reshape(1, n)
    elif bias_kind == "bn":
        bias = fill_det(batch * n, seeds[2]).reshape(batch, n)
    d = fill_det(batch * m * n, seeds[3]).reshape(batch, m, n) if binary != "none" else None
    for bi in range(batch):
        acc = a[bi].astype(np.float64) @ b[0 if b_shared else bi].astype(np.float64)
        c = (np.float32(alpha) * acc.astype(np.float32)).astype(np.float32)
        for i in range(m):
            for j in range(n):
                x = float(c[i, j])
                if bias is not None:
                    x += float(bias[bi if bias_kind == "bn" else 0, j])
                x = act64(x, act)
                if binary == "add_scaled":
                    x += float(np.float32(beta)) * float(d[bi, i, j])
                elif binary == "mul":
                    x *= float(d[bi, i, j])
                out[bi, i, j] = np.float32(x)
    return out


def main():
    g = {"fill_det": {}, "lcg_range": {}, "gemm": []}
    for seed in (0, 1, 2, 7, 42, 71, 0xC0FFEE):
        g["fill_det"][str(seed)] = [float(v) for v in fill_det(16, seed)]
    g["lcg_range"]["0xC0FFEE:1:300"] = lcg_ranges(0xC0FFEE, 1, 300, 24)
    cases = [
        dict(batch=1, m=33, n=20, k=47, seeds=[71, 72, 74, 75], alpha=1.0, act="gelu", bias_kind="n",
             binary="add_scaled", beta=0.75, b_shared=True),
        dict(batch=3, m=8, n=12, k=16, seeds=[91, 92, 93, 94], alpha=0.5, act="silu", bias_kind="bn",
             binary="mul", beta=0.0, b_shared=True),
        dict(batch=2, m=70, n=68, k=64, seeds=[11, 12, 13, 14], alpha=1.0, act="relu", bias_kind="none",
             binary="none", beta=0.0, b_shared=False),
    ]
    for c in cases:
        out = gemm_case(**c)
        flat = out.reshape(-1)
        idx = list(range(0, flat.size, max(1, flat.size // 97)))
        g["gemm"].append(dict(case=c, indices=idx, values=[float(flat[i]) for i in idx],
                              checksum=float(np.sum(flat.astype(np.float64)))))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.json")
    with open(path, "w") as f:
        json.dump(g, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
