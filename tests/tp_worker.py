"""One rank of the tensor-parallel tests (started by tests/test_tp.py with RANK / WORLD_SIZE /
MASTER_* in the environment).  `cpu`: numpy shards + gloo collectives against the unsharded
host forward.  `gpu`: the sharded device runner against the single-GPU runner and the host."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
from llama_ref import RefLlama  # noqa: E402


def small_cfg(ta, **kw):
    base = dict(layers=2, embd=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024, t_max=96,
                weight_sigma=0.05, norm_jitter=0.25, seed=7)
    base.update(kw)
    return ta.LlamaConfig(**base)


class ShardedRef:
    """The host forward of one rank's shard; collectives where the device graph has them."""

    def __init__(self, ref: RefLlama, plan: dict, dist, torch):
        self.ref, self.p, self.dist, self.torch = ref, plan, dist, torch
        self.k = [np.zeros((0, plan["kv_l"], ref.cfg.head_dim)) for _ in ref.layers]
        self.v = [np.zeros((0, plan["kv_l"], ref.cfg.head_dim)) for _ in ref.layers]
        self.pos = 0

    def all_reduce(self, x):
        t = self.torch.from_numpy(np.ascontiguousarray(x))
        self.dist.all_reduce(t)
        return t.numpy()

    def forward(self, tokens):
        ref, p, c = self.ref, self.p, self.ref.cfg
        t, pos0 = len(tokens), self.pos
        x = ref.embd[np.asarray(tokens, dtype=np.int64)]
        scale = float(np.float32(1.0) / np.sqrt(np.float32(c.head_dim)))
        f16 = lambda a: a.astype(np.float32).astype(np.float16).astype(np.float64)  # noqa: E731
        q0, qw, kv0, kvw, f0, fl = p["q0"], p["q_w"], p["kv0"], p["kv_w"], p["f0"], p["ffn_l"]
        for li, L in enumerate(ref.layers):
            xn = ref._rms(x, L["attn_norm"])
            q = ref._rope(xn @ L["wq"][:, q0:q0 + qw], p["heads_l"], pos0).reshape(t, p["heads_l"], c.head_dim)
            k = f16(ref._rope(xn @ L["wk"][:, kv0:kv0 + kvw], p["kv_l"], pos0)).reshape(t, p["kv_l"], c.head_dim)
            v = f16(xn @ L["wv"][:, kv0:kv0 + kvw]).reshape(t, p["kv_l"], c.head_dim)
            self.k[li] = np.concatenate([self.k[li], k])
            self.v[li] = np.concatenate([self.v[li], v])
            K, V = self.k[li], self.v[li]
            out = np.empty((t, p["heads_l"], c.head_dim))
            for h in range(p["heads_l"]):
                g = h // p["group_l"]
                s = (q[:, h, :] @ K[:, g, :].T) * scale
                kpos = np.arange(K.shape[0])[None, :]
                qpos = (pos0 + np.arange(t))[:, None]
                s = np.where(kpos <= qpos, s, -np.inf)
                s = s - s.max(axis=1, keepdims=True)
                pr = np.exp(s)
                out[:, h, :] = (pr @ V[:, g, :]) / pr.sum(axis=1, keepdims=True)
            o = out.reshape(t, qw) @ L["wo"][q0:q0 + qw, :]
            if p["adds_residual"]:
                o = o + x
            o = self.all_reduce(o)
            on = ref._rms(o, L["ffn_norm"])
            up = on @ L["w_up"][:, f0:f0 + fl]
            gate = on @ L["w_gate"][:, f0:f0 + fl]
            act = gate / (1.0 + np.exp(-gate)) * up
            xo = act @ L["w_down"][f0:f0 + fl, :]
            if p["adds_residual"]:
                xo = xo + o
            x = self.all_reduce(xo)
        self.pos += t
        last = ref._rms(x[-1:], ref.output_norm)
        local = (last @ ref.lm_head[:, p["v0"]:p["v0"] + p["vocab_l"]])[0]
        parts = [self.torch.zeros(p["vocab_l"], dtype=self.torch.float64) for _ in range(self.dist.get_world_size())]
        self.dist.all_gather(parts, self.torch.from_numpy(np.ascontiguousarray(local)))
        return np.concatenate([q.numpy() for q in parts])


def main_cpu():
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ta = entry.load_package()
    orc = entry.load_oracle()
    cfg = small_cfg(ta, heads=4 if world <= 2 else 8, embd=256 if world <= 2 else 512)
    ref_full, ref_shard = RefLlama(orc, cfg), RefLlama(orc, cfg)
    sh = ShardedRef(ref_shard, ta.shard_plan(cfg, rank, world), dist, torch)
    prompt = [5, 900, 31, 64, 512, 77, 1]
    for step_tokens in (prompt, [3], [1000]):
        want = ref_full.forward(step_tokens)
        got = sh.forward(step_tokens)
        err = np.abs(got - want).max() / np.abs(want).max()
        assert err < 1e-12, f"rank {rank}: sharded host forward differs, rel {err:.3e}"
    # sharded greedy pick: every rank folds its vocabulary slice to one (value, global index) pair, the
    # ranks exchange the pairs and fold them with the same rule -- the maximum, ties to the LARGEST
    # index (shaders/op_argmax_f32.comp:44-75) -- so a tie that spans ranks resolves as on one device
    def fold(pairs):
        bv, bi = -np.inf, 0
        for v, i in pairs:
            if v > bv or (v == bv and i > bi):
                bv, bi = v, i
        return bv, bi

    vocab_l = 96
    full = np.random.default_rng(99).standard_normal(world * vocab_l).astype(np.float32)
    top = float(full.max()) + 1.0
    tie_at = [5, vocab_l + 7, (world - 1) * vocab_l + 3]         # the same maximum on the first, second and last rank
    full[tie_at] = top
    mine = full[rank * vocab_l:(rank + 1) * vocab_l]
    local = fold((float(v), rank * vocab_l + i) for i, v in enumerate(mine))
    gathered = [None] * world
    dist.all_gather_object(gathered, local)
    _, picked = fold(gathered)
    want = max(i for i, v in enumerate(full) if v == top)
    assert picked == want == max(tie_at), f"rank {rank}: sharded argmax picked {picked}, one device picks {want}"
    dist.barrier()
    dist.destroy_process_group()
    print("TP-CPU-OK", rank)


def main_gpu():
    import torch
    import torch.distributed as dist
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    world = dist.get_world_size()
    ta = entry.load_package()
    orc = entry.load_oracle()
    cfg = small_cfg(ta, heads=4 if world <= 2 else 8, embd=256 if world <= 2 else 512)
    ctx = ta.Context(False, f"index:{rank}")
    ex = ta.Executor(ctx, 2, 256)
    comm = ta.Comm.from_torch_distributed(ctx)
    assert comm.world == world and comm.rank == rank
    model = ta.Llama(ex, cfg, comm)
    ref = RefLlama(orc, cfg)
    prompt = [5, 900, 31, 64, 512, 77, 1]
    nxt, _ = model.prefill(prompt)
    want = ref.forward(prompt)
    got = model.logits().astype(np.float64)
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err <= 2e-4, f"rank {rank}: prefill logits rel err {err:.3e}"
    assert nxt == int(np.argmax(want))
    toks, _ = model.decode(nxt, 16)
    fed = nxt
    for i in range(16):
        want = ref.forward([fed])
        top = np.sort(want)[-2:]
        if top[1] - top[0] > 1e-3 * np.abs(want).max():
            assert toks[i] == int(np.argmax(want)), f"rank {rank} step {i}"
        fed = toks[i]
    # logits after sharded decode steps are gathered on demand and must match the host forward
    got = model.logits().astype(np.float64)
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err <= 2e-4, f"rank {rank}: decode logits rel err {err:.3e}"
    # the sharded argmax op on its own, with the same maximum placed on the first and the last rank
    vocab_l = 4000
    sl = np.random.default_rng(7 + rank).standard_normal(vocab_l).astype(np.float32)
    if rank == 0:
        sl[11] = 50.0
    if rank == world - 1:
        sl[123] = 50.0
    t_sl = ta.Tensor.uninit_device(ctx, (vocab_l,))
    ex.upload(sl, t_sl)
    cell = ta.PosCell(ctx)
    for _ in range(3):      # repeated uses advance the arrival words in step on every rank
        ex.run_exec_ops([ta.ExecOp.argmax_sharded(t_sl, rank * vocab_l, cell, comm)])
        assert cell.get() == (world - 1) * vocab_l + 123, f"rank {rank}: sharded argmax {cell.get()}"
    # all-reduce of prefill-sized activations (NCCL, or the two-step peer kernel under its switch): exact on integer-valued
    # inputs, repeated so that the per-CTA call counts advance, at a ragged and at the largest size
    for rows, cols in ((300, 256), (37, 1028), (512, 2048)):
        t_big = ta.Tensor.uninit_device(ctx, (rows, cols))
        base = (np.arange(rows * cols, dtype=np.int64) % 8191).astype(np.float32).reshape(rows, cols)
        for rep in range(3):
            ex.upload(base * (rank + 1) + rep, t_big)
            ex.run_exec_ops([ta.ExecOp.all_reduce(t_big, comm)])
            want_sum = base * (world * (world + 1) // 2) + rep * world
            assert np.array_equal(ex.download(t_big), want_sum), f"rank {rank}: all-reduce {rows}x{cols} rep {rep}"
        t_big.close()
    # every rank must hold the same token stream
    t = torch.tensor(toks, dtype=torch.int64, device="cuda")
    ref_t = t.clone()
    dist.broadcast(ref_t, src=0)
    assert torch.equal(t, ref_t), f"rank {rank}: token stream differs from rank 0"
    dist.barrier()
    model.close()
    comm.close()
    dist.destroy_process_group()
    print("TP-GPU-OK", rank)


def main_wait():
    """A bounded wait of the peer exchange runs out without faulting anything: rank 1 sits one
    all-reduce out (a host-side choice, nothing of it is in flight), rank 0's kernel gives up after
    5 ms, its call fails with the peer-wait message, and after a collective resync the next matched
    all-reduce is correct on both ranks."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    ta = entry.load_package()
    ctx = ta.Context(False, f"index:{rank}")
    ex = ta.Executor(ctx, 2, 16)
    comm = ta.Comm.from_torch_distributed(ctx)
    n = 2048
    t = ta.Tensor.uninit_device(ctx, (1, n))
    mine = np.arange(n, dtype=np.float32) * (rank + 1)
    ex.upload(mine, t)
    ex.run_exec_ops([ta.ExecOp.all_reduce(t, comm)])                      # a matched call first
    assert np.array_equal(ex.download(t).reshape(-1), np.arange(n, dtype=np.float32) * 3)
    dist.barrier()
    comm.set_wait_limit_ns(5_000_000)
    if rank == 0:
        ex.upload(mine, t)
        try:
            ex.run_exec_ops([ta.ExecOp.all_reduce(t, comm)])
            raise AssertionError("the unmatched all-reduce returned success")
        except ta.TensorAshError as exc:
            assert "wait for a peer rank" in str(exc), str(exc)
    dist.barrier()                                                         # rank 1 learns of it on the host
    comm.resync()
    comm.set_wait_limit_ns(10_000_000_000)
    ex.upload(mine, t)
    ex.run_exec_ops([ta.ExecOp.all_reduce(t, comm)])
    assert np.array_equal(ex.download(t).reshape(-1), np.arange(n, dtype=np.float32) * 3), f"rank {rank}: sum after resync"
    dist.barrier()
    t.close()
    comm.close()
    ex.close()
    dist.destroy_process_group()
    print("TP-WAIT-OK", rank)


if __name__ == "__main__":
    {"cpu": main_cpu, "gpu": main_gpu, "wait": main_wait}[sys.argv[1]]()
