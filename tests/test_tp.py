"""Tensor-parallel llama: the sharding rule, the collective plumbing and the sharded graphs.

CPU (gloo, world_size 2, runs anywhere): every rank builds its shard of a small model on the
host with `shard_plan`, runs the sharded forward in numpy with `torch.distributed`
all-reduce / all-gather at exactly the points the device graph has its collectives, and must
reproduce the unsharded forward.  That pins the host-side logic of the N > 1 path: which
columns / rows / heads a rank owns, that rank 0 alone adds the residual, and the rank order of
the gathered logits.

GPU (needs >= 2 devices, skipped otherwise): the same model through
`ta_llama_create_random_tp` on 2 ranks against the single-GPU runner and the host forward.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "tp_worker.py")


def run_workers(mode: str, world: int, port: int, timeout: int = 600, **extra_env):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0", **extra_env)
    procs = []
    for rank in range(world):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, WORKER, mode], env=e, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append((p.returncode, out))
    return outs


def test_shard_plan_covers_every_column_once(ta):
    cfg = ta.LlamaConfig()   # 32 heads, 4 kv heads, ffn 5632, vocab 32000
    for world in (1, 2, 4, 8):
        plans = [ta.shard_plan(cfg, r, world) for r in range(world)]
        assert sum(p["q_w"] for p in plans) == cfg.embd
        assert [p["q0"] for p in plans] == [r * cfg.embd // world for r in range(world)]
        assert sum(p["ffn_l"] for p in plans) == cfg.ffn and sum(p["vocab_l"] for p in plans) == cfg.vocab
        assert sum(p["adds_residual"] for p in plans) == 1
        for r, p in enumerate(plans):
            # every query head of the rank must map to a kv head the rank holds
            group = cfg.heads // cfg.kv_heads
            for h in range(r * p["heads_l"], (r + 1) * p["heads_l"]):
                assert p["kv_first"] <= h // group < p["kv_first"] + p["kv_l"]
        if world <= cfg.kv_heads:
            assert sum(p["kv_w"] for p in plans) == cfg.kv_heads * cfg.head_dim
        else:
            assert all(p["kv_l"] == 1 for p in plans)
    with pytest.raises(ValueError):
        ta.shard_plan(cfg, 0, 3)


@pytest.mark.parametrize("world,port", [(2, 29611), (4, 29613)])
def test_sharded_forward_over_gloo_matches_unsharded(ta, orc, world, port):
    """world 4 on 2 kv heads exercises kv heads shared by neighbouring ranks."""
    outs = run_workers("cpu", world, port)
    for rc, out in outs:
        assert rc == 0, out
        assert "TP-CPU-OK" in out, out


@pytest.mark.gpu
@pytest.mark.parametrize("world,port", [(2, 29612), (4, 29614)])
def test_sharded_llama_on_devices_matches_host_forward(ta, orc, world, port):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    outs = run_workers("gpu", world, port)
    for rc, out in outs:
        assert rc == 0, out
        assert "TP-GPU-OK" in out, out


@pytest.mark.gpu
def test_two_step_peer_all_reduce_experiment_is_exact(ta, orc):
    """The same worker with the prefill-sized all-reduces routed to the two-step peer kernel (an
    experiment switch; NCCL carries them by default): integer-valued sums must be exact."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    outs = run_workers("gpu", 2, 29618, TA_EXPERIMENT="peer_allreduce_big=1")
    for rc, out in outs:
        assert rc == 0, out
        assert "TP-GPU-OK" in out, out


@pytest.mark.gpu
def test_peer_exchange_wait_runs_out_and_recovers(ta):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    outs = run_workers("wait", 2, 29616)
    for rc, out in outs:
        assert rc == 0, out
        assert "TP-WAIT-OK" in out, out
