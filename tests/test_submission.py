"""Concurrency, churn and failure reporting of the executor on the GPU
(tests/correctness/submission.rs:45-77,176-211 and tests/correctness/churn.rs:44-110 in the
reference), plus the bounded-wait self-test: a device-side wait that nothing completes must end in
an error the host reads, with the context still usable."""
import os
import threading

import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


def test_concurrent_submitters_share_one_executor(ta, orc):
    """8 threads, 4 slots: every thread uploads, multiplies and downloads its own matrices through the
    same executor and checks its own result (submission.rs:45-77)."""
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 4, 8)
    m = n = k = 64
    errors = []

    def worker(t):
        try:
            a, ha = upload_det(ta, ctx, ex, orc, (m, k), 10_000 + t)
            b, hb = upload_det(ta, ctx, ex, orc, (k, n), 20_000 + t)
            c = ta.Tensor.uninit_device(ctx, (m, n))
            ex.run_matmuls([ta.MatmulCall(a, b, c)])
            e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, m, n, k))
            assert e <= orc.tolerance(k), f"thread {t}: err {e}"
        except Exception as exc:  # noqa: BLE001
            errors.append((t, repr(exc)))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(8)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    ex.close()
    ctx.close()


def test_concurrent_heavy_load(ta, orc):
    """16 threads x 50 submissions on 4 slots (submission.rs:176-211); the tensor-core tile is in play
    (96 rows), so slots hand the status word, scratch and streams back and forth under contention."""
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 4, 4)
    m = n = k = 96
    errors = []

    def worker(t):
        try:
            a, ha = upload_det(ta, ctx, ex, orc, (m, k), 50_000 + t)
            b, hb = upload_det(ta, ctx, ex, orc, (k, n), 60_000 + t)
            c = ta.Tensor.uninit_device(ctx, (m, n))
            for _ in range(50):
                ex.run_matmuls([ta.MatmulCall(a, b, c)])
            e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, m, n, k))
            assert e <= orc.tolerance(k), f"thread {t}: err {e}"
        except Exception as exc:  # noqa: BLE001
            errors.append((t, repr(exc)))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(16)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    ex.close()
    ctx.close()


def one_cycle(ta, orc, out):
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 64)
    a, ha = upload_det(ta, ctx, ex, orc, (8, 8), 1)
    b, hb = upload_det(ta, ctx, ex, orc, (8, 8), 2)
    c = ta.Tensor.uninit_device(ctx, (8, 8))
    ex.run_matmuls([ta.MatmulCall(a, b, c)])
    e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, 8, 8, 8))
    assert e <= orc.tolerance(8)
    out.append(ctx.device_name)
    for t in (a, b, c):
        t.close()
    ex.close()
    ctx.close()


def test_context_churn_keeps_device_and_leaks_no_fds(ta, orc):
    """50 create / dispatch / destroy cycles, half of them on fresh threads (churn.rs:44-110): the
    device never changes and the count of open file descriptors settles."""
    names, fds = [], []
    for i in range(50):
        if i % 2:
            th = threading.Thread(target=one_cycle, args=(ta, orc, names))
            th.start()
            th.join()
        else:
            one_cycle(ta, orc, names)
        fds.append(len(os.listdir("/proc/self/fd")))
    assert len(names) == 50 and len(set(names)) == 1, set(names)
    assert fds[-1] <= fds[4] + 2, f"open fds grew from {fds[4]} to {fds[-1]}"


def test_bounded_wait_runs_out_without_faulting_anything(gpu, orc):
    """The kernel waits 5 ms on a barrier nothing completes, gives up, raises the status word and
    returns; the host call fails with the bounded-wait message; the next call on the same executor
    (same slots, same status words) succeeds and is correct."""
    ta, ctx, ex = gpu
    for _ in range(3):                       # every slot of the executor sees it at least once
        with pytest.raises(ta.TensorAshError, match="gave up on a bounded device-side wait"):
            ex.selftest_bounded_wait(5_000_000)
    a, ha = upload_det(ta, ctx, ex, orc, (128, 256), 71)
    b, hb = upload_det(ta, ctx, ex, orc, (256, 128), 72)
    c = ta.Tensor.uninit_device(ctx, (128, 128))
    for _ in range(3):
        ex.run_matmuls([ta.MatmulCall(a, b, c)])
    e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, 128, 128, 256))
    assert e <= orc.tolerance(256)
    with pytest.raises(ta.TensorAshError, match="out of range"):
        ex.selftest_bounded_wait(0)


def test_prepared_create_executes_nothing(gpu, orc):
    """Creating a prepared object records only (src/executor/graph_ops.rs:249-353): an accumulating op
    has been applied exactly once after the first run, not once more at create time."""
    ta, ctx, ex = gpu
    a, ha = upload_det(ta, ctx, ex, orc, (64, 64), 81)
    b, hb = upload_det(ta, ctx, ex, orc, (64, 64), 82)
    c = ta.Tensor.uninit_device(ctx, (64, 64))
    ex.upload(np.zeros(64 * 64, np.float32), c)
    ops = [ta.ExecOp.matmul(ta.MatmulOpEx(ta.MatmulCall(a, b, c, 1.0, True)))]
    prep = ex.prepare_exec_ops(ops)
    assert not ex.download(c).any(), "prepare_exec_ops executed the accumulating op at create time"
    prep.run()
    once = orc.cpu_bmm(ha, hb, 1, 64, 64, 64)
    e, _ = orc.max_abs_err(ex.download(c), once)
    assert e <= orc.tolerance(64)
    prep.run()
    e, _ = orc.max_abs_err(ex.download(c), 2.0 * once)
    assert e <= 2 * orc.tolerance(64)
    prep.close()
    prep2 = ex.prepare_ops([ta.MatmulOp(ta.MatmulCall(a, b, c, 1.0, True))])
    e, _ = orc.max_abs_err(ex.download(c), 2.0 * once)
    assert e <= 2 * orc.tolerance(64), "prepare_ops executed at create time"
    prep2.close()
