"""ta_split_k2_noalloc: the split-K2 entry point for callers that cannot allocate.

Such callers (allocator callbacks, real-time or fault-handling paths, processes
whose device memory is fully budgeted at start-up) hand over plain device
pointers; the partial planes live in a fixed 4 MiB array inside the library's
device image.  The test calls the entry point twice in a row through the C ABI
and checks both results against ta_matmul_split_k2 on an executor that keeps the
same SIMT stage-1 kernel (so bitwise equal) and against the CPU oracle, and it
checks the property the entry point exists for: once the first call has been
made, further calls leave the device's free-memory figure (cudaMemGetInfo)
exactly where it was.  It lives in a file of its own that pytest collects last,
and it passes both alone in a fresh process and after the rest of the suite,
because it depends on no state left by other tests."""
import ctypes as C

import numpy as np
import pytest

from conftest import upload_det

pytestmark = pytest.mark.gpu


def free_device_bytes():
    import torch
    return torch.cuda.mem_get_info(0)[0]      # cudaMemGetInfo on the device both libraries share


def test_noalloc_matches_split_k2_twice_in_a_row(gpu, orc):
    ta, ctx, _ = gpu
    ex = ta.Executor(ctx, 2, 8, "split_k2_m64n64")      # ta_matmul_split_k2 on the same SIMT stage 1
    L = ta.lib()
    cases = [((64, 256, 4096), 64, 1.0), ((37, 41, 1088), 16, 0.75)]   # second call reuses the array
    for rep in range(2):
        for (m, n, k), splits, alpha in cases:
            a, ha = upload_det(ta, ctx, ex, orc, (m, k), 401 + rep)
            b, hb = upload_det(ta, ctx, ex, orc, (k, n), 402 + rep)
            c_ref = ta.Tensor.uninit_device(ctx, (m, n))
            c_new = ta.Tensor.uninit_device(ctx, (m, n))
            ex.run_matmuls_split_k2([ta.MatmulCall(a, b, c_ref, alpha)], splits)
            ex.upload(np.full(m * n, -3.0, np.float32), c_new)
            rc = L.ta_split_k2_noalloc(a.device_ptr, b.device_ptr, c_new.device_ptr, m, n, k, splits,
                                       C.c_float(alpha), None)
            assert rc == 0, L.ta_last_error().decode()
            got, want = ex.download(c_new), ex.download(c_ref)
            assert got.tobytes() == want.tobytes(), f"rep {rep} {m}x{n}x{k}: differs from ta_matmul_split_k2"
            e, _ = orc.max_abs_err(got, orc.cpu_bmm(ha, hb, 1, m, n, k, alpha=alpha))
            assert e <= 2.0 * orc.tolerance(k)
    ex.close()


def test_noalloc_calls_after_the_first_allocate_nothing(gpu, orc):
    ta, ctx, ex = gpu
    L = ta.lib()
    m, n, k, splits = 64, 128, 2048, 8
    a, _ = upload_det(ta, ctx, ex, orc, (m, k), 411)
    b, _ = upload_det(ta, ctx, ex, orc, (k, n), 412)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    args = (a.device_ptr, b.device_ptr, c.device_ptr, m, n, k, splits, C.c_float(1.0), None)
    assert L.ta_split_k2_noalloc(*args) == 0, L.ta_last_error().decode()   # may pay the lazy module load
    free_device_bytes()                                                     # the query's own first-use costs
    before = free_device_bytes()
    for _ in range(5):
        assert L.ta_split_k2_noalloc(*args) == 0, L.ta_last_error().decode()
        assert free_device_bytes() == before, "a call after the first changed the device's free memory"


def test_noalloc_rejects_what_does_not_fit(gpu, orc):
    ta, ctx, ex = gpu
    L = ta.lib()
    a = ta.Tensor.uninit_device(ctx, (128, 4096))
    b = ta.Tensor.uninit_device(ctx, (4096, 512))
    c = ta.Tensor.uninit_device(ctx, (128, 512))
    args = (a.device_ptr, b.device_ptr, c.device_ptr, 128, 512, 4096)
    assert L.ta_split_k2_noalloc(*args, 32, C.c_float(1.0), None) == -1      # 32*128*512 = 2 Mi floats
    assert "more than the fixed" in L.ta_last_error().decode()
    assert L.ta_split_k2_noalloc(*args, 16, C.c_float(1.0), None) == 0       # exactly 1 Mi floats fits
    assert L.ta_split_k2_noalloc(*args, 1, C.c_float(1.0), None) == -1
    assert L.ta_split_k2_noalloc(None, b.device_ptr, c.device_ptr, 128, 512, 4096, 4, C.c_float(1.0), None) == -1
    assert L.ta_split_k2_noalloc(a.device_ptr, b.device_ptr, c.device_ptr, 128, 512, 4, 8, C.c_float(1.0), None) == -1
    assert "exceeds K=4" in L.ta_last_error().decode()
