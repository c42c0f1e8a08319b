"""The measured tuner and its persistent store: host arithmetic and the store format
on CPU (ref src/executor/tuning.rs:319-374, src/pipeline/tuning.rs:60-199), one measured run on the
GPU under a private cache directory."""
import os

import pytest


def test_median_known_answers(ta):
    # src/executor/tuning.rs:350-355
    assert ta.tune_median([]) is None
    assert ta.tune_median([9, 1, 5]) == 5
    assert ta.tune_median([8, 2]) == 5
    assert ta.tune_median([3, 4]) == 3                      # mean of the middle pair, rounded down
    assert ta.tune_median([2**63, 2**63 + 2]) == 2**63 + 1  # no overflow in the pair sum


def test_candidate_order_is_balanced_in_measured_pairs(ta):
    # src/executor/tuning.rs:357-374
    for rnd in range(5):
        order = sorted(ta.tune_candidate_at(19, rnd, off) for off in range(19))
        assert order == list(range(19))
    for rounds in (2, 4):
        rank_sums = [0] * 19
        for rnd in range(1, rounds + 1):
            for rank in range(19):
                rank_sums[ta.tune_candidate_at(19, rnd, rank)] += rank
        assert all(s == rank_sums[0] for s in rank_sums)
    assert [ta.tune_candidate_at(5, 0, o) for o in range(5)] == [0, 1, 2, 3, 4]
    assert [ta.tune_candidate_at(5, 1, o) for o in range(5)] == [0, 1, 2, 3, 4]
    assert [ta.tune_candidate_at(5, 2, o) for o in range(5)] == [4, 3, 2, 1, 0]
    assert [ta.tune_candidate_at(5, 3, o) for o in range(5)] == [3, 4, 0, 1, 2]
    assert [ta.tune_candidate_at(5, 4, o) for o in range(5)] == [2, 1, 0, 4, 3]


def header_of(ta, tmp_path):
    """The header line this build writes: save an empty store and read it back."""
    empty_in, out = tmp_path / "none.txt", tmp_path / "hdr.txt"
    assert ta.tune_store_rewrite(str(empty_in), str(out)) == 0
    return out.read_text().splitlines()[0]


def test_store_round_trip_tokens_sorting_and_rejections(ta, tmp_path):
    hdr = header_of(ta, tmp_path)
    assert hdr.startswith("tensor-ash-tune-v3 ")
    src = tmp_path / "in.txt"
    src.write_text("\n".join([
        hdr,
        "1 4096 4096 4096 tf32x3_m128n256",
        "1 64 64 65536 ffma_m64n64 splitk2=64",
        "1 512 2048 2048 f16w_umma_m128n128 bf16",
        "1 512 2048 2048 tf32x3_m128n128",                 # same shape, f32 B: a separate key
        "1 8 8 8 no_such_kernel",                          # unknown kernel: skipped
        "garbage line",                                    # malformed: skipped
        "2 128 128 1024 ffma_m128n128 splitk2=1",          # split count outside 2..65535: dropped, entry kept
        "2 128 128 2048 ffma_m128n128 splitk2=70000",
    ]) + "\n")
    out = tmp_path / "out.txt"
    assert ta.tune_store_rewrite(str(src), str(out)) == 6
    lines = out.read_text().splitlines()
    assert lines[0] == hdr
    assert lines[1:] == [
        "1 64 64 65536 ffma_m64n64 splitk2=64",
        "1 512 2048 2048 tf32x3_m128n128",
        "1 512 2048 2048 f16w_umma_m128n128 bf16",
        "1 4096 4096 4096 tf32x3_m128n256",
        "2 128 128 1024 ffma_m128n128",
        "2 128 128 2048 ffma_m128n128",
    ]
    # a second pass is the identity
    again = tmp_path / "again.txt"
    assert ta.tune_store_rewrite(str(out), str(again)) == 6
    assert again.read_text() == out.read_text()
    # no temporary file is left behind
    assert sorted(p.name for p in tmp_path.iterdir()) == ["again.txt", "hdr.txt", "in.txt", "out.txt"]


def test_store_with_a_stale_header_is_discarded_whole(ta, tmp_path):
    src = tmp_path / "stale.txt"
    src.write_text("tensor-ash-tune-v3 backend=cuda-sm100a kernels=0000000000000000\n1 64 64 64 ffma_m64n64\n")
    assert ta.tune_store_rewrite(str(src)) == 0
    src.write_text("")
    assert ta.tune_store_rewrite(str(src)) == 0
    assert ta.tune_store_rewrite(str(tmp_path / "missing.txt")) == 0


def test_store_path_follows_xdg_cache_home(ta, tmp_path, monkeypatch):
    monkeypatch.setenv("XDG_CACHE_HOME", str(tmp_path))
    p = ta.tune_store_path("NVIDIA B200")
    assert p == str(tmp_path / "tensor-ash" / "tuned_kernels_cuda_nvidia_b200.txt")
    monkeypatch.delenv("XDG_CACHE_HOME")
    monkeypatch.setenv("HOME", str(tmp_path))
    assert ta.tune_store_path("x") == str(tmp_path / ".cache" / "tensor-ash" / "tuned_kernels_cuda_x.txt")


def test_experiment_switch_names(ta):
    ta.experiment_check("tf32x3_chunk_kb=32, peer_allreduce=0,gemv_ksplit=4")
    # every switch the integration notes list parses
    ta.experiment_check("tf32x3_ksplit=128,gemv_bulk=1,gemv_umma=0,gemv_handoff=0,gemv_peer_wide=0,f16w_pre=1,f16w_apad=0,"
                        "f16w_splitk=2,f16w_bn=128,f16w_tma_store=0,f16w_dual=0,attn_chunks=16,attn_pairs=0,attn_wide=0,flash_groups=1,"
                        "pos_stage=0,splitk2_tensor=0,pdl=0,peer_allreduce_big=1")
    ta.experiment_check("")
    with pytest.raises(ta.TensorAshError, match="unknown switch 'nope'"):
        ta.experiment_check("nope=1")
    with pytest.raises(ta.TensorAshError, match="not name=value"):
        ta.experiment_check("pdl")


@pytest.mark.gpu
def test_tune_persists_a_winner_and_routes_it(ta, orc, tmp_path, monkeypatch):
    """ta_executor_create_v2(tune=1) under a private XDG_CACHE_HOME: the first plain call of a shape
    measures the candidates, a line for the shape appears in the store, the executor (and a new one
    that loads the store) route the recorded kernel, and results stay correct.  f16-weight shapes
    are tuned too."""
    import numpy as np
    from conftest import upload_det

    monkeypatch.setenv("XDG_CACHE_HOME", str(tmp_path))
    ctx = ta.Context(False, "index:0")
    store = ta.tune_store_path(ctx.device_name)
    assert not os.path.exists(store)
    ex = ta.Executor(ctx, 2, 8, "auto", tune=True)
    m, n, k = 256, 384, 512
    a, ha = upload_det(ta, ctx, ex, orc, (m, k), 91)
    b, hb = upload_det(ta, ctx, ex, orc, (k, n), 92)
    c = ta.Tensor.uninit_device(ctx, (m, n))
    ex.run_matmuls([ta.MatmulCall(a, b, c)])             # first sight: tunes, then runs
    e, _ = orc.max_abs_err(ex.download(c), orc.cpu_bmm(ha, hb, 1, m, n, k))
    assert e <= orc.tolerance(k)
    lines = open(store).read().splitlines()
    mine = [ln for ln in lines[1:] if ln.startswith(f"1 {m} {n} {k} ")]
    assert len(mine) == 1, lines
    winner = mine[0].split()[4]
    assert winner in dict(ta.kernel_specs())
    info = ex.dispatch_info_for(1, m, n, k)
    assert info.kernel == winner or info.split_k2_splits
    # explicit call for an f16-weight shape
    ex.tune_shape(1, 128, 256, 512, b_f16=True)
    lines = open(store).read().splitlines()
    f16 = [ln for ln in lines[1:] if ln.startswith("1 128 256 512 ")]
    assert len(f16) == 1 and f16[0].endswith(" bf16") and f16[0].split()[4].startswith("f16w_"), lines
    ex.close()
    # a fresh executor without tuning loads the store and routes the recorded winners
    ex2 = ta.Executor(ctx, 2, 8, "auto", tune=False)
    assert ex2.dispatch_info_for(1, m, n, k).kernel == winner
    assert ex2.dispatch_info_for(1, 128, 256, 512, b_f16=True).kernel == f16[0].split()[4]
    bt = ta.Tensor.uninit_device_f16(ctx, (512, 256))
    at, hat = upload_det(ta, ctx, ex2, orc, (128, 512), 93)
    hbt = orc.fill_det(512 * 256, 94)
    ex2.upload(hbt, bt)
    ct = ta.Tensor.uninit_device(ctx, (128, 256))
    ex2.run_matmuls([ta.MatmulCall(at, bt, ct)])
    ref = orc.cpu_bmm(hat, orc.round_via_f16(hbt), 1, 128, 256, 512)
    assert np.abs(ex2.download(ct).reshape(-1) - ref.reshape(-1)).max() <= 2e-3 * max(1.0, np.abs(ref).max())
    ex2.close()
    ctx.close()
