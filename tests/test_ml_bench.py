"""The ml_bench tool (tools/ml-bench of the reference, on this library's C ABI).

CPU cases restate the reference's unit tests for the case parser and the sample summary
(tools/ml-bench/src/bench/cases.rs:170-245) and its environment switches (env.rs:58-108); GPU
cases run the subcommands and check the CSV columns, the route report and the validations.
"""
import csv
import io
import os
import subprocess

import pytest

import __graft_entry__ as entry


def ml_bench(*args, **env):
    exe = os.path.join(entry.PKG_DIR, "bin", "ml_bench")
    if not os.path.exists(exe):
        entry.build()
    e = dict(os.environ)
    for k in list(e):
        if k.startswith("ML_"):
            del e[k]
    e.update({k: str(v) for k, v in env.items()})
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=600, env=e)


def test_case_parser_validates_compact_specs():
    for bad, why in [("", "non-empty label"), ("odd,1,2,3", "missing K"), ("odd,1,2,0,4", "zero N"),
                     ("odd,1,2,3,4,5", "unknown flag '5'"), ("odd,1,2,3,4,f16w,x", "extra fields"),
                     ("odd,1,x,3,4", "invalid M='x'"), ("odd,1,-2,3,4", "invalid M='-2'")]:
        r = ml_bench("cases", bad)
        assert r.returncode != 0 and why in r.stderr, (bad, r.stderr)
    r = ml_bench("cases")
    assert r.returncode != 0 and "at least one label,b,m,n,k" in r.stderr
    r = ml_bench("frobnicate")
    assert r.returncode != 0 and "unknown subcommand 'frobnicate'" in r.stderr


def test_sample_summary_even_median_nearest_rank_p95_and_invalid_samples():
    assert ml_bench("summary").stdout.strip() == "none"
    assert ml_bench("summary", "nan", "inf", "-1").stdout.strip() == "none"
    assert ml_bench("summary", "2.5").stdout.strip() == "count=1 min=2.5 median=2.5 p95=2.5"
    r = ml_bench("summary", *[str(v) for v in range(20, 0, -1)])
    assert r.stdout.strip() == "count=20 min=1 median=10.5 p95=19"
    assert ml_bench("summary", "3", "nan", "1", "-2", "2").stdout.strip() == "count=3 min=1 median=2 p95=3"


CSV_COLUMNS = ("device,kind,label,b,m,n,k,flops,wall_ms,gpu_ms,tflops,percent_peak,sample_count,gpu_sample_count,"
               "wall_min_ms,wall_median_ms,wall_p95_ms,gpu_min_ms,gpu_median_ms,gpu_p95_ms,host_overhead_min_ms,"
               "host_overhead_median_ms,host_overhead_p95_ms,wall_tflops,kernel,tile_m,tile_n,tile_k,strategy,"
               "split_k2_splits").split(",")


@pytest.mark.gpu
def test_correctness_and_self_check():
    r = ml_bench("correctness")
    assert r.returncode == 0 and r.stdout.startswith("CORRECTNESS OK (err="), r.stderr
    r = ml_bench("correctness", ML_B=3, ML_M=129, ML_N=67, ML_K=515, ML_KERNEL="ffma")
    assert r.returncode == 0 and "CORRECTNESS OK" in r.stdout, r.stderr
    r = ml_bench("self-check", ML_SLOTS=3)
    assert r.returncode == 0 and "status: OK" in r.stdout and "executor_slots: 3" in r.stdout and "B200" in r.stdout


@pytest.mark.gpu
def test_cases_csv_has_the_reference_columns_and_routes():
    r = ml_bench("cases", "sq 512,1,512,512,512", "odd,2,129,67,515", "w16,1,256,512,256,f16w", "row,1,1,1024,1024,f16w",
                 ML_OUTPUT="CSV", ML_ITERS=5, ML_WARMUP=2, ML_PEAK_TFLOPS=100)
    assert r.returncode == 0, r.stderr
    rows = list(csv.reader(io.StringIO(r.stdout)))
    assert rows[0] == CSV_COLUMNS and len(rows) == 5
    rec = [dict(zip(CSV_COLUMNS, row)) for row in rows[1:]]
    assert [x["label"] for x in rec] == ["sq 512", "odd", "w16", "row"]
    assert rec[0]["kernel"].startswith("tf32x3") and rec[0]["strategy"] == "data_parallel" and rec[0]["split_k2_splits"] == ""
    assert rec[1]["kernel"].startswith("ffma_")                     # N = 67: no 16-byte rows, SIMT tiles
    assert rec[2]["kernel"].startswith("f16w_umma_") and "row_bda" in rec[3]["kernel"]
    for x in rec:
        assert int(x["sample_count"]) == 5 and int(x["gpu_sample_count"]) == 5
        assert float(x["flops"]) == 2.0 * int(x["b"]) * int(x["m"]) * int(x["n"]) * int(x["k"])
        assert float(x["gpu_min_ms"]) <= float(x["gpu_median_ms"]) <= float(x["gpu_p95_ms"])
        assert abs(float(x["percent_peak"]) - float(x["tflops"])) < 1e-2          # peak 100 -> % == TF/s
        assert "B200" in x["device"] and x["kind"] == "discrete"
    r = ml_bench("cases", "deep,1,64,64,8192", ML_OUTPUT="csv", ML_ITERS=3, ML_SPLIT_K2=8)
    assert r.returncode == 0, r.stderr
    x = dict(zip(CSV_COLUMNS, list(csv.reader(io.StringIO(r.stdout)))[1]))
    assert x["strategy"] == "split_k2" and x["split_k2_splits"] == "8"


@pytest.mark.gpu
def test_table_sweep_single_prepared_and_transfer():
    r = ml_bench("sweep", ML_SWEEP="SMOKE", ML_ITERS=3)
    assert r.returncode == 0, r.stderr
    assert "kernel / route" in r.stdout and "smoke 128^3 B=1" in r.stdout and "smoke 256^3 B=1" in r.stdout
    r = ml_bench("single", ML_M=512, ML_N=512, ML_K=512, ML_ITERS=3)
    assert r.returncode == 0 and "B=1 M=512 N=512 K=512" in r.stdout, r.stderr
    r = ml_bench("prepared", ML_ITERS=50, ML_WARMUP=5)
    assert r.returncode == 0, r.stderr
    assert "all outputs validated" in r.stdout and "prepared replay" in r.stdout and "pipelined x2" in r.stdout
    r = ml_bench("concurrent", ML_THREADS=6, ML_ITERS=20, ML_SLOTS=3)
    assert r.returncode == 0 and "concurrent: 6 threads x 20 iters of 512^3" in r.stdout, r.stderr
    r = ml_bench("transfer", ML_TRANSFER_MB=8, ML_ITERS=4)
    assert r.returncode == 0 and "transfer: 8 MiB x 4 samples" in r.stdout, r.stderr
    r = ml_bench("transfer", ML_TRANSFER_MB=8, ML_ITERS=4, ML_OUTPUT="csv")
    assert r.returncode == 0 and r.stdout.splitlines()[0].startswith("device,kind,bytes,iters,upload_gibs")


# ---- thesis harness (tools/ml-bench/src/bench/thesis/*.rs, benchmarks/THESES.md)
def test_thesis_expectations_parser(tmp_path):
    """expect.rs:114-136: sections, keys, comments; malformed lines are errors."""
    f = tmp_path / "e.toml"
    f.write_text('\n# top comment\n["NVIDIA GeForce RTX 3070"]\nmem_bw_gbps = 448.0   # spec sheet\nt3_barrier_us = 7.7\n\n'
                 '[bare-name]\nx = 1\n')
    r = ml_bench("thesis", "parse", str(f), "NVIDIA GeForce RTX 3070")
    assert r.returncode == 0 and r.stdout.splitlines() == ["mem_bw_gbps = 448", "t3_barrier_us = 7.7"], r.stdout + r.stderr
    assert ml_bench("thesis", "parse", str(f), "bare-name").stdout.strip() == "x = 1"
    assert "no section for 'unknown'" in ml_bench("thesis", "parse", str(f), "unknown").stdout
    for text, why in [("key = 1.0", "key before any [section]"), ("[sec]\nkey 1.0", "expected key = value"),
                      ("[sec]\nkey = fast", "value is not a number"), ("[unterminated\n", "unterminated section header")]:
        f.write_text(text)
        r = ml_bench("thesis", "parse", str(f), "sec")
        assert r.returncode != 0 and why in r.stderr, (text, r.stderr)


def test_thesis_options_and_committed_expectations():
    """mod.rs:365-378: selection and validation of thesis ids; the committed file has a B200 section."""
    r = ml_bench("thesis", "--list")
    assert r.returncode == 0 and all(f"  t{i}  " in r.stdout for i in (1, 2, 4, 6, 7))
    r = ml_bench("thesis", "t9")
    assert r.returncode != 0 and "unknown thesis 't9'" in r.stderr
    r = ml_bench("thesis", "--model")
    assert r.returncode != 0 and "--model needs a value" in r.stderr
    path = os.path.join(entry.PKG_DIR, "thesis-expectations.toml")
    r = ml_bench("thesis", "parse", path, "NVIDIA B200")
    keys = dict(line.split(" = ") for line in r.stdout.splitlines())
    assert {"mem_bw_gbps", "t1_min_bw_frac", "t2_min_bw_frac", "t6_min_tflops", "t6_ref_tflops"} <= set(keys)
    assert float(keys["mem_bw_gbps"]) > 1000


@pytest.mark.gpu
def test_thesis_kernel_level_rows_on_the_gpu():
    """t2, t4 and t6 need no model: every row is printed with a verdict and none FAILs against the
    committed B200 section (the tool's exit status is the gate)."""
    r = ml_bench("thesis", "t2", "t4", "t6", ML_ITERS=10)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "performance-thesis results" in r.stdout
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("| T")]
    assert sum(ln.startswith("| T2") for ln in lines) == 5 and sum(ln.startswith("| T6") for ln in lines) == 4
    assert not any("FAIL" in ln for ln in lines)
    assert all("umma" in ln for ln in lines if ln.startswith("| T6"))


@pytest.mark.gpu
def test_thesis_token_exactness_on_the_random_model():
    r = ml_bench("thesis", "t7", "--random")
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("| T7")]
    assert len(lines) == 4 and all("PASS" in ln and "17 / 17" in ln for ln in lines), r.stdout
