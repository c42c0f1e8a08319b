"""Builds tests/c_abi_smoke.c with gcc against include/tensor_ash.h, links it to
the library and runs it on the GPU: the C-level acceptance test of the drop-in
boundary (the reference's counterpart is examples/c_smoke.c)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_smoke(tmp_path, ta):
    from tensor_ash_b200 import capi
    exe = tmp_path / "c_abi_smoke"
    libdir = os.path.dirname(capi.lib_path())
    subprocess.run(["gcc", "-std=c99", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "c_abi_smoke.c"), "-o", str(exe), "-L", libdir,
                    "-ltensor_ash", f"-Wl,-rpath,{libdir}", "-lm"], check=True)
    return exe


def test_c_program_compiles_and_links(tmp_path, ta):
    assert build_smoke(tmp_path, ta).exists()


@pytest.mark.gpu
def test_c_program_runs(tmp_path, ta):
    exe = build_smoke(tmp_path, ta)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "smoke OK" in out.stdout
