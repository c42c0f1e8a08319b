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


@pytest.mark.gpu
def test_reference_c_smoke_runs_unchanged(orc):
    """The reference's own acceptance program (examples/c_smoke.c:21-244), compiled unchanged from
    the reference tree by `make -C oracle ref_c_smoke` (the build step does it wherever that tree
    exists; the binary travels with the built libraries), passes against this library."""
    exe = orc.build_ref_c_smoke()
    if exe is None:
        pytest.skip("oracle/_ref/c_smoke was not built: the reference tree is not present on this machine")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "tensor-ash C smoke OK" in out.stdout
    for line in ("plain matmul OK", "bias+silu op OK", "prepared replay OK", "f16 matmul OK", "rms_norm OK",
                 "softmax(prefix=2) OK", "copy_strided transpose OK"):
        assert line in out.stdout, out.stdout
