"""Shared fixtures.  GPU tests are marked ``gpu`` and call through the C ABI;
everything else runs on a machine without a GPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def orc():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def ta():
    """The package; builds the shared library first when it is missing."""
    pkg_lib = os.path.join(entry.PKG_DIR, "lib", "libtensor_ash.so")
    if not os.path.exists(pkg_lib):
        entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def gpu(ta):
    """(package, context, executor) on cuda:0 -- the analogue of the reference's
    tests/common/mod.rs:86-92 make_setup(2, 8) with tuning off."""
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 8, "auto", tune=False)
    yield ta, ctx, ex
    ex.close()
    ctx.close()


def upload_det(ta, ctx, ex, orc, shape, seed):
    """tests/common/mod.rs:48-61: create, fill_det(seed), upload; returns (tensor, host)."""
    import numpy as np

    t = ta.Tensor.uninit_device(ctx, shape)
    host = orc.fill_det(int(np.prod(shape)), seed)
    ex.upload(host, t)
    return t, host
