import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def built():
    """Builds the library and the oracle once per session (nvcc cross-compiles without a GPU)."""
    entry.build()
    return True


@pytest.fixture(scope="session")
def oracle_mod(built):
    return entry.load_oracle()


@pytest.fixture(scope="session")
def oracle(oracle_mod):
    return oracle_mod.Oracle()


@pytest.fixture(scope="session")
def ref_cpu(oracle_mod):
    """The reference's own CPU quantiser, when oracle/_ref was built (it needs the reference tree)."""
    try:
        return oracle_mod.RefCpu()
    except (FileNotFoundError, OSError):
        return None


@pytest.fixture(scope="session")
def pkg(built):
    return entry.load_package()


@pytest.fixture(scope="session")
def lib(pkg):
    return pkg.lib()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(GOLDEN, "nf4_golden.npz"))


def golden_names(npz):
    return sorted({k.rsplit(".", 1)[0] for k in npz.files})


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def glibc_uniform(seed, n, lo=-10.0, hi=10.0):
    """Input generator of the reference's quantiser tests (utils/random.hpp:8-35): glibc srand/rand."""
    import ctypes
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(ctypes.c_uint(seed))
    r = np.fromiter((libc.rand() for _ in range(n)), dtype=np.int64, count=n)
    u = r.astype(np.float32) / np.float32(2147483647)
    return (np.float32(lo) + u * np.float32(hi - lo)).astype(np.float32)


def make_c2_like(rows, cols, seed, outlier_frac=0.001):
    """Benchmark configuration 2: N(0,1) with a few columns scaled by U[20,100]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    ncol = max(1, int(round(outlier_frac * cols)))
    chosen = rng.choice(cols, size=ncol, replace=False)
    for c in chosen:
        x[:, c] *= np.float32(rng.uniform(20.0, 100.0))
    return x
