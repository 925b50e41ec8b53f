import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def qb():
    """The product package (ctypes binding of the C ABI)."""
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure)."""
    return entry.load_oracle()


@pytest.fixture(scope="session")
def ctx(qb):
    c = qb.Context(0)
    yield c
    c.close()


@pytest.fixture(autouse=True)
def _release_device_arrays(request):
    yield
    if "ctx" in request.fixturenames:
        c = request.getfixturevalue("ctx")
        c.sync()
        c.release_arrays()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CUDA kernels (oracle/_ref/libqw3ref.so), or None if not built."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libqw3ref.so")
    if not os.path.exists(path):
        return None
    return ctypes.CDLL(path)


def std_mt19937_uniform(rs, n, a, b):
    """n draws of std::uniform_real_distribution<float>(a, b) on a std::mt19937 (libstdc++):
    one 32-bit output per value, u = float(raw) / 2^32 (clamped below 1), x = u * (b - a) + a."""
    raw = rs._bit_generator.random_raw(n).astype(np.uint32)
    u = raw.astype(np.float32) / np.float32(4294967296.0)
    u = np.minimum(u, np.nextafter(np.float32(1.0), np.float32(0.0)))
    return (u * np.float32(b - a) + np.float32(a)).astype(np.float32)


def tiny_ocfg(orc, qb):
    return orc.ModelConfig(**qb.configs.tiny().as_dict())


@pytest.fixture(scope="session")
def ref_attn():
    """The reference's native decode attention (oracle/_ref/libqw3ref_attn.so, `make -C oracle ref-attn`), or None."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libqw3ref_attn.so")
    if not os.path.exists(path):
        return None
    return ctypes.CDLL(path)
