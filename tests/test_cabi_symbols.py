"""CPU tests of the drop-in boundary: the library loads and exports what include/qw3b200.h declares."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qw3b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(qb):
    L = qb.lib()
    names = declared_symbols()
    assert len(names) >= 50
    for n in names:
        assert hasattr(L, n), "libqw3b200.so does not export " + n
    missing = [n for n in names if n not in qb.binding.SIGNATURES]
    assert not missing, "binding.py has no signature for " + ", ".join(missing)


def test_header_cites_reference_for_each_entry_point():
    text = open(os.path.join(ROOT, "include", "qw3b200.h")).read()
    assert text.count("src/") + text.count("device_backend.hpp") >= 25


def test_no_cpu_fallback_without_gpu(qb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(qb.QbError):
        qb.Context(0)


def test_oracle_is_not_reachable_from_the_product():
    pkg = os.path.join(ROOT, "kvmem-qw3_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cuh", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower() or f == "binding.py" and False, (dirpath, f)


def test_split_policy_of_library_and_oracle_agree(qb, orc):
    """The number of K segments fixes the fp32 summation order of every projection: the library's policy (a host
    function, no GPU needed) and the oracle's restatement must be the same function of the weight shape."""
    L = qb.lib()
    shapes = [(n, k) for n in (32, 96, 128, 256, 1024, 2048, 4096, 5120, 6144, 10240, 14336, 16480, 17408, 34816, 151936)
              for k in (128, 256, 512, 2176, 4352, 5120, 6144, 8704, 10240, 17408)]
    for n, k in shapes:
        assert L.qb_ksplit_policy(n, k) == orc.ksplit_policy(n, k), (n, k)
    assert L.qb_ksplit_policy(5120, 17408) == 7 and L.qb_ksplit_policy(16480, 5120) == 2 and L.qb_ksplit_policy(34816, 5120) == 1
