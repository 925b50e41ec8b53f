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
