"""The shared library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "skywalker_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skw_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from skywalker_b200 import _capi
    lib = _capi.load()
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), "library does not export %s" % n
        assert n in _capi.SIGNATURES, "python binding misses %s" % n
    assert sorted(_capi.SIGNATURES) == names


def test_no_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from skywalker_b200.api import Context, SkwError
    with pytest.raises(SkwError) as e:
        Context(0)
    assert "no CPU path" in str(e.value)


def test_khop_layout_needs_no_gpu():
    from skywalker_b200.api import Context
    assert Context.khop_layout([25, 10]) == (276, 26)
    assert Context.khop_layout([2, 2, 2]) == (15, 7)


def test_product_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "skywalker_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), os.path.join(dirpath, f)
