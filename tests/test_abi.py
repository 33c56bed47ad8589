"""The C-ABI library loads and exports every symbol include/tessel_b200.h declares (no
compute calls: there is no GPU here), and fails loudly without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "tessel_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from tessel_b200 import _lib
    names = declared()
    assert len(names) >= 20
    lib = _lib.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared but not exported"
    bound = {n for n, _, _ in _lib.SYMBOLS}
    assert bound == set(names), f"ctypes table and header disagree: {bound ^ set(names)}"


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from tessel_b200.gpu import Gpu, GpuError
    with pytest.raises(GpuError) as e:
        Gpu(0)
    assert "CUDA error" in str(e.value) or "device" in str(e.value)


def test_host_rng_matches_reference_generator():
    """tb200_rng_uniform is src/bench.rs:13-35 (checked against the oracle's restatement)."""
    import numpy as np
    import oracle
    from tessel_b200.model import Rng
    assert np.array_equal(Rng(12345).uniform(1000), oracle.Rng(12345).uniform(1000))
