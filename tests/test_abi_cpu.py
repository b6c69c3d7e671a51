"""The C-ABI library loads without a GPU and exports every symbol the public
header declares; the Python loader's signature table covers the same set."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    src = open(os.path.join(ROOT, "include", "tlb200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tlb_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from cpp_tensorlib_b200 import _lib
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/tlb200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names


def test_no_compute_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from cpp_tensorlib_b200 import TlbError, check, lib
    assert lib().tlb_device_count() == 0
    with pytest.raises(TlbError):
        check(lib().tlb_init(0))
    assert lib().tlb_q4_bytes(4864, 896) == 2179072 + 544768  # include/types.h:29-31
