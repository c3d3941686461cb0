"""The C-ABI library loads without a GPU and exports every entry point the header declares."""
import ctypes
import os
import re

import pytest

from colormlm_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "polaris_s14_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"S14_API\s+[^;(]*?\b(s14_\w+)\s*\(", text)))


def test_header_declares_what_python_binds():
    declared = _declared()
    assert len(declared) >= 70
    assert sorted(L.SIGNATURES) == declared


def test_library_exports_every_declared_symbol(cuda_lib):
    handle = ctypes.CDLL(L.LIB_PATH)
    missing = [name for name in _declared() if not hasattr(handle, name)]
    assert not missing, missing


def test_every_entry_point_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(os.path.join(ROOT, "include", "polaris_s14_cuda.h")).read()
    assert text.count(".rs:") + text.count(".py:") + text.count(".comp:") >= 30


def test_calls_fail_loudly_without_a_device(cuda_lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    rc = cuda_lib.s14_ctx_create(0, ctypes.byref(h))
    assert rc == L.ERR_CUDA or rc == L.ERR_CONTRACT
    assert cuda_lib.s14_last_error()
