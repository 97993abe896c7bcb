"""The C-ABI library loads without a GPU and exports what include/mgpt_moe.h declares."""
import ctypes as ct
import os
import re

import pytest

from mgpt_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mgpt_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgpt_moe_[a-z_0-9]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from mgpt_b200 import build
        build.build()
    return _lib.load()


def test_header_and_binding_agree():
    assert _declared() == sorted(_lib.SYMBOLS)


def test_every_declared_symbol_is_exported(lib):
    for name in _declared():
        assert hasattr(lib, name), name


def test_argument_checks_need_no_gpu(lib):
    h = ct.c_void_p()
    assert lib.mgpt_moe_create(None, ct.byref(h)) == 1
    bad = _lib.Config(16, 64, 4, 5, 0.01, 0, 0, 0)          # top_k > num_experts
    assert lib.mgpt_moe_create(ct.byref(bad), ct.byref(h)) == 1
    assert b"top_k" in lib.mgpt_moe_last_error()
    bad = _lib.Config(12, 64, 4, 2, 0.01, 0, 0, 0)          # embed_dim not a multiple of 8
    assert lib.mgpt_moe_create(ct.byref(bad), ct.byref(h)) == 1
    assert lib.mgpt_moe_num_params(None) == 0
    assert lib.mgpt_moe_workspace_bytes(None, 16) == 0
    assert lib.mgpt_moe_launch_count(1) >= 0


def test_no_silent_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ct.c_void_p()
    cfg = _lib.Config(16, 64, 4, 2, 0.01, 0, 0, 0)
    assert lib.mgpt_moe_create(ct.byref(cfg), ct.byref(h)) == 2      # MGPT_MOE_ECUDA
    from mgpt_b200 import MoELayer, MoeError
    with pytest.raises(MoeError):
        MoELayer(16, 64, 4, 2)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "mgpt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"import\s+oracle|from\s+oracle|liboracle|libmgpt_ref|oracle/|moe_oracle", src), f
