"""CPU: the C-ABI library loads, exports every symbol include/repdl_b200.h declares, and rejects
bad arguments before touching the GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "repdl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(repdl_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for name in ["repdl_b200_mm", "repdl_b200_conv2d", "repdl_b200_conv2d_grad_input",
                 "repdl_b200_conv2d_grad_kernel", "repdl_b200_sum1d", "repdl_b200_sum2d_dim0",
                 "repdl_b200_sum2d_dim1", "repdl_b200_sum4d_dim023", "repdl_b200_exp",
                 "repdl_b200_log", "repdl_b200_sqrt", "repdl_b200_div", "repdl_b200_div_scalar",
                 "repdl_b200_softmax", "repdl_b200_cross_entropy"]:
        assert name in syms


def test_library_exports_every_declared_symbol():
    from repdl_b200 import _cabi
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    # and the ctypes table covers every declaration
    assert sorted(_cabi.SIGNATURES) == declared_symbols()


def test_version_and_arch():
    from repdl_b200._cabi import lib
    assert lib.repdl_b200_version() >= 100
    assert lib.repdl_b200_sm_arch() == 100
    assert lib.repdl_b200_strerror(0) == b"success"
    assert b"NULL" in lib.repdl_b200_strerror(-1)


def test_argument_validation_needs_no_gpu():
    from repdl_b200._cabi import lib
    assert lib.repdl_b200_mm(None, None, None, -1, 4, 4, 0, 0, 4, 4, 4, None) == -2
    assert lib.repdl_b200_mm(None, None, None, 4, 4, 4, 0, 0, 4, 4, 4, None) == -1
    assert lib.repdl_b200_mm(None, None, None, 0, 4, 4, 0, 0, 4, 4, 4, None) == 0
    assert lib.repdl_b200_exp(None, None, -5, None) == -2
    assert lib.repdl_b200_exp(None, None, 0, None) == 0
    assert lib.repdl_b200_exp(None, None, 8, None) == -1
    assert lib.repdl_b200_conv2d(None, None, None, 1, 3, 8, 8, 4, 3, 3, 1, 1, 0, 0, 2, None) == -2
    assert lib.repdl_b200_cross_entropy(None, None, None, 4, 4, None, None) == -1


def test_ops_reject_cpu_tensors():
    import torch
    from repdl_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.mm(torch.zeros(2, 2), torch.zeros(2, 2))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.exp(torch.zeros(4))


def test_dropin_extension_exports_reference_names():
    """backend/cuda/bind.cpp:12-19 of the reference registers exactly these ten names."""
    from repdl_b200 import dropin
    mod = dropin.load_extension()
    for name in ["conv2d", "conv2d_grad_input", "conv2d_grad_kernel", "cross_entropy", "mm",
                 "softmax", "sum1d", "sum2d_dim0", "sum2d_dim1", "sum4d_dim023", "exp2d", "log1d"]:
        assert callable(getattr(mod, name))
