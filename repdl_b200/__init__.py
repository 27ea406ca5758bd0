"""repdl_b200 -- bit-reproducible operator backend for NVIDIA B200 (sm_100a).

A from-scratch replacement for the CUDA operator backend of microsoft/RepDL
(backend/cuda/*, bound in backend/cuda/bind.cpp:6-19 and called from repdl/ops.py:12-157).
`repdl_b200.ops` mirrors the reference's `repdl.ops` names and argument meaning;
`repdl_b200.install()` registers the PyTorch extension as `repdl.backend.cuda` so the reference's
own Python layers run on top of these kernels unchanged.
"""
from . import _cabi  # noqa: F401  (raises if the CUDA library is missing)
from . import ops  # noqa: F401
from .dropin import install  # noqa: F401

__all__ = ["ops", "install"]
