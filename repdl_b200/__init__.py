"""repdl_b200 -- bit-reproducible operator backend for NVIDIA B200 (sm_100a).

A from-scratch replacement for the CUDA operator backend of microsoft/RepDL
(backend/cuda/*, bound in backend/cuda/bind.cpp:6-19 and called from repdl/ops.py:12-157).
`repdl_b200.ops` mirrors the reference's `repdl.ops` names and argument meaning;
`repdl_b200.install()` registers the PyTorch extension as `repdl.backend.cuda` so the reference's
own Python layers run on top of these kernels unchanged.

Submodules load on first use (so that `python -m repdl_b200.build` can run before the shared
library exists); touching `ops` without a built librepdl_b200.so raises ImportError -- there is no
fallback implementation.
"""
import importlib

__all__ = ["ops", "install", "workloads", "build"]


def install():
    from .dropin import install as _install
    return _install()


def __getattr__(name):
    if name in ("ops", "workloads", "build", "_cabi", "dropin", "nn", "optim", "dist"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
