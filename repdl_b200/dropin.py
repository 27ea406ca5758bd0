"""Registers this package's PyTorch extension as `repdl.backend.cuda`.

microsoft/RepDL's operator layer imports its two backends with
`from .backend import cpu` / `from .backend import cuda` (repdl/ops.py:8-9) and dispatches on
`input.is_cuda`.  `install()` puts this package's extension module into `sys.modules` under the
name `repdl.backend.cuda` (and as the attribute `repdl.backend.cuda` once `repdl.backend` is
imported), so that an unmodified RepDL install -- `repdl.ops`, `repdl.nn`, `repdl.optim`,
`repdl.from_torch_module` -- runs its CUDA path on these kernels.  Call it BEFORE `import repdl`.
"""
import glob
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def load_extension():
    """Imports repdl_b200/backend/cuda*.so (module name `cuda`, init symbol PyInit_cuda)."""
    cands = sorted(glob.glob(os.path.join(_HERE, "backend", "cuda*.so")))
    if not cands:
        raise ImportError("repdl_b200: backend/cuda*.so is missing; build it with "
                          "`python -m repdl_b200.build` (there is no fallback)")
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("cuda", cands[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def install():
    """Makes `repdl.backend.cuda` resolve to this package's extension. Returns the module."""
    if "repdl.ops" in sys.modules:
        raise RuntimeError("repdl_b200.install() must run before `import repdl`")
    mod = load_extension()
    sys.modules["repdl.backend.cuda"] = mod

    class _Finder:
        """After `repdl.backend` is imported, expose the module as its `cuda` attribute."""

        @staticmethod
        def find_spec(name, path=None, target=None):
            if name == "repdl.backend.cuda":
                return importlib.util.spec_from_loader(name, _Loader())
            return None

    class _Loader:
        @staticmethod
        def create_module(spec):
            return mod

        @staticmethod
        def exec_module(module):
            return None

    sys.meta_path.insert(0, _Finder())
    return mod
