"""TEST INFRASTRUCTURE -- Python face of the CPU oracle (oracle/repdl_oracle.c).

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference leg of
bench.py may import this package.  It is the checker, never the product: the
CUDA library in repdl_b200/ neither imports nor links it.

Functions take and return CPU torch tensors (fp32, int64 targets) and mirror the
names of the reference's operator layer (repdl/ops.py:12-157) plus exp2d/log1d
(backend/cpu/math.cpp:19-47).  ``ref()`` returns the reference's own CPU backend
(oracle/_ref, built by oracle/build_ref.sh from the unmodified sources) when it
has been built, else None.
"""
import ctypes
import os
import sys

import torch

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        _lib = ctypes.CDLL(path)
        _lib.oracle_sum1d.restype = ctypes.c_float
        _lib.oracle_sum1d_carry.restype = ctypes.c_float
        _lib.oracle_cross_entropy.restype = ctypes.c_float
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return int(lib().oracle_num_threads())


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _i(v):
    return ctypes.c_int64(int(v))


def _f32(t):
    assert t.dtype == torch.float32 and t.device.type == "cpu", (t.dtype, t.device)
    return t


def mm(a, b, transA=False, transB=False):
    _f32(a), _f32(b)
    M = a.shape[1] if transA else a.shape[0]
    K = a.shape[0] if transA else a.shape[1]
    N = b.shape[0] if transB else b.shape[1]
    assert (b.shape[1] if transB else b.shape[0]) == K
    c = torch.empty(M, N)
    lib().oracle_mm(_p(a), _i(a.stride(0)), _i(a.stride(1)), _p(b), _i(b.stride(0)),
                    _i(b.stride(1)), _p(c), _i(M), _i(N), _i(K), int(transA), int(transB))
    return c


def conv2d(x, k, stride=(1, 1), padding=(0, 0), groups=1):
    x, k = _f32(x).contiguous(), _f32(k).contiguous()
    N, IC, H, W = x.shape
    OC, _, KH, KW = k.shape
    OH = (H + 2 * padding[0] - KH) // stride[0] + 1
    OW = (W + 2 * padding[1] - KW) // stride[1] + 1
    o = torch.empty(N, OC, OH, OW)
    lib().oracle_conv2d(_p(x), _p(k), _p(o), _i(N), _i(IC), _i(H), _i(W), _i(OC), _i(KH), _i(KW),
                        _i(stride[0]), _i(stride[1]), _i(padding[0]), _i(padding[1]), _i(groups))
    return o


def conv2d_grad_input(input_shape, k, go, stride=(1, 1), padding=(0, 0)):
    k, go = _f32(k).contiguous(), _f32(go).contiguous()
    OC, IC, KH, KW = k.shape
    N, _, OH, OW = go.shape
    H, W = input_shape[2], input_shape[3]
    gi = torch.empty(N, IC, H, W)
    lib().oracle_conv2d_grad_input(_p(go), _p(k), _p(gi), _i(N), _i(IC), _i(H), _i(W), _i(OC),
                                   _i(KH), _i(KW), _i(OH), _i(OW), _i(stride[0]), _i(stride[1]),
                                   _i(padding[0]), _i(padding[1]))
    return gi


def conv2d_grad_kernel(x, weight_shape, go, stride=(1, 1), padding=(0, 0)):
    x, go = _f32(x).contiguous(), _f32(go).contiguous()
    N, IC, H, W = x.shape
    _, OC, OH, OW = go.shape
    KH, KW = weight_shape[2], weight_shape[3]
    gk = torch.empty(OC, IC, KH, KW)
    lib().oracle_conv2d_grad_kernel(_p(go), _p(x), _p(gk), _i(N), _i(IC), _i(H), _i(W), _i(OC),
                                    _i(KH), _i(KW), _i(OH), _i(OW), _i(stride[0]), _i(stride[1]),
                                    _i(padding[0]), _i(padding[1]))
    return gk


def sum1d(x, average=False):
    x = _f32(x).contiguous()
    return torch.tensor(lib().oracle_sum1d(_p(x), _i(x.numel()), int(average)))


def sum1d_carry(x, carry):
    x = _f32(x).contiguous()
    return lib().oracle_sum1d_carry(_p(x), _i(x.numel()), ctypes.c_float(carry))


def _squeeze(out, keepdim):
    # backend/cpu/summation.cpp:38,57,77: squeeze() drops EVERY unit dimension
    return out if keepdim else out.squeeze()


def sum2d_dim0(x, keepdim=False, average=False):
    x = _f32(x).contiguous()
    M, N = x.shape
    out = torch.empty(1, N)
    lib().oracle_sum2d_dim0(_p(x), _p(out), _i(M), _i(N), int(average))
    return _squeeze(out, keepdim)


def sum2d_dim1(x, keepdim=False, average=False):
    x = _f32(x).contiguous()
    M, N = x.shape
    out = torch.empty(M, 1)
    lib().oracle_sum2d_dim1(_p(x), _p(out), _i(M), _i(N), int(average))
    return _squeeze(out, keepdim)


def sum4d_dim023(x, keepdim=False, average=False):
    x = _f32(x).contiguous()
    N, C, H, W = x.shape
    out = torch.empty(1, C, 1, 1)
    lib().oracle_sum4d_dim023(_p(x), _p(out), _i(N), _i(C), _i(H), _i(W), int(average))
    return _squeeze(out, keepdim)


def _unary(fn, x):
    x = _f32(x).contiguous()
    y = torch.empty_like(x)
    fn(_p(x), _p(y), _i(x.numel()))
    return y


def exp(x):
    return _unary(lib().oracle_exp, x)


def log(x):
    return _unary(lib().oracle_log, x)


def sqrt(x):
    return _unary(lib().oracle_sqrt, x)


def div(x, other):
    x = _f32(x).contiguous()
    y = torch.empty_like(x)
    if isinstance(other, torch.Tensor) and other.numel() > 1:
        d = _f32(other).expand_as(x).contiguous()
        lib().oracle_div(_p(x), _p(d), _p(y), _i(x.numel()), 0)
    else:
        d = torch.tensor([float(other)], dtype=torch.float32)
        lib().oracle_div(_p(x), _p(d), _p(y), _i(x.numel()), 1)
    return y


def softmax(x):
    x = _f32(x).contiguous()
    y = torch.empty_like(x)
    lib().oracle_softmax(_p(x), _p(y), _i(x.shape[0]), _i(x.shape[1]))
    return y


def cross_entropy(x, target):
    x = _f32(x).contiguous()
    t = target.to(torch.int64).contiguous()
    return torch.tensor(lib().oracle_cross_entropy(_p(x), _p(t), _i(x.shape[0]), _i(x.shape[1]),
                                                   None))


# --------------------------------------------------------------------------- #
# The reference itself (oracle/_ref), when built
# --------------------------------------------------------------------------- #
class _Ref:
    """Handles to the unmodified reference: .cpu (repdl.backend.cpu), .math
    (exp2d/log1d shim), .site (path to put on sys.path to import its `repdl`)."""

    def __init__(self, cpu, math, site):
        self.cpu, self.math, self.site = cpu, math, site


_ref = False


def ref_site():
    site = os.path.join(_HERE, "_ref", "site")
    return site if os.path.isdir(os.path.join(site, "repdl")) else None


def ref():
    """The reference's own CPU backend as built into oracle/_ref, or None."""
    global _ref
    if _ref is False:
        _ref = None
        site = ref_site()
        mpath = os.path.join(_HERE, "_ref", "refmath.so")
        if site and os.path.exists(mpath):
            import glob
            import importlib.util

            cands = glob.glob(os.path.join(site, "repdl", "backend", "cpu*.so"))
            if cands:
                spec = importlib.util.spec_from_file_location("repdl_ref_backend_cpu", cands[0])
                # the module's init symbol is PyInit_cpu
                spec = importlib.util.spec_from_file_location("cpu", cands[0])
                cpu = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(cpu)
                spec = importlib.util.spec_from_file_location("refmath", mpath)
                rm = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(rm)
                _ref = _Ref(cpu, rm, site)
    return _ref


def _f(v):
    """A Python scalar the way ATen hands it to an fp32 kernel."""
    return ctypes.c_float(float(torch.tensor(float(v), dtype=torch.float32)))


def sgd_step(p, g, lr):
    """In place on the fp32 CPU tensor p: p += g * -lr (two roundings)."""
    assert p.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous()
    lib().oracle_sgd_step(_p(p), _p(_f32(g)), _i(p.numel()), _f(-lr))


def adam_step(p, g, m, v, step, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, vmax=None):
    """One Adam.step of repdl/optim.py:56-83 for one parameter tensor, in place on p, m, v (and vmax
    with amsgrad); `step` is the 1-based step count."""
    import math
    for t in (p, g, m, v) + ((vmax,) if vmax is not None else ()):
        assert t.dtype == torch.float32 and t.is_contiguous()
    b1, b2 = betas
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    lib().oracle_adam_step(_p(p), _p(g), _p(m), _p(v), _p(vmax) if vmax is not None else None,
                           _i(p.numel()), _f(b1), _f(1 - b1), _f(b2), _f(1 - b2), _f(math.sqrt(bc2)),
                           _f(eps), _f(-(lr / bc1)), _f(weight_decay))
