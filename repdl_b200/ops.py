"""Operator layer: same names, argument order and result shapes as microsoft/RepDL's
repdl/ops.py:12-157, plus exp / log / sum (the reference keeps exp2d / log1d internal,
backend/cpu/math.cpp:19-47).  Every function takes CUDA fp32 tensors, allocates the result on the
input's device with torch, and enqueues one or two kernels of librepdl_b200.so on the current
stream.  CPU tensors are rejected: this package has no CPU path.
"""
from typing import Union

import torch

from ._cabi import check, lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(t, name, dim=None, dtype=torch.float32):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("repdl_b200 runs on CUDA tensors only; %s is on %s" % (name, t.device))
    if t.dtype != dtype:
        raise TypeError("%s must be %s, got %s" % (name, dtype, t.dtype))
    if dim is not None and t.dim() != dim:
        raise ValueError("%s must have %d dimensions, got %d" % (name, dim, t.dim()))
    return t


def _rowmajor(t):
    """A view/copy whose innermost stride is 1 and whose row pitch is usable as a leading dim."""
    if t.stride(1) == 1 and t.stride(0) >= max(1, t.shape[1]):
        return t
    return t.contiguous()


def mm(input: torch.Tensor, mat2: torch.Tensor, transA: bool = False,
       transB: bool = False) -> torch.Tensor:
    _need(input, "input", 2), _need(mat2, "mat2", 2)
    M = input.shape[1] if transA else input.shape[0]
    K = input.shape[0] if transA else input.shape[1]
    N = mat2.shape[0] if transB else mat2.shape[1]
    if (mat2.shape[1] if transB else mat2.shape[0]) != K:
        raise ValueError("mm: inner dimensions differ")
    a, b = _rowmajor(input), _rowmajor(mat2)
    out = torch.empty((M, N), dtype=torch.float32, device=input.device)
    with torch.cuda.device(input.device):
        check(lib.repdl_b200_mm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(transA),
                                int(transB), a.stride(0), b.stride(0), max(N, 1),
                                _stream(input)), "mm")
    return out


def _out_extent(size, pad, k, stride, what):
    if stride <= 0:
        raise ValueError(what + ": stride must be positive")
    if size + 2 * pad < k:
        raise ValueError(what + ": the kernel does not fit into the padded image")
    return (size + 2 * pad - k) // stride + 1


def conv2d(input, weight, stride, padding, groups, bias=None, relu=False) -> torch.Tensor:
    """conv2d of the reference (repdl/ops.py), optionally with the layer's epilogue in the same launch:
    `+ bias[oc]` (what Conv2dFunction.forward does next, repdl/nn/conv.py:27-28) and `max(., 0)` (a ReLU
    behind the layer); same bits as the separate element-wise kernels."""
    _need(input, "input", 4), _need(weight, "weight", 4)
    x, k = input.contiguous(), weight.contiguous()
    N, IC, H, W = x.shape
    OC, ICg, KH, KW = k.shape
    if ICg * groups != IC:
        raise ValueError("conv2d: weight.shape[1] * groups != input channels")
    OH = _out_extent(H, padding[0], KH, stride[0], "conv2d")
    OW = _out_extent(W, padding[1], KW, stride[1], "conv2d")
    out = torch.empty((N, OC, OH, OW), dtype=torch.float32, device=x.device)
    b = None
    if bias is not None:
        _need(bias, "bias", 1)
        if bias.shape[0] != OC or bias.device != x.device:
            raise ValueError("conv2d: bias must hold one value per output channel, on the input's device")
        b = bias.contiguous()
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_conv2d_bias_act(x.data_ptr(), k.data_ptr(), b.data_ptr() if b is not None else None,
                                             out.data_ptr(), N, IC, H, W, OC, KH, KW, stride[0], stride[1],
                                             padding[0], padding[1], groups, int(bool(relu)), _stream(x)), "conv2d")
    return out


def conv2d_grad_input(input_shape, weight, grad_output, stride, padding) -> torch.Tensor:
    _need(weight, "weight", 4), _need(grad_output, "grad_output", 4)
    k, go = weight.contiguous(), grad_output.contiguous()
    OC, IC, KH, KW = k.shape
    N = go.shape[0]
    H, W = int(input_shape[2]), int(input_shape[3])
    # the kernels index grad_output with the extents they derive from H and W: it must have them
    want = (N, OC, _out_extent(H, padding[0], KH, stride[0], "conv2d_grad_input"),
            _out_extent(W, padding[1], KW, stride[1], "conv2d_grad_input"))
    if tuple(go.shape) != want:
        raise ValueError("conv2d_grad_input: grad_output has shape %s, this convolution's output has %s"
                         % (tuple(go.shape), want))
    out = torch.empty((N, IC, H, W), dtype=torch.float32, device=go.device)
    with torch.cuda.device(go.device):
        check(lib.repdl_b200_conv2d_grad_input(go.data_ptr(), k.data_ptr(), out.data_ptr(), N, IC, H,
                                               W, OC, KH, KW, stride[0], stride[1], padding[0],
                                               padding[1], _stream(go)), "conv2d_grad_input")
    return out


def _check_grad_output(go, N, OC, H, W, KH, KW, stride, padding, what, weight_shape=None):
    if weight_shape is not None and (int(weight_shape[0]) != OC):
        raise ValueError("%s: grad_output has %d channels, the kernel %d" % (what, OC, int(weight_shape[0])))
    want = (N, OC, _out_extent(H, padding[0], KH, stride[0], what), _out_extent(W, padding[1], KW, stride[1], what))
    if tuple(go.shape) != want:
        raise ValueError("%s: grad_output has shape %s, this convolution's output has %s"
                         % (what, tuple(go.shape), want))


def conv2d_grad_kernel(input, weight_shape, grad_output, stride, padding) -> torch.Tensor:
    _need(input, "input", 4), _need(grad_output, "grad_output", 4)
    x, go = input.contiguous(), grad_output.contiguous()
    N, IC, H, W = x.shape
    OC = go.shape[1]
    KH, KW = int(weight_shape[2]), int(weight_shape[3])
    _check_grad_output(go, N, OC, H, W, KH, KW, stride, padding, "conv2d_grad_kernel", weight_shape)
    out = torch.empty((OC, IC, KH, KW), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_conv2d_grad_kernel(go.data_ptr(), x.data_ptr(), out.data_ptr(), N, IC,
                                                H, W, OC, KH, KW, stride[0], stride[1], padding[0],
                                                padding[1], _stream(x)), "conv2d_grad_kernel")
    return out


def conv2d_grad_kernel_bias(input, weight_shape, grad_output, stride, padding):
    """(conv2d_grad_kernel, sum4d_dim023(grad_output)) from one pass over grad_output, or None when
    the shape is not one the fused kernel takes (the caller then makes the two calls)."""
    _need(input, "input", 4), _need(grad_output, "grad_output", 4)
    x, go = input.contiguous(), grad_output.contiguous()
    N, IC, H, W = x.shape
    OC = go.shape[1]
    KH, KW = int(weight_shape[2]), int(weight_shape[3])
    _check_grad_output(go, N, OC, H, W, KH, KW, stride, padding, "conv2d_grad_kernel_bias", weight_shape)
    gw = torch.empty((OC, IC, KH, KW), dtype=torch.float32, device=x.device)
    gb = torch.empty((OC,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        status = lib.repdl_b200_conv2d_grad_kernel_bias(go.data_ptr(), x.data_ptr(), gw.data_ptr(),
                                                        gb.data_ptr(), N, IC, H, W, OC, KH, KW, stride[0],
                                                        stride[1], padding[0], padding[1], _stream(x))
    if status == -5:  # REPDL_E_UNSUPPORTED
        return None
    check(status, "conv2d_grad_kernel_bias")
    return gw, gb


def _factor(average, count):
    # backend/cpu/summation.cpp:15: float factor = average ? 1.0 / N : 1.0 (double division, then fp32)
    import numpy as np
    return float(np.float32(1.0 / count)) if average and count else 1.0


def sum1d(input: torch.Tensor, average: bool = False) -> torch.Tensor:
    x = _need(input, "input", 1).contiguous()
    n = x.numel()
    out = torch.empty((), dtype=torch.float32, device=x.device)
    nbytes = lib.repdl_b200_sum1d_scratch_bytes(n)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_sum1d(x.data_ptr(), out.data_ptr(), n, _factor(average, n),
                                   scratch.data_ptr(), nbytes, _stream(x)), "sum1d")
    return out


def sum2d_dim0(input: torch.Tensor, keepdim: bool = False, average: bool = False) -> torch.Tensor:
    x = _need(input, "input", 2).contiguous()
    M, N = x.shape
    out = torch.empty((1, N), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_sum2d_dim0(x.data_ptr(), out.data_ptr(), M, N, _factor(average, M),
                                        _stream(x)), "sum2d_dim0")
    return out if keepdim else out.squeeze()  # squeeze() drops every unit dim, as summation.cpp:38


def sum2d_dim1(input: torch.Tensor, keepdim: bool = False, average: bool = False) -> torch.Tensor:
    x = _need(input, "input", 2).contiguous()
    M, N = x.shape
    out = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_sum2d_dim1(x.data_ptr(), out.data_ptr(), M, N, _factor(average, N),
                                        _stream(x)), "sum2d_dim1")
    return out if keepdim else out.squeeze()


def sum4d_dim023(input: torch.Tensor, keepdim: bool = False, average: bool = False) -> torch.Tensor:
    x = _need(input, "input", 4).contiguous()
    N, C, H, W = x.shape
    out = torch.empty((1, C, 1, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_sum4d_dim023(x.data_ptr(), out.data_ptr(), N, C, H * W,
                                          _factor(average, N * H * W), _stream(x)), "sum4d_dim023")
    return out if keepdim else out.squeeze()


def sum(input: torch.Tensor, dim=None, keepdim: bool = False, average: bool = False) -> torch.Tensor:
    """Dispatches to the four fixed-order sums by rank and reduced dims."""
    if input.dim() == 1 and dim in (None, 0, (0,)):
        return sum1d(input, average)
    if input.dim() == 2 and dim in (0, (0,)):
        return sum2d_dim0(input, keepdim, average)
    if input.dim() == 2 and dim in (1, -1, (1,)):
        return sum2d_dim1(input, keepdim, average)
    if input.dim() == 4 and tuple(dim) == (0, 2, 3):
        return sum4d_dim023(input, keepdim, average)
    raise NotImplementedError("sum over dim=%r of a %d-d tensor" % (dim, input.dim()))


def _unary(fn, name, input):
    x = _need(input, "input").contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(fn(x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)), name)
    return out


def exp(input: torch.Tensor) -> torch.Tensor:
    return _unary(lib.repdl_b200_exp, "exp", input)


def log(input: torch.Tensor) -> torch.Tensor:
    return _unary(lib.repdl_b200_log, "log", input)


def sqrt(input: torch.Tensor) -> torch.Tensor:
    return _unary(lib.repdl_b200_sqrt, "sqrt", input)


def div(input: torch.Tensor, other: Union[torch.Tensor, float]) -> torch.Tensor:
    x = _need(input, "input").contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        if isinstance(other, torch.Tensor) and other.numel() != 1:
            d = _need(other, "other").expand_as(x).contiguous()
            check(lib.repdl_b200_div(x.data_ptr(), d.data_ptr(), out.data_ptr(), x.numel(),
                                     _stream(x)), "div")
        else:
            import numpy as np
            d = float(other) if not isinstance(other, torch.Tensor) else float(other.item())
            check(lib.repdl_b200_div_scalar(x.data_ptr(), float(np.float32(d)), out.data_ptr(),
                                            x.numel(), _stream(x)), "div")
    return out


def softmax(input: torch.Tensor) -> torch.Tensor:
    x = _need(input, "input", 2).contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_softmax(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                                     _stream(x)), "softmax")
    return out


def cross_entropy(input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    x = _need(input, "input", 2).contiguous()
    t = _need(target, "target", 1, torch.int64).contiguous()
    if t.shape[0] != x.shape[0]:
        raise ValueError("cross_entropy: target length != rows")
    out = torch.empty((), dtype=torch.float32, device=x.device)
    rows = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_cross_entropy(x.data_ptr(), t.data_ptr(), out.data_ptr(), x.shape[0],
                                           x.shape[1], rows.data_ptr(), _stream(x)), "cross_entropy")
    return out


def cross_entropy_grad(input: torch.Tensor, target: torch.Tensor, grad_loss: torch.Tensor) -> torch.Tensor:
    """Gradient of cross_entropy(input, target) with respect to input, times grad_loss (a scalar tensor):
    (softmax - one_hot) * float(1 / rows) * grad_loss with the three roundings of the reference's backward
    (repdl/nn/loss.py:29-33), in one launch.  Class indices must be valid (torch's one_hot would raise)."""
    x = _need(input, "input", 2).contiguous()
    t = _need(target, "target", 1, torch.int64).contiguous()
    if t.shape[0] != x.shape[0]:
        raise ValueError("cross_entropy_grad: target length != rows")
    g = _need(grad_loss.reshape(1), "grad_loss", 1).contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.repdl_b200_cross_entropy_grad(x.data_ptr(), t.data_ptr(), g.data_ptr(), out.data_ptr(), x.shape[0],
                                                x.shape[1], _stream(x)), "cross_entropy_grad")
    return out


def _with_nvtx_ranges():
    """REPDL_B200_NVTX=1: every public operator runs inside an NVTX range named after it, so that a
    timeline profiler shows which operator each kernel belongs to (off by default: the ranges cost
    two host calls per operator)."""
    import functools
    import os
    if os.environ.get("REPDL_B200_NVTX", "0") != "1":
        return
    names = ["mm", "conv2d", "conv2d_grad_input", "conv2d_grad_kernel", "conv2d_grad_kernel_bias",
             "sum1d", "sum2d_dim0", "sum2d_dim1", "sum4d_dim023", "exp", "log", "sqrt", "div",
             "softmax", "cross_entropy"]

    def ranged(fn, label):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            torch.cuda.nvtx.range_push(label)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        return wrapper
    for n in names:
        globals()[n] = ranged(globals()[n], "repdl_b200." + n)


_with_nvtx_ranges()
