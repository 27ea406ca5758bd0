"""Reproducible layers on top of repdl_b200.ops.

Host-side mirror of the part of microsoft/RepDL's `repdl.nn` that the operator backend serves:
Linear (repdl/nn/linear.py:11-54), Conv2d (repdl/nn/conv.py:11-115), CrossEntropyLoss
(repdl/nn/loss.py:11-70) and `from_torch_module` (repdl/__init__.py:15-65).  Each autograd
function calls the same operators in the same order as the reference's, so a model converted with
this module and one converted with the reference's package produce identical bits.  Everything
that is not a repdl operator (ReLU, max-pooling, flatten, bias adds, one-hot) is a single IEEE
operation per element in torch and is left to torch, exactly as the reference does.
"""
from copy import copy

import torch

from . import ops


# Side streams for operator calls of one backward pass that do not depend on each other, per device.
_side = {}


def _concurrently(*thunks):
    """Launches each thunk (one operator call returning one tensor, or None) so that they may overlap.

    The weight gradient of a convolution is a few thousand long dependent FMA chains and the bias
    gradient a few dozen even longer add chains: both are bound by instruction latency and leave most
    of the GPU idle, and neither depends on the other or on the input gradient.  The first thunk runs
    on the current stream, the others on side streams that start after everything already queued on
    the current stream; the current stream then waits for them, so callers see ordinary stream
    semantics.  Every operator is deterministic on its own, so the bits do not depend on the overlap.
    """
    live = [i for i, t in enumerate(thunks) if t is not None]
    out = [None] * len(thunks)
    if len(live) <= 1:
        for i in live:
            out[i] = thunks[i]()
        return out
    main = torch.cuda.current_stream()
    key = (main.device.index, main.cuda_stream)
    slots = _side.setdefault(key, [])
    while len(slots) < len(live) - 1:
        slots.append((torch.cuda.Stream(device=main.device), torch.cuda.Event(), torch.cuda.Event()))
    ready = slots[0][1]
    ready.record(main)
    out[live[0]] = thunks[live[0]]()
    for (stream, _, done), i in zip(slots, live[1:]):
        stream.wait_event(ready)
        with torch.cuda.stream(stream):
            out[i] = thunks[i]()
        out[i].record_stream(main)   # allocated from the side stream's pool, consumed on the main one
        done.record(stream)
    for (_, _, done), _ in zip(slots, live[1:]):
        main.wait_event(done)
    return out


# Work of a backward pass that nothing else in that pass waits for (weight and bias gradients):
# side streams that are only joined when the backward pass ends.
_late = {}
_pending = []


def _join_deferred():
    """End-of-backward callback: the stream that ran the backward pass waits for the deferred work."""
    while _pending:
        main, done = _pending.pop()
        main.wait_event(done)


def _deferred(thunk, reads, params):
    """Runs thunk() -- operator calls whose results only the optimizer will read -- on a side stream
    and returns at once; the calling stream is made to wait for it when the backward pass ends
    (autograd's end-of-pass callbacks), so that the latency-bound weight-gradient chains of one layer
    overlap the backward of the layers below it.  Only used when the results are not consumed
    during the pass: every parameter in `params` must have no gradient yet (autograd then just
    keeps the tensor; accumulating into an existing gradient would read it at once).  Returns None
    if that does not hold, or outside a backward pass: the caller then computes in stream order.
    `reads` are the tensors the side stream reads: the allocator must not recycle them for this
    stream's later allocations before the side stream is done with them."""
    if any(p is not None and p.grad is not None for p in params):
        return None
    main = torch.cuda.current_stream()
    try:  # (queued on every deferral: the callback drains the list, extra calls find it empty)
        torch.autograd.Variable._execution_engine.queue_callback(_join_deferred)
    except Exception:  # not inside a backward pass of the autograd engine
        return None
    key = (main.device.index, main.cuda_stream)
    ring = _late.setdefault(key, {"streams": [torch.cuda.Stream(device=main.device) for _ in range(3)], "next": 0})
    stream = ring["streams"][ring["next"] % len(ring["streams"])]
    ring["next"] += 1
    ready = torch.cuda.Event()
    ready.record(main)
    stream.wait_event(ready)
    with torch.cuda.stream(stream):
        out = thunk()
    for t in reads:
        t.record_stream(stream)
    for t in (out if isinstance(out, (tuple, list)) else (out,)):
        if t is not None:
            t.record_stream(main)
    done = torch.cuda.Event()
    done.record(stream)
    _pending.append((main, done))
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.bias_ref = bias
        out = ops.mm(x, weight, transB=True)       # x [B,in] times weight[out,in]^T
        if bias is not None:
            out += bias
        return out

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = ops.mm(g, weight)

        def param_grads():
            w = ops.mm(g, x, transA=True) if ctx.needs_input_grad[1] else None
            b = ops.sum2d_dim0(g) if ctx.needs_input_grad[2] else None
            return w, b
        late = _deferred(param_grads, (g, x), (weight, ctx.bias_ref)) if ctx.needs_input_grad[1] else None
        gw, gb = late if late is not None else param_grads()
        return gx, gw, gb


def linear(x, weight, bias=None):
    if x.dim() != 2:
        raise NotImplementedError("linear expects a 2-d input")
    return _Linear.apply(x, weight, bias)


class Linear(torch.nn.Linear):
    def forward(self, x):
        return linear(x, self.weight, self.bias)


class _Conv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, groups, relu=False):
        ctx.bias_ref = bias
        ctx.cfg = (stride, padding, groups)
        ctx.relu = bool(relu)
        # the bias addition (repdl/nn/conv.py:27-28) and, if asked for, the ReLU behind the layer run in the
        # convolution's epilogue: the same separately rounded operations, two launches fewer each
        out = ops.conv2d(x, weight, stride, padding, groups, bias=bias, relu=relu)
        if relu:
            ctx.save_for_backward(x, weight, out)
        else:
            ctx.save_for_backward(x, weight)
        return out

    @staticmethod
    def backward(ctx, g):
        stride, padding, groups = ctx.cfg
        if groups != 1:
            raise NotImplementedError("grouped convolution has no backward (as in the reference)")
        if ctx.relu:
            x, weight, out = ctx.saved_tensors
            g = torch.ops.aten.threshold_backward(g, out, 0)  # what autograd runs for a ReLU module
        else:
            x, weight = ctx.saved_tensors
        need = ctx.needs_input_grad
        if need[1] and need[2]:
            # the weight / bias gradient chains go to a side stream that is only joined at the end
            # of the backward pass; the input gradient, which the layers below wait for, runs here
            late = _deferred(lambda: ops.conv2d_grad_kernel_bias(x, weight.shape, g, stride, padding),
                             (g, x), (weight, ctx.bias_ref))
            if late is not None:
                gx = ops.conv2d_grad_input(x.shape, weight, g, stride, padding) if need[0] else None
                return gx, late[0], late[1], None, None, None, None
        if need[1] and need[2]:
            # weight and bias gradient from one pass over g (the bias chain rides on the row operand of
            # the weight-gradient kernel); the input gradient overlaps on a side stream
            box = {}

            def fused():
                box["r"] = ops.conv2d_grad_kernel_bias(x, weight.shape, g, stride, padding)
                return box["r"][0] if box["r"] is not None else g.new_empty(0)
            _, gx = _concurrently(
                fused,
                (lambda: ops.conv2d_grad_input(x.shape, weight, g, stride, padding)) if need[0] else None)
            if box["r"] is not None:
                return gx, box["r"][0], box["r"][1], None, None, None, None
            gb, gw = _concurrently(
                lambda: ops.sum4d_dim023(g),
                lambda: ops.conv2d_grad_kernel(x, weight.shape, g, stride, padding))
            return gx, gw, gb, None, None, None, None
        # launch order matters: the two latency-bound operators first (measured on B200 for the second
        # layer of the CNN workload: 0.95 ms in this order, 1.22 ms with the weight gradient first, 1.34 ms
        # with the throughput-bound input gradient first, 1.38 ms one after the other)
        gb, gw, gx = _concurrently(
            (lambda: ops.sum4d_dim023(g)) if need[2] else None,
            (lambda: ops.conv2d_grad_kernel(x, weight.shape, g, stride, padding)) if need[1] else None,
            (lambda: ops.conv2d_grad_input(x.shape, weight, g, stride, padding)) if need[0] else None)
        return gx, gw, gb, None, None, None, None


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, relu=False):
    if isinstance(padding, str) or _pair(dilation) != (1, 1) or x.dim() != 4:
        raise NotImplementedError("conv2d: string padding, dilation and non-4-d inputs are unsupported")
    return _Conv2d.apply(x, weight, bias, _pair(stride), _pair(padding), groups, relu)


class Conv2d(torch.nn.Conv2d):
    fused_relu = False  # set by from_torch_module(..., fuse_relu=True) when a ReLU module follows the layer

    def forward(self, x):
        if self.padding_mode != "zeros":
            raise NotImplementedError("padding_mode must be 'zeros'")
        return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups,
                      self.fused_relu)


class _MaxPool2d(torch.autograd.Function):
    """max_pool2d over non-overlapping windows on the library's two streaming kernels (torch's backward
    kernel is written for overlapping windows).  Same maximum, same position for the gradient."""

    @staticmethod
    def forward(ctx, x, kh, kw):
        from ._cabi import check, lib
        x = x.contiguous()
        N, C, H, W = x.shape
        y = torch.empty((N, C, H // kh, W // kw), dtype=torch.float32, device=x.device)
        idx = torch.empty(y.shape, dtype=torch.int32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.repdl_b200_maxpool2d(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N * C, H, W, kh, kw,
                                           torch.cuda.current_stream(x.device).cuda_stream), "maxpool2d")
        ctx.save_for_backward(idx)
        ctx.geom = (tuple(x.shape), kh, kw)
        return y

    @staticmethod
    def backward(ctx, g):
        from ._cabi import check, lib
        (idx,) = ctx.saved_tensors
        shape, kh, kw = ctx.geom
        g = g.contiguous()
        gx = torch.empty(shape, dtype=torch.float32, device=g.device)
        with torch.cuda.device(g.device):
            check(lib.repdl_b200_maxpool2d_backward(g.data_ptr(), idx.data_ptr(), gx.data_ptr(), shape[0] * shape[1],
                                                    shape[2], shape[3], kh, kw,
                                                    torch.cuda.current_stream(g.device).cuda_stream),
                  "maxpool2d_backward")
        return gx, None, None


class MaxPool2d(torch.nn.MaxPool2d):
    def forward(self, x):
        k = _pair(self.kernel_size)
        s = _pair(self.stride if self.stride is not None else self.kernel_size)
        if (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and k == s and _pair(self.padding) == (0, 0)
                and _pair(self.dilation) == (1, 1) and not self.ceil_mode and not self.return_indices
                and x.shape[2] >= k[0] and x.shape[3] >= k[1] and x.numel() > 0):
            return _MaxPool2d.apply(x, k[0], k[1])
        return super().forward(x)  # overlapping or padded windows: torch's kernels


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        ctx.save_for_backward(logits, target)
        return ops.cross_entropy(logits, target)

    @staticmethod
    def backward(ctx, g):
        logits, target = ctx.saved_tensors
        gl = None
        if ctx.needs_input_grad[0]:
            # (softmax - one_hot) * (1/B) * g : three separately rounded steps (repdl/nn/loss.py:29-33),
            # in one launch
            gl = ops.cross_entropy_grad(logits, target, g)
        return gl, None


def cross_entropy(logits, target):
    if logits.dim() != 2 or target.dim() != 1:
        raise NotImplementedError("cross_entropy expects [B, C] logits and [B] class indices")
    return _CrossEntropy.apply(logits, target)


class CrossEntropyLoss(torch.nn.CrossEntropyLoss):
    def forward(self, logits, target):
        if (self.weight is not None or self.ignore_index != -100 or self.reduction != "mean"
                or self.label_smoothing != 0.0):
            raise NotImplementedError("only the plain mean-reduced cross entropy is implemented")
        return cross_entropy(logits, target)


_SWAPS = {torch.nn.Linear: Linear, torch.nn.Conv2d: Conv2d, torch.nn.CrossEntropyLoss: CrossEntropyLoss,
          torch.nn.MaxPool2d: MaxPool2d}


def from_torch_module(module, fuse_relu=False):
    """Returns a copy of `module` in which every torch.nn.Linear / Conv2d / CrossEntropyLoss (exact
    types only) is replaced by its reproducible twin sharing the same parameter values (and every
    torch.nn.MaxPool2d by one that runs non-overlapping windows on this library's kernels); Sequential
    containers are rebuilt and any other module is shallow-copied with converted children.

    fuse_relu: inside a Sequential, a torch.nn.ReLU (exact type, not in-place-sensitive: its input is
    not used elsewhere) that directly follows a Conv2d is folded into the convolution's epilogue and
    replaced by torch.nn.Identity (the indices of the other modules, and so the state_dict keys, do not
    change).  Same bits; one forward launch less per pair."""
    cls = _SWAPS.get(type(module))
    if cls is Linear:
        new = Linear(module.in_features, module.out_features, module.bias is not None,
                     device=module.weight.device, dtype=module.weight.dtype)
        new.load_state_dict(module.state_dict())
        return new
    if cls is Conv2d:
        new = Conv2d(module.in_channels, module.out_channels, module.kernel_size, module.stride,
                     module.padding, module.dilation, module.groups, module.bias is not None,
                     module.padding_mode, device=module.weight.device, dtype=module.weight.dtype)
        new.load_state_dict(module.state_dict())
        return new
    if cls is MaxPool2d:
        return MaxPool2d(module.kernel_size, module.stride, module.padding, module.dilation,
                         module.return_indices, module.ceil_mode)
    if cls is CrossEntropyLoss:
        return CrossEntropyLoss(weight=module.weight, ignore_index=module.ignore_index,
                                reduction=module.reduction, label_smoothing=module.label_smoothing)
    if type(module) is torch.nn.Sequential:
        mods = [from_torch_module(m, fuse_relu) for m in module]
        if fuse_relu:
            for i in range(len(mods) - 1):
                if type(mods[i]) is Conv2d and type(mods[i + 1]) is torch.nn.ReLU:
                    mods[i].fused_relu = True
                    mods[i + 1] = torch.nn.Identity()
        return torch.nn.Sequential(*mods)
    new = copy(module)
    new._modules = dict(new._modules)
    for name, child in module.named_children():
        new._modules[name] = from_torch_module(child, fuse_relu)
    return new
