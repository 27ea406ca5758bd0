"""Optimizers with a fixed, explicit operation order, one multi-tensor kernel per step.

`Adam` mirrors microsoft/RepDL's `repdl.optim.Adam` (repdl/optim.py:11-85): same constructor, same
state (`step`, `exp_avg`, `exp_avg_sq`, `max_exp_avg_sq`), and per element the same operations in
the same order with the same roundings -- but all parameter tensors of a group are updated by one
launch of `repdl_b200_adam_step` instead of about a dozen element-wise launches per tensor.

The reference ships no SGD.  `SGD` here is the plain update used by the CNN training
configuration: p <- p + (g * -lr), two separately rounded fp32 operations per element -- the style
of the reference's own update line (repdl/optim.py:83).  torch's `add_(g, alpha=-lr)` is avoided on
purpose: ATen evaluates it as ONE fused multiply-add on hosts and GPUs that have FMA.
"""
import ctypes
import math

import torch


def _f32(v):
    """A Python scalar the way ATen hands it to an fp32 kernel."""
    return float(torch.tensor(float(v), dtype=torch.float32))


def _ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _check_params(tensors, what):
    for t in tensors:
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise RuntimeError("%s: dense fp32 CUDA tensors only (this package has no CPU path)" % what)


def _by_device(params):
    groups = {}
    for p in params:
        groups.setdefault(p.device, []).append(p)
    return groups.items()


class SGD(torch.optim.Optimizer):
    def __init__(self, params, lr=0.01):
        super().__init__(params, dict(lr=lr))

    @torch.no_grad()
    def step(self, closure=None):
        from ._cabi import check, lib
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for dev, ps in _by_device([p for p in group["params"] if p.grad is not None]):
                grads = [p.grad.contiguous() for p in ps]
                _check_params(ps + grads, "SGD")
                sizes = (ctypes.c_int64 * len(ps))(*[p.numel() for p in ps])
                with torch.cuda.device(dev):
                    check(lib.repdl_b200_sgd_step(_ptr_array(ps), _ptr_array(grads), sizes, len(ps),
                                                  _f32(-group["lr"]),
                                                  torch.cuda.current_stream(dev).cuda_stream), "sgd_step")
        return loss


class Adam(torch.optim.Adam):
    @torch.no_grad()
    def step(self, closure=None):
        from ._cabi import check, lib
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            # the bias corrections depend on the step count, so tensors are batched per count
            batches = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients, please consider SparseAdam instead")
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    if group["amsgrad"]:
                        state["max_exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                state["step"] += 1
                batches.setdefault((p.device, state["step"]), []).append(p)
            for (dev, step), ps in batches.items():
                grads = [p.grad.contiguous() for p in ps]
                ms = [self.state[p]["exp_avg"] for p in ps]
                vs = [self.state[p]["exp_avg_sq"] for p in ps]
                vmax = [self.state[p]["max_exp_avg_sq"] for p in ps] if group["amsgrad"] else None
                _check_params(ps + grads + ms + vs + (vmax or []), "Adam")
                bias_correction1 = 1 - beta1 ** step
                bias_correction2 = 1 - beta2 ** step
                step_size = group["lr"] / bias_correction1
                sizes = (ctypes.c_int64 * len(ps))(*[p.numel() for p in ps])
                with torch.cuda.device(dev):
                    check(lib.repdl_b200_adam_step(
                        _ptr_array(ps), _ptr_array(grads), _ptr_array(ms), _ptr_array(vs),
                        _ptr_array(vmax) if vmax is not None else None, sizes, len(ps),
                        _f32(beta1), _f32(1 - beta1), _f32(beta2), _f32(1 - beta2),
                        _f32(math.sqrt(bias_correction2)), _f32(group["eps"]), _f32(-step_size),
                        _f32(group["weight_decay"]), torch.cuda.current_stream(dev).cuda_stream), "adam_step")
        return loss
