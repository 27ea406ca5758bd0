"""Optimizers with a fixed, explicit operation order.

The reference ships only Adam (repdl/optim.py:11-85).  `SGD` here is the plain update used by the
CNN training configuration: p <- p + (g * -lr), written as two separately rounded fp32 operations
per element -- the style of the reference's own update line (repdl/optim.py:83).  torch's
`add_(g, alpha=-lr)` is avoided on purpose: ATen evaluates it as ONE fused multiply-add on hosts
and GPUs that have FMA, so its bits depend on where it runs.
"""
import torch


class SGD(torch.optim.Optimizer):
    def __init__(self, params, lr=0.01):
        super().__init__(params, dict(lr=lr))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    p.add_(p.grad.mul(-group["lr"]))
        return loss
