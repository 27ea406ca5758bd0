"""GPU: the multi-tensor optimizer kernels (repdl_b200.optim.Adam / SGD) reproduce, step by step, the
parameter hashes of the reference's own Adam (repdl/optim.py) run on CPU tensors and of the
two-rounding SGD update (tests/golden/optim_steps.json, written by tests/golden/make_golden.py optim),
and agree with the oracle's restatement."""
import json
import os

import pytest
import torch

import cases
import oracle

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden", "optim_steps.json")


def golden():
    with open(GOLD) as f:
        return json.load(f)


@pytest.mark.parametrize("name,wd,ams", cases.OPTIM_CONFIGS, ids=[c[0] for c in cases.OPTIM_CONFIGS])
def test_fused_adam_matches_reference_adam(name, wd, ams):
    from repdl_b200 import optim
    got = cases.run_optimizer(lambda ps: optim.Adam(ps, lr=0.01, weight_decay=wd, amsgrad=ams), device="cuda")
    assert got == golden()["adam_" + name]
    assert got == cases.run_oracle_adam(oracle, wd, ams)


def test_fused_sgd_matches_two_rounding_update():
    from repdl_b200 import optim
    got = cases.run_optimizer(lambda ps: optim.SGD(ps, lr=0.01), device="cuda")
    assert got == golden()["sgd"]
    assert got == cases.run_oracle_sgd(oracle)


def test_more_tensors_than_one_launch_takes_and_special_values():
    """60 tensors (three launches of 24 + 24 + 12), empty tensors among them, and gradients with inf,
    NaN and zeros: the fused Adam equals the oracle on every tensor."""
    from repdl_b200 import optim
    g = torch.Generator().manual_seed(4)
    shapes = [(0,) if i % 13 == 5 else (1 + (i * 37) % 211,) for i in range(60)]
    params = [torch.randn(*s, generator=g) for s in shapes]
    ps = [torch.nn.Parameter(p.clone().cuda()) for p in params]
    opt = optim.Adam(ps, lr=0.003, weight_decay=0.01, amsgrad=True)
    cpu = [p.clone() for p in params]
    ms, vs, vm = ([torch.zeros_like(p) for p in cpu] for _ in range(3))
    for step in range(1, 4):
        grads = [torch.randn(*s, generator=g) for s in shapes]
        if step == 2:
            grads[3][0] = float("inf")
            grads[7][-1] = float("nan")
            grads[9].zero_()
        for p, gr in zip(ps, grads):
            p.grad = gr.cuda()
        opt.step()
        for p, gr, m, v, vx in zip(cpu, grads, ms, vs, vm):
            oracle.adam_step(p, gr.contiguous(), m, v, step, lr=0.003, weight_decay=0.01, vmax=vx)
        for i, (a, b) in enumerate(zip(ps, cpu)):
            # NaNs must be NaNs in the same places; everything else bit for bit
            a = a.detach().cpu()
            assert torch.equal(torch.isnan(a), torch.isnan(b)), (step, i)
            keep = ~torch.isnan(b)
            assert torch.equal(a[keep].view(torch.int32), b[keep].view(torch.int32)), (step, i)
