"""GPU: configuration 4 -- the CNN training step (conv, ReLU, conv, ReLU, max-pool, flatten, linear,
ReLU, linear, cross entropy; SGD lr 0.01; batch 256; the same batch every step) -- must reproduce,
step by step, the hashes the reference's own Python layers produced on its CPU backend
(tests/golden/cnn_steps.json, written by tests/golden/make_golden.py cnn)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "cnn_steps.json")


def _hash_params(model):
    import hashlib
    h = hashlib.sha256()
    for p in model.parameters():
        h.update(p.data.cpu().numpy().tobytes())
    return h.hexdigest()


def _train(model, loss_fn, x, y, steps, checkpoints):
    from cases import sha
    seen = {}
    for step in range(steps):
        for p in model.parameters():
            p.grad = None
        logits = model(x)
        loss = loss_fn(logits, y)
        loss.backward()
        with torch.no_grad():
            for p in model.parameters():
                p.add_(p.grad.mul(-0.01))
        if step in checkpoints:
            seen[step] = {"loss_hex": "%08x" % (loss.detach().cpu().view(torch.int32).item() & 0xFFFFFFFF),
                          "logits": sha(logits), "params": _hash_params(model)}
    return seen


@pytest.mark.skipif(not os.path.exists(GOLD), reason="cnn_steps.json not generated")
@pytest.mark.parametrize("fuse_relu", [False, True], ids=["layers_as_given", "relu_in_the_conv_epilogue"])
def test_cnn_training_matches_reference_cpu_hashes(fuse_relu):
    from cases import sha
    from repdl_b200 import nn as rnn
    from repdl_b200 import workloads
    gold = json.load(open(GOLD))
    torch.manual_seed(3)
    model = rnn.from_torch_module(workloads.cnn_torch_model(), fuse_relu=fuse_relu)
    assert sum(type(m) is torch.nn.Identity for m in model) == (2 if fuse_relu else 0)
    x, y = workloads.cnn_batch(256)
    assert [sha(x), sha(y)] == gold["input_sha256"]
    assert _hash_params(model) == gold["init_params"]
    model = model.cuda()
    loss_fn = rnn.CrossEntropyLoss()
    want = {s["step"]: s for s in gold["steps"]}
    seen = _train(model, loss_fn, x.cuda(), y.cuda(), 100, set(want))
    for step in sorted(want):
        for key in ("loss_hex", "logits", "params"):
            assert seen[step][key] == want[step][key], (step, key)
    with torch.no_grad():
        assert sha(model(x.cuda())) == gold["final_logits"]
    assert _hash_params(model) == gold["final_params"]


DROPIN = r"""
import json, sys, torch
sys.path.insert(0, {root!r})
import repdl_b200
ext = repdl_b200.install()                    # becomes repdl.backend.cuda
sys.path.insert(0, {site!r})
import repdl                                  # the reference's own, unmodified Python package
assert repdl.ops.cuda is ext
from repdl_b200 import workloads
sys.path.insert(0, {tests!r})
from cases import sha
torch.manual_seed(3)
model = repdl.from_torch_module(workloads.cnn_torch_model())
x, y = workloads.cnn_batch(256)
model = model.cuda(); x = x.cuda(); y = y.cuda()
loss_fn = repdl.nn.CrossEntropyLoss()
out = []
for step in range(3):
    for p in model.parameters():
        p.grad = None
    logits = model(x); loss = loss_fn(logits, y); loss.backward()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(p.grad.mul(-0.01))
    out.append(dict(step=step, logits=sha(logits), params=repdl.utils.get_hash(model)))
# the reference's Adam on top of these kernels runs too (repdl/optim.py)
opt = repdl.optim.Adam(model.parameters(), lr=0.01)
loss = loss_fn(model(x), y); opt.zero_grad(); loss.backward(); opt.step()
# batch norm (repdl/nn/batchnorm.py, repdl/func.py) is built from the same operators: the reference's
# own CPU backend and this package's CUDA backend must agree bit for bit, forward and backward
def bn_run(dev):
    torch.manual_seed(5)
    net = repdl.from_torch_module(torch.nn.Sequential(
        torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(), torch.nn.Flatten(),
        torch.nn.Linear(8 * 6 * 6, 4))).to(dev)  # (the reference's BatchNorm1d backward raises on its own CPU backend)
    xi = torch.rand(10, 3, 6, 6).to(dev); yi = torch.randint(0, 4, (10,)).to(dev)
    l = repdl.nn.CrossEntropyLoss()(net(xi), yi); l.backward()
    return [sha(l)] + [sha(p.grad) for p in net.parameters()]
bn_cpu, bn_gpu = bn_run("cpu"), bn_run("cuda")
print(json.dumps(dict(steps=out, bn_equal=bn_cpu == bn_gpu, bn_n=len(bn_cpu))))
"""


@pytest.mark.skipif(not os.path.exists(GOLD), reason="cnn_steps.json not generated")
def test_reference_python_layers_run_unchanged_on_the_dropin():
    """`repdl.from_torch_module`, `repdl.nn` and `repdl.optim` of the reference run unmodified with
    this package's extension installed as `repdl.backend.cuda`, and give the reference's hashes."""
    import oracle
    site = oracle.ref_site()
    if site is None:
        pytest.skip("the reference's Python package is not installed under oracle/_ref")
    code = DROPIN.format(root=ROOT, site=site, tests=os.path.join(ROOT, "tests"))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    got = json.loads(res.stdout.strip().splitlines()[-1])
    assert got["bn_equal"] and got["bn_n"] == 7, got
    got = got["steps"]
    want = {s["step"]: s for s in json.load(open(GOLD))["steps"]}
    for rec in got:
        assert rec["logits"] == want[rec["step"]]["logits"], rec["step"]
        assert rec["params"] == want[rec["step"]]["params"], rec["step"]


BN_DROPIN = r"""
import json, sys, torch
sys.path.insert(0, {root!r})
import repdl_b200
repdl_b200.install()
sys.path.insert(0, {site!r})
import repdl, repdl.func
sys.path.insert(0, {tests!r})
from cases import sha
res = {{}}
# the mean functions behind batch norm (repdl/func.py:47-121), forward and backward
g = torch.Generator().manual_seed(8)
for name, fn, shape in (("mean1d", repdl.func.mean1d, (4097,)), ("mean2d_dim0", repdl.func.mean2d_dim0, (129, 70)),
                        ("mean2d_dim0_wide", repdl.func.mean2d_dim0, (33, 1025)),
                        ("mean4d_dim023", repdl.func.mean4d_dim023, (9, 5, 13, 11)),
                        ("mean4d_dim023_big", repdl.func.mean4d_dim023, (16, 32, 26, 26))):
    x = (torch.randn(*shape, generator=g) * 3 + 0.5)
    w = torch.randn(*shape, generator=g)
    out = []
    for dev in ("cpu", "cuda"):
        xi = x.detach().clone().to(dev).requires_grad_(True)
        y = fn(xi)
        try:  # (the reference's own mean2d_dim0 backward raises on a shape error, on either backend)
            y.backward(torch.ones_like(y))
            gsha = sha(xi.grad)
        except RuntimeError:
            gsha = "backward raises"
        out.append((sha(y.detach()), gsha))
    res[name] = out[0] == out[1]
# BatchNorm2d of the reference on both backends: training steps (batch statistics, running statistics
# updated), then evaluation with the running statistics; several shapes
for tag, (N, C, H, W) in (("bn_small", (10, 8, 6, 6)), ("bn_odd", (7, 5, 9, 4)), ("bn_cnn", (32, 32, 26, 26)), ("bn_wide", (2, 3, 5, 40))):
    outs = []  # (one channel: the reference's own expand_as raises, on either backend)
    for dev in ("cpu", "cuda"):
        torch.manual_seed(11)
        bn = repdl.from_torch_module(torch.nn.Sequential(torch.nn.BatchNorm2d(C))).to(dev)
        gi = torch.Generator().manual_seed(12)
        rec = []
        for it in range(2):
            xi = (torch.randn(N, C, H, W, generator=gi) * 2 + 1).to(dev).requires_grad_(True)
            yi = bn(xi)
            yi.backward(torch.randn(N, C, H, W, generator=gi).to(dev))
            rec += [sha(yi.detach()), sha(xi.grad)] + [sha(p.grad) for p in bn.parameters()]
            with torch.no_grad():
                for p in bn.parameters():
                    p.add_(p.grad.mul(-0.1)); p.grad = None
        rec += [sha(b) for b in bn.buffers() if b.dtype == torch.float32]
        bn.eval()
        with torch.no_grad():
            rec.append(sha(bn((torch.randn(N, C, H, W, generator=gi)).to(dev))))
        outs.append(rec)
    res[tag] = outs[0] == outs[1]
print(json.dumps(res))
"""


def test_reference_batch_norm_and_means_on_the_dropin():
    """The reference's BatchNorm2d (repdl/nn/batchnorm.py:12-97) and the mean functions under it
    (repdl/func.py:47-121), unmodified, on this package's kernels: forward, backward, running
    statistics and evaluation mode give the bits of the reference's own CPU backend."""
    import oracle
    site = oracle.ref_site()
    if site is None:
        pytest.skip("the reference's Python package is not installed under oracle/_ref")
    code = BN_DROPIN.format(root=ROOT, site=site, tests=os.path.join(ROOT, "tests"))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    got = json.loads(res.stdout.strip().splitlines()[-1])
    assert len(got) == 9 and all(got.values()), got
