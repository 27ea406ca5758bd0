"""Small, seeded parity cases shared by the golden-fixture generator, the oracle tests (CPU) and
the CUDA parity tests (GPU).  Each case is (name, op, args-builder); inputs are rebuilt from the
seed wherever the case runs, so the fixtures only need to hold output hashes.

`run_case(impl, case)` evaluates a case on an implementation that exposes the operator names of
microsoft/RepDL's repdl/ops.py (the oracle package, the reference backend adapter below, or
repdl_b200.ops with tensors moved to the GPU).
"""
import hashlib

import torch


def sha(t):
    """SHA-256 of the tensor's bytes -- the comparator of the reference (repdl/utils.py:10-13)."""
    return hashlib.sha256(t.detach().cpu().contiguous().numpy().tobytes()).hexdigest()


def _g(seed):
    return torch.Generator().manual_seed(seed)


def _randn(seed, *shape, scale=1.0):
    return torch.randn(*shape, generator=_g(seed)) * scale


SPECIAL_BITS = [
    0x7F800001, 0xFFC12345, 0x7FA5A5A5, 0xFF800000, 0x7F800000, 0x00000000, 0x80000000, 0x00000001,
    0x80000001, 0x807FFFFF, 0x007FFFFF, 0x00800000, 0xC2B00000, 0x42B00000, 0xBF800000, 0x3F800000,
    0xFFFFFFFF, 0x7FFFFFFF, 0x41178FEB, 0xC16912CD, 0x42B17218, 0x42B17217, 0xC2CFF1B5, 0xC2CFF1B4,
    0xC2AEAC50, 0xC2AEAC4F, 0x3F7FFFFF, 0x3F800001, 0x7F7FFFFF, 0xFF7FFFFF, 0x33800000, 0xB3800000,
]


def special_values(extra_random=1 << 16, seed=11):
    bits = torch.tensor([b - (1 << 32) if b >= (1 << 31) else b for b in SPECIAL_BITS],
                        dtype=torch.int32)
    rnd = torch.randint(-2 ** 31, 2 ** 31, (extra_random,), generator=_g(seed), dtype=torch.int64)
    return torch.cat([bits, rnd.to(torch.int32)]).view(torch.float32)


def build_cases():
    cases = []
    # ---- mm: tails around the tile sizes, all four transposes --------------------------------
    shapes = [(1, 1, 1), (7, 5, 3), (33, 65, 17), (64, 64, 16), (65, 63, 15), (128, 128, 32),
              (129, 127, 33), (200, 72, 130), (256, 10, 128), (10, 128, 256), (300, 260, 47),
              (4, 4, 0),
              # few outputs over a long K: the thin-tile configuration with several slabs in flight
              (40, 70, 1100), (33, 31, 2049),
              # ragged edges of the two large-tile configurations (192 x 128 and 128 x 256 outputs per CTA)
              (2500, 3100, 37), (2040, 16380, 17)]
    for si, (M, N, K) in enumerate(shapes):
        for ta in (False, True):
            for tb in (False, True):
                def mk(M=M, N=N, K=K, ta=ta, tb=tb, si=si):
                    a = _randn(100 + si, *((K, M) if ta else (M, K)))
                    b = _randn(200 + si, *((N, K) if tb else (K, N)))
                    return (a, b, ta, tb)
                cases.append(("mm_%dx%dx%d_%d%d" % (M, N, K, ta, tb), "mm", mk))

    # tiny products that underflow to -0 and a K tail: the padded tail must not flip -0 to +0
    def mk_negzero():
        a = torch.full((5, 19), -1e-30)
        b = torch.full((19, 6), 1e-30)
        a[0, :] = 0.0
        return (a, b, False, False)
    cases.append(("mm_negzero_tail", "mm", mk_negzero))

    def mk_strided():
        a = _randn(301, 40, 100)[:, 10:58]       # row pitch 100, 48 columns
        b = _randn(302, 48, 80)[:, ::2]          # inner stride 2 -> copied by the wrapper
        return (a, b, False, False)
    cases.append(("mm_strided", "mm", mk_strided))

    # ---- conv -----------------------------------------------------------------------------------
    conv_cfgs = [
        # N, IC, H, W, OC, KH, KW, stride, padding, groups
        (2, 3, 9, 10, 4, 3, 3, (1, 1), (0, 0), 1),
        (2, 4, 9, 10, 6, 3, 3, (2, 1), (1, 2), 2),
        (3, 2, 7, 7, 5, 3, 2, (2, 3), (2, 2), 1),
        (1, 1, 28, 28, 32, 3, 3, (1, 1), (0, 0), 1),
        (2, 32, 12, 12, 64, 3, 3, (1, 1), (1, 1), 1),
        (2, 8, 6, 6, 8, 1, 1, (1, 1), (0, 0), 8),
        (1, 3, 5, 5, 2, 5, 5, (1, 1), (2, 2), 1),
        # long chains for conv2d_grad_kernel: ragged channel / column counts, row chunks of odd length,
        # strides with padding, rows wider than one chunk, a 1x1 kernel
        (5, 5, 15, 13, 11, 3, 3, (1, 1), (0, 0), 1),
        (4, 7, 17, 19, 9, 3, 3, (2, 2), (1, 1), 1),
        (3, 3, 20, 23, 10, 5, 3, (1, 2), (2, 0), 1),
        (1, 2, 3, 300, 3, 2, 3, (1, 1), (0, 1), 1),
        (2, 2, 4, 530, 5, 3, 3, (1, 2), (1, 1), 1),
        (6, 20, 10, 10, 12, 1, 1, (1, 1), (0, 0), 1),
        (3, 4, 16, 16, 8, 3, 3, (1, 1), (1, 1), 1),
    ]
    for ci, (N, IC, H, W, OC, KH, KW, s, p, g) in enumerate(conv_cfgs):
        def mk(N=N, IC=IC, H=H, W=W, OC=OC, KH=KH, KW=KW, s=s, p=p, g=g, ci=ci):
            return (_randn(400 + ci, N, IC, H, W), _randn(500 + ci, OC, IC // g, KH, KW), s, p, g)
        cases.append(("conv2d_%d" % ci, "conv2d", mk))
        if g == 1:
            OH, OW = (H + 2 * p[0] - KH) // s[0] + 1, (W + 2 * p[1] - KW) // s[1] + 1

            def mk_gi(N=N, IC=IC, H=H, W=W, OC=OC, KH=KH, KW=KW, s=s, p=p, ci=ci, OH=OH, OW=OW):
                return ((N, IC, H, W), _randn(500 + ci, OC, IC, KH, KW),
                        _randn(600 + ci, N, OC, OH, OW), s, p)

            def mk_gk(N=N, IC=IC, H=H, W=W, OC=OC, KH=KH, KW=KW, s=s, p=p, ci=ci, OH=OH, OW=OW):
                return (_randn(400 + ci, N, IC, H, W), (OC, IC, KH, KW),
                        _randn(600 + ci, N, OC, OH, OW), s, p)
            cases.append(("conv2d_grad_input_%d" % ci, "conv2d_grad_input", mk_gi))
            cases.append(("conv2d_grad_kernel_%d" % ci, "conv2d_grad_kernel", mk_gk))

    # operands that force the exact path of the padded implicit-GEMM forms: an infinity next to zero
    # padding, and values so small that products vanish (each output meets the infinity at most once,
    # so no NaN -- whose payload is not part of the contract -- is produced)
    def unsafe_operands(x_inf=True):
        x = _randn(470, 3, 4, 16, 16)
        x.view(-1)[::37] *= 1e-30
        x.view(-1)[5::91] *= -1e-38
        if x_inf:
            x[1, 2, 0, 15] = float("inf")
        k = _randn(570, 8, 4, 3, 3)
        k.view(-1)[::13] *= 1e-25
        go = _randn(670, 3, 8, 16, 16)
        go.view(-1)[3::29] *= 1e-33
        go[2, 5, 15, 0] = float("-inf")
        return x, k, go
    cases.append(("conv2d_unsafe", "conv2d",
                  lambda: (unsafe_operands()[0], unsafe_operands()[1], (1, 1), (1, 1), 1)))
    cases.append(("conv2d_grad_input_unsafe", "conv2d_grad_input",
                  lambda: ((3, 4, 16, 16), unsafe_operands()[1], unsafe_operands()[2], (1, 1), (1, 1))))
    cases.append(("conv2d_grad_kernel_unsafe", "conv2d_grad_kernel",
                  lambda: (unsafe_operands(False)[0], (8, 4, 3, 3), unsafe_operands()[2], (1, 1), (1, 1))))

    # ---- sums -----------------------------------------------------------------------------------
    for n in (0, 1, 5, 4095, 4096, 4097, 100000):
        for avg in (False, True):
            if n == 0 and avg:
                continue
            cases.append(("sum1d_%d_%d" % (n, avg), "sum1d",
                          lambda n=n, avg=avg: (_randn(700, n, scale=100.0), avg)))
    # massive cancellation and binade hovering
    def mk_cancel():
        x = _randn(701, 50000, scale=1e6)
        x[::2] = -x[1::2] * (1 + 2 ** -20)
        return (x, False)
    cases.append(("sum1d_cancel", "sum1d", mk_cancel))

    def mk_hover():
        x = _randn(702, 60000, scale=3.0)
        x[0] = 1048576.0
        return (x, False)
    cases.append(("sum1d_hover", "sum1d", mk_hover))

    # long chains (the summarised path): the same stress patterns at sizes above one node
    def mk_long(seed, n, scale, first=None, dist="normal"):
        def mk():
            g = _g(seed)
            if dist == "normal":
                x = torch.randn(n, generator=g) * scale
            elif dist == "lognormal":
                x = torch.empty(n).log_normal_(0, 2, generator=g) * (torch.randint(0, 2, (n,), generator=g).float() * 2 - 1)
            elif dist == "halves":      # every add is an exact tie once |s| is in [2^23, 2^24)
                x = (torch.randint(-8, 8, (n,), generator=g).float() + 0.5)
            elif dist == "wide":        # magnitudes spread over 60 binades
                x = torch.randn(n, generator=g) * torch.exp2(torch.randint(-30, 30, (n,), generator=g).float())
            elif dist == "tiny":        # mostly absorbed
                x = torch.randn(n, generator=g) * 1e-3
            elif dist == "pos":         # one sign only: the chain saturates at a power of two
                x = torch.rand(n, generator=g) * scale
            if first is not None:
                x[0] = first
            return (x, False)
        return mk
    cases.append(("sum1d_long_normal", "sum1d", mk_long(730, 300001, 100.0)))
    cases.append(("sum1d_long_lognormal", "sum1d", mk_long(731, 1 << 20, 1.0, dist="lognormal")))
    cases.append(("sum1d_long_hover_up", "sum1d", mk_long(732, 500000, 3.0, first=1048576.0)))
    cases.append(("sum1d_long_hover_neg", "sum1d", mk_long(733, 500000, 3.0, first=-2097152.0)))
    cases.append(("sum1d_long_ties", "sum1d", mk_long(734, 400000, 1.0, first=12000000.0, dist="halves")))
    cases.append(("sum1d_long_ties_neg", "sum1d", mk_long(735, 400000, 1.0, first=-9000000.0, dist="halves")))
    cases.append(("sum1d_long_wide", "sum1d", mk_long(736, 400000, 1.0, dist="wide")))
    cases.append(("sum1d_long_absorbed", "sum1d", mk_long(737, 700000, 1.0, first=4.0e6, dist="tiny")))
    cases.append(("sum1d_long_signflips", "sum1d", mk_long(738, 300000, 1.0e-3)))

    cases.append(("sum1d_long_saturate_pos", "sum1d", mk_long(742, 400000, 1.0, first=16700000.0, dist="pos")))
    cases.append(("sum1d_long_saturate_neg", "sum1d", mk_long(743, 400000, -1.0, first=-16700000.0, dist="pos")))
    cases.append(("sum1d_long_boundary_neg", "sum1d", mk_long(744, 500000, 0.05, first=-1048576.0)))
    cases.append(("sum1d_long_boundary_pos", "sum1d", mk_long(745, 500000, 0.05, first=2097152.0)))
    cases.append(("sum1d_long_lognormal_neg", "sum1d", mk_long(746, 1 << 20, 1.0, first=-1048000.0, dist="lognormal")))

    def mk_long_cancel():
        x = _randn(739, 400000, scale=1e6)
        x[::2] = -x[1::2] * (1 + 2 ** -20)
        return (x, True)
    cases.append(("sum1d_long_cancel_mean", "sum1d", mk_long_cancel))

    def mk_long_inf():
        x = _randn(740, 200000, scale=10.0)
        x[150000] = float("inf")
        return (x, False)
    cases.append(("sum1d_long_inf", "sum1d", mk_long_inf))

    def mk_long_subnormal():
        x = _randn(741, 200000, scale=1e-41)   # subnormal inputs: the state stays below 2^-104
        return (x, False)
    cases.append(("sum1d_long_subnormal", "sum1d", mk_long_subnormal))
    for (M, N) in [(1, 1), (37, 53), (256, 10), (256, 128), (130, 4096), (5, 4100), (1, 7), (9, 1)]:
        for kd in (False, True):
            for avg in (False, True):
                cases.append(("sum2d_dim0_%dx%d_%d%d" % (M, N, kd, avg), "sum2d_dim0",
                              lambda M=M, N=N, kd=kd, avg=avg: (_randn(710, M, N, scale=10.0), kd, avg)))
                cases.append(("sum2d_dim1_%dx%d_%d%d" % (M, N, kd, avg), "sum2d_dim1",
                              lambda M=M, N=N, kd=kd, avg=avg: (_randn(711, M, N, scale=10.0), kd, avg)))
    # the last three: chains longer than one staged tile of 4096 with short, one-element and long segments
    for (N, C, H, W) in [(3, 5, 7, 2), (4, 64, 24, 24), (2, 1, 1, 1), (5, 3, 13, 11), (40, 3, 11, 13),
                         (5000, 2, 1, 1), (9, 2, 30, 31)]:
        for kd in (False, True):
            for avg in (False, True):
                cases.append(("sum4d_%dx%dx%dx%d_%d%d" % (N, C, H, W, kd, avg), "sum4d_dim023",
                              lambda N=N, C=C, H=H, W=W, kd=kd, avg=avg:
                              (_randn(720, N, C, H, W, scale=10.0), kd, avg)))

    # ---- elementwise ----------------------------------------------------------------------------
    cases.append(("exp_special", "exp", lambda: (special_values(),)))
    cases.append(("log_special", "log", lambda: (special_values(),)))
    cases.append(("log_abs_special", "log", lambda: (special_values().abs(),)))
    cases.append(("sqrt_special", "sqrt", lambda: (special_values(),)))
    cases.append(("div10_special", "div", lambda: (special_values(), 10.0)))
    cases.append(("div_tensor_special", "div",
                  lambda: (special_values(), torch.roll(special_values(), 7))))
    cases.append(("exp_range", "exp", lambda: (torch.linspace(-110, 95, 200003),)))
    cases.append(("log_range", "log", lambda: (torch.logspace(-44, 38, 200003),)))
    cases.append(("exp_unaligned", "exp", lambda: (torch.linspace(-20, 20, 1003)[1:],)))

    # ---- composites -----------------------------------------------------------------------------
    for (M, N) in [(256, 10), (1, 1), (37, 1000), (64, 3)]:
        cases.append(("softmax_%dx%d" % (M, N), "softmax",
                      lambda M=M, N=N: (_randn(800, M, N, scale=5.0),)))
        if M == 1:
            continue  # the reference itself raises for one row (squeeze() makes it 0-d before log1d)
        cases.append(("cross_entropy_%dx%d" % (M, N), "cross_entropy",
                      lambda M=M, N=N: (_randn(800, M, N, scale=5.0),
                                        torch.randint(0, N, (M,), generator=_g(801)))))
    return cases


def run_case(impl, case, to_device=None):
    name, op, mk = case
    args = mk()
    if to_device is not None:
        args = tuple(a.to(to_device) if isinstance(a, torch.Tensor) else a for a in args)
    return getattr(impl, op)(*args)


class RefAdapter:
    """Presents the reference's CPU backend (oracle.ref()) under the names of repdl/ops.py."""

    def __init__(self, ref):
        self.cpu, self.math = ref.cpu, ref.math

    def mm(self, a, b, ta=False, tb=False):
        return self.cpu.mm(a, b, ta, tb)

    def conv2d(self, x, k, s, p, g):
        return self.cpu.conv2d(x, k, s[0], s[1], p[0], p[1], g)

    def conv2d_grad_input(self, shape, k, go, s, p):
        return self.cpu.conv2d_grad_input(go, k, shape[2], shape[3], s[0], s[1], p[0], p[1])

    def conv2d_grad_kernel(self, x, wshape, go, s, p):
        return self.cpu.conv2d_grad_kernel(go, x, wshape[2], wshape[3], s[0], s[1], p[0], p[1])

    def sum1d(self, x, avg=False):
        return self.cpu.sum1d(x, avg)

    def sum2d_dim0(self, x, kd=False, avg=False):
        return self.cpu.sum2d_dim0(x, kd, avg)

    def sum2d_dim1(self, x, kd=False, avg=False):
        return self.cpu.sum2d_dim1(x, kd, avg)

    def sum4d_dim023(self, x, kd=False, avg=False):
        return self.cpu.sum4d_dim023(x, kd, avg)

    def exp(self, x):
        return self.math.exp2d(x.view(1, -1)).view(x.shape)

    def log(self, x):
        return self.math.log1d(x.reshape(-1)).view(x.shape)

    def sqrt(self, x):  # repdl/ops.py:122-123
        return x.to(dtype=torch.float64).sqrt().to(dtype=torch.float32)

    def div(self, x, other):  # repdl/ops.py:98-103
        if isinstance(other, torch.Tensor):
            return x.div(other)
        return x.div(torch.tensor(other, device=x.device))

    def softmax(self, x):
        return self.cpu.softmax(x)

    def cross_entropy(self, x, t):
        return self.cpu.cross_entropy(x, t)


# ---- optimizer steps ----------------------------------------------------------------------------
OPTIM_SHAPES = [(37,), (5, 7), (300,), (1,), (64, 33)]
OPTIM_CONFIGS = [  # name, weight_decay, amsgrad
    ("plain", 0.0, False), ("decay", 0.01, False), ("amsgrad", 0.0, True), ("both", 0.02, True)]
OPTIM_STEPS = 6


def optim_inputs():
    """Initial parameters and the gradients of every step (magnitudes from 1e-6 to 100)."""
    g = torch.Generator().manual_seed(9)
    params = [torch.randn(*s, generator=g) for s in OPTIM_SHAPES]
    grads = []
    for _ in range(OPTIM_STEPS):
        grads.append([torch.randn(*s, generator=g) * 10 ** float(torch.randint(-6, 3, (1,), generator=g))
                      for s in OPTIM_SHAPES])
    return params, grads


def run_optimizer(make_optimizer, device="cpu"):
    """Runs OPTIM_STEPS steps of the optimizer `make_optimizer(params)` returns; the hash of all
    parameters after every step."""
    params, grads = optim_inputs()
    ps = [torch.nn.Parameter(p.clone().to(device)) for p in params]
    opt = make_optimizer(ps)
    hashes = []
    for step_grads in grads:
        for p, gr in zip(ps, step_grads):
            p.grad = gr.clone().to(device)
        opt.step()
        hashes.append(sha(torch.cat([p.detach().cpu().reshape(-1) for p in ps])))
    return hashes


def run_oracle_adam(oracle, weight_decay, amsgrad, lr=0.01):
    params, grads = optim_inputs()
    ps = [p.clone() for p in params]
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    vm = [torch.zeros_like(p) for p in ps] if amsgrad else [None] * len(ps)
    hashes = []
    for st, step_grads in enumerate(grads, 1):
        for p, gr, m, v, vx in zip(ps, step_grads, ms, vs, vm):
            oracle.adam_step(p, gr.contiguous(), m, v, st, lr=lr, weight_decay=weight_decay, vmax=vx)
        hashes.append(sha(torch.cat([p.reshape(-1) for p in ps])))
    return hashes


def run_oracle_sgd(oracle, lr=0.01):
    params, grads = optim_inputs()
    ps = [p.clone() for p in params]
    hashes = []
    for step_grads in grads:
        for p, gr in zip(ps, step_grads):
            oracle.sgd_step(p, gr.contiguous(), lr)
        hashes.append(sha(torch.cat([p.reshape(-1) for p in ps])))
    return hashes
