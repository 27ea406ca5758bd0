"""GPU: seeded random shapes through the operators with many code paths (convolutions and their
gradients: padding, strides, ragged tiles, row chunks of every length, rows wider than a chunk;
products around every tile size; chain sums), each compared bit for bit with the CPU oracle.  The
oracle itself is pinned to the reference on the fixed cases of tests/cases.py."""
import os
import random

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
SCALE = int(os.environ.get("REPDL_FUZZ_SCALE", "1"))  # more shapes per run when hunting


def bits_equal(a, b):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    return a.shape == b.shape and torch.equal(a.view(torch.int32).reshape(-1), b.view(torch.int32).reshape(-1))


def equal_up_to_nan_payload(a, b):
    """Bit-equal, except that where both hold a NaN the payload may differ (a NaN result of an
    accumulating operator is NaN on both sides, its payload is outside the contract)."""
    a, b = a.detach().cpu().contiguous().reshape(-1), b.detach().cpu().contiguous().reshape(-1)
    if a.shape != b.shape or not torch.equal(torch.isnan(a), torch.isnan(b)):
        return False
    keep = ~torch.isnan(b)
    return torch.equal(a[keep].view(torch.int32), b[keep].view(torch.int32))


def _randn(g, *shape):
    # a few exact zeros and a wide range of magnitudes, no non-finite values
    x = torch.randn(*shape, generator=g)
    scale = 10.0 ** torch.randint(-3, 3, (1,), generator=g).item()
    x = x * scale
    if x.numel() > 4:
        x.view(-1)[:: max(3, x.numel() // 7)] = 0.0
    return x


def conv_configs(seed, count):
    rnd = random.Random(seed)
    out = []
    while len(out) < count:
        wide = rnd.random() < 0.1
        N, IC, OC = rnd.randint(1, 6), rnd.randint(1, 9), rnd.randint(1, 20)
        H, W = rnd.randint(3, 40), (rnd.randint(260, 600) if wide else rnd.randint(3, 40))
        if wide:
            H, N = rnd.randint(3, 6), rnd.randint(1, 2)
        KH, KW = rnd.randint(1, 5), rnd.randint(1, 5)
        sH, sW = rnd.randint(1, 3), rnd.randint(1, 3)
        pH, pW = rnd.choice([0, 0, 1, 2, 3]), rnd.choice([0, 0, 1, 2, 3])
        if H + 2 * pH < KH or W + 2 * pW < KW:
            continue
        out.append((N, IC, H, W, OC, KH, KW, (sH, sW), (pH, pW)))
    return out


@pytest.mark.parametrize("cfg", conv_configs(20240, 60 * SCALE), ids=lambda c: "x".join(map(str, c[:7])) + "_s%d%d_p%d%d" % (c[7] + c[8]))
def test_conv_and_gradients_random_shapes(cfg):
    from repdl_b200 import ops
    N, IC, H, W, OC, KH, KW, s, p = cfg
    g = torch.Generator().manual_seed(hash(cfg) & 0xFFFFFF)
    OH, OW = (H + 2 * p[0] - KH) // s[0] + 1, (W + 2 * p[1] - KW) // s[1] + 1
    x, k, go = _randn(g, N, IC, H, W), _randn(g, OC, IC, KH, KW), _randn(g, N, OC, OH, OW)
    same = bits_equal
    if (N + IC + H + W + OC) % 4 == 0:
        # operands that send the zero-padded forms to their exact fallback: values whose products
        # vanish, and one infinity (which meets exact zeros of the other operand, hence NaNs)
        for t in (x, k, go):
            t.view(-1)[1::5] *= 1e-30
            t.view(-1)[2::11] *= 1e-38
        x.view(-1)[x.numel() // 2] = float("inf")
        go.view(-1)[go.numel() // 3] = float("-inf")
        same = equal_up_to_nan_payload
    xd, kd, god = x.cuda(), k.cuda(), go.cuda()
    assert same(ops.conv2d(xd, kd, s, p, 1), oracle.conv2d(x, k, s, p, 1))
    assert same(ops.conv2d_grad_input(x.shape, kd, god, s, p), oracle.conv2d_grad_input(x.shape, k, go, s, p))
    want_gk = oracle.conv2d_grad_kernel(x, k.shape, go, s, p)
    assert same(ops.conv2d_grad_kernel(xd, k.shape, god, s, p), want_gk)
    fused = ops.conv2d_grad_kernel_bias(xd, k.shape, god, s, p)  # None: shape not taken by the fused kernel
    if fused is not None:
        assert same(fused[0], want_gk)
        assert same(fused[1].reshape(-1), oracle.sum4d_dim023(go).reshape(-1))


def window_conv_configs(seed, count):
    """Shapes of the stride-1, three-column kernels with many planes, which take the staged-window
    kernel: strips that do not divide the image, rows that are not a multiple of 4 pixels, channel
    counts around the 32 / 64-channel tiles, plane counts that are not a multiple of a chunk."""
    rnd = random.Random(seed)
    out = []
    while len(out) < count:
        N, IC, OC = rnd.randint(1, 4), rnd.randint(8, 40), rnd.randint(16, 72)
        H, W = rnd.randint(3, 34), rnd.randint(3, 34)
        KH = rnd.randint(1, 5)
        pH, pW = rnd.choice([0, 0, 1, 2]), rnd.choice([0, 1, 1, 2])
        if H + 2 * pH < KH or W + 2 * pW < 3:
            continue
        out.append((N, IC, H, W, OC, KH, 3, (1, 1), (pH, pW)))
    return out


@pytest.mark.parametrize("cfg", window_conv_configs(515, 24 * SCALE), ids=lambda c: "x".join(map(str, c[:7])) + "_p%d%d" % c[8])
def test_conv_window_kernel_random_shapes(cfg):
    from repdl_b200 import ops
    N, IC, H, W, OC, KH, KW, s, p = cfg
    g = torch.Generator().manual_seed(hash(cfg) & 0xFFFFFF)
    OH, OW = H + 2 * p[0] - KH + 1, W + 2 * p[1] - KW + 1
    x, k, go = _randn(g, N, IC, H, W), _randn(g, OC, IC, KH, KW), _randn(g, N, OC, OH, OW)
    same = bits_equal
    if (N + IC + H + W + OC) % 4 == 0:  # operands that force the exact fallback of some tiles
        x.view(-1)[1::97] *= 1e-30
        k.view(-1)[5::131] *= 1e-38
        go.view(-1)[go.numel() // 3] = float("-inf")
        same = equal_up_to_nan_payload
    xd, kd, god = x.cuda(), k.cuda(), go.cuda()
    assert same(ops.conv2d(xd, kd, s, p, 1), oracle.conv2d(x, k, s, p, 1))
    assert same(ops.conv2d_grad_input(x.shape, kd, god, s, p), oracle.conv2d_grad_input(x.shape, k, go, s, p))
    if IC % 2 == 0 and OC % 2 == 0:  # grouped forward convolution
        k2 = k[:, :IC // 2].contiguous()
        assert same(ops.conv2d(xd, k2.cuda(), s, p, 2), oracle.conv2d(x, k2, s, p, 2))


@pytest.mark.parametrize("cfg", [
    # N, IC, H, W, OC, KH, KW, stride, padding: weight-gradient chains whose chunks are segments of one
    # output row (rows longer than a chunk), with and without 16-byte copies of grad_output, padded,
    # and a whole image per chunk with a ragged last ring
    (1, 16, 5, 402, 72, 3, 3, (1, 1), (0, 0)),
    (1, 16, 5, 403, 72, 3, 3, (1, 1), (0, 0)),
    (2, 16, 4, 900, 72, 3, 3, (1, 1), (1, 1)),
    (3, 2, 4, 1000, 5, 2, 3, (1, 1), (0, 1)),
    (5, 3, 27, 31, 9, 3, 3, (1, 1), (0, 0)),
    (4, 16, 13, 19, 72, 3, 3, (1, 1), (2, 2)),
], ids=lambda c: "x".join(map(str, c[:7])) + "_p%d%d" % c[8])
def test_conv_weight_gradient_chunk_geometries(cfg):
    from repdl_b200 import ops
    N, IC, H, W, OC, KH, KW, s, p = cfg
    g = torch.Generator().manual_seed(sum(cfg[:7]))
    OH, OW = (H + 2 * p[0] - KH) // s[0] + 1, (W + 2 * p[1] - KW) // s[1] + 1
    x, go = _randn(g, N, IC, H, W), _randn(g, N, OC, OH, OW)
    want_w = oracle.conv2d_grad_kernel(x, (OC, IC, KH, KW), go, s, p)
    assert bits_equal(ops.conv2d_grad_kernel(x.cuda(), (OC, IC, KH, KW), go.cuda(), s, p), want_w)
    fused = ops.conv2d_grad_kernel_bias(x.cuda(), (OC, IC, KH, KW), go.cuda(), s, p)
    if fused is not None:
        assert bits_equal(fused[0], want_w)
        assert bits_equal(fused[1], oracle.sum4d_dim023(go, False, False))


@pytest.mark.parametrize("cfg", [
    # N, IC, H, W, OC, KH, KW, stride, padding, groups: one shape per forward kernel (short chains, the staged
    # window, the implicit GEMM with 32 and 64 channels per tile, the direct loop)
    (2, 3, 12, 13, 40, 3, 3, (1, 1), (1, 1), 1),
    (2, 16, 12, 13, 40, 3, 3, (1, 1), (1, 1), 1),
    (2, 16, 12, 13, 24, 5, 2, (2, 1), (1, 0), 1),
    (2, 16, 12, 13, 70, 4, 4, (1, 2), (0, 2), 2),
    (1, 2, 20, 9, 3, 9, 9, (1, 1), (4, 4), 1),
], ids=lambda c: "x".join(map(str, c[:7])) + "_g%d" % c[9])
def test_conv_epilogue_bias_and_relu(cfg):
    """conv2d with bias and ReLU in the kernel's epilogue equals the three separate launches (and the
    oracle's convolution followed by the same two element-wise operations), NaN and -0 included."""
    from repdl_b200 import ops
    N, IC, H, W, OC, KH, KW, s, p, groups = cfg
    g = torch.Generator().manual_seed(sum(cfg[:7]) + 5)
    x, k, b = _randn(g, N, IC, H, W), _randn(g, OC, IC // groups, KH, KW), _randn(g, OC)
    x.view(-1)[1] = float("nan")
    b[0] = -0.0
    k[0] = 0.0          # channel 0: conv = +0 (or NaN), + -0 -> +0; relu keeps +0
    want = oracle.conv2d(x, k, s, p, groups) + b.view(1, -1, 1, 1)
    xd, kd, bd = x.cuda(), k.cuda(), b.cuda()
    plain = ops.conv2d(xd, kd, s, p, groups)
    assert equal_up_to_nan_payload(ops.conv2d(xd, kd, s, p, groups, bias=bd), plain + bd.view(1, -1, 1, 1))
    assert equal_up_to_nan_payload(ops.conv2d(xd, kd, s, p, groups, bias=bd), want)
    fused = ops.conv2d(xd, kd, s, p, groups, bias=bd, relu=True)
    assert equal_up_to_nan_payload(fused, torch.relu(plain + bd.view(1, -1, 1, 1)))
    assert equal_up_to_nan_payload(ops.conv2d(xd, kd, s, p, groups, relu=True), torch.relu(plain))


@pytest.mark.parametrize("cfg", [(3, 5, 24, 24, 2, 2), (2, 3, 13, 17, 2, 2), (1, 4, 9, 10, 3, 3), (2, 2, 7, 31, 2, 3),
                                 (1, 1, 2, 2, 2, 2), (4, 6, 5, 5, 5, 5)], ids=lambda c: "x".join(map(str, c)))
def test_maxpool_over_disjoint_windows(cfg):
    """repdl_b200.nn.MaxPool2d (kernel = stride) against torch's CPU max_pool2d, forward and backward:
    ties (many equal values, zeros of both signs), NaNs and rows / columns beyond the last whole window."""
    from repdl_b200 import nn as rnn
    N, C, H, W, kh, kw = cfg
    g = torch.Generator().manual_seed(sum(cfg))
    x = torch.randint(-2, 3, (N, C, H, W), generator=g).float()      # few distinct values: ties everywhere
    x.view(-1)[::5] *= _randn(g, x.view(-1)[::5].numel())
    x.view(-1)[3::17] = -0.0
    if x.numel() > 40:
        x.view(-1)[7::41] = float("nan")
    xc = x.clone().requires_grad_(True)
    yc = torch.nn.functional.max_pool2d(xc, (kh, kw))
    go = _randn(g, *yc.shape)
    yc.backward(go)
    pool = rnn.from_torch_module(torch.nn.Sequential(torch.nn.MaxPool2d((kh, kw))))[0]
    assert type(pool) is rnn.MaxPool2d
    xd = x.cuda().requires_grad_(True)
    yd = pool(xd)
    yd.backward(go.cuda())
    assert equal_up_to_nan_payload(yd, yc) and bits_equal(xd.grad, xc.grad)
    # windows that overlap are left to torch
    if H >= 3 and W >= 3:
        over = rnn.MaxPool2d(3, stride=2)
        assert equal_up_to_nan_payload(over(x.cuda()), torch.nn.functional.max_pool2d(x, 3, 2))


SHORT_CHAIN_CONVS = [
    # N, IC, H, W, OC, KH, KW, stride, padding, groups: at most 64 taps per output
    (3, 1, 28, 28, 32, 3, 3, (1, 1), (0, 0), 1),   # 9 taps
    (2, 3, 19, 23, 40, 3, 3, (1, 1), (1, 1), 1),   # 27 taps, channels beyond one block of 32, padding
    (2, 3, 17, 16, 7, 4, 4, (2, 1), (2, 3), 1),    # 48 taps (the loop form), stride, wide padding
    (1, 2, 9, 31, 33, 5, 5, (1, 2), (2, 2), 1),    # 50 taps
    (2, 4, 12, 12, 10, 3, 3, (1, 1), (1, 0), 2),   # groups: 18 taps per output
    (1, 1, 3, 3, 1, 3, 3, (1, 1), (2, 2), 1),      # more padding than image
    (2, 7, 10, 11, 5, 3, 3, (3, 2), (1, 1), 1),    # 63 taps
    (2, 6, 8, 8, 12, 1, 1, (1, 1), (0, 0), 3),     # 1 x 1, grouped: 2 taps
]


@pytest.mark.parametrize("cfg", SHORT_CHAIN_CONVS, ids=lambda c: "x".join(map(str, c[:7])) + "_g%d" % c[9])
def test_conv_short_chains(cfg):
    """Forward convolutions with few taps per output (first layers) take the kernel that owns a pixel x 32
    channels per thread and skips padding taps like the reference; -0 results and tiny operands included."""
    from repdl_b200 import ops
    N, IC, H, W, OC, KH, KW, s, p, groups = cfg
    g = torch.Generator().manual_seed(sum(cfg[:7]) * 31 + groups)
    x, k = _randn(g, N, IC, H, W), _randn(g, OC, IC // groups, KH, KW)
    x.view(-1)[::7] = -0.0
    x.view(-1)[3::11] *= 1e-30
    k.view(-1)[2::5] *= -1e-25
    assert bits_equal(ops.conv2d(x.cuda(), k.cuda(), s, p, groups), oracle.conv2d(x, k, s, p, groups))


def test_conv_padding_keeps_a_negative_zero():
    """An accumulator can become -0 without any operand being tiny enough for its products to vanish:
    -3 * 2^-149 plus (3 - 2^-22) * 2^-149 rounds to -0.  The padding tap behind it must then leave
    -0 alone (the reference skips it), so operands this small have to take the exact path."""
    from repdl_b200 import ops
    a, b = 1.5 * 2.0 ** -74, (1.5 - 2.0 ** -23) * 2.0 ** -74
    # (1 plane, 1 x 3 taps): the gather kernel; (8 planes, 3 x 3 taps): the staged-window kernel.  The
    # two values sit at the end of the last row of the last plane, so that only padding taps follow.
    for IC, OC, KH in ((1, 2, 1), (8, 16, 3)):
        x = torch.zeros(2, IC, 8, 64)
        k = torch.zeros(OC, IC, KH, 3)
        x[:, IC - 1, 7, 62], x[:, IC - 1, 7, 63] = a, b
        k[:, IC - 1, KH // 2, 0], k[:, IC - 1, KH // 2, 1], k[:, IC - 1, KH // 2, 2] = -(2.0 ** -74), 2.0 ** -74, 1.0
        want = oracle.conv2d(x, k, (1, 1), (KH // 2, 1), 1)
        assert want[0, 0, 7, 63].view(torch.int32).item() == -2 ** 31  # -0.0 in the corner
        assert bits_equal(ops.conv2d(x.cuda(), k.cuda(), (1, 1), (KH // 2, 1), 1), want)


def mm_shapes(seed, count):
    rnd = random.Random(seed)
    return [(rnd.randint(1, 420), rnd.randint(1, 420), rnd.choice([0, 1, 15, 16, 17, rnd.randint(1, 700)]),
             rnd.random() < 0.5, rnd.random() < 0.5) for _ in range(count)]


@pytest.mark.parametrize("shape", mm_shapes(77, 40 * SCALE), ids=lambda s: "%dx%dx%d_%d%d" % s)
def test_mm_random_shapes(shape):
    from repdl_b200 import ops
    M, N, K, ta, tb = shape
    g = torch.Generator().manual_seed(M * 1000003 + N * 1009 + K)
    a = _randn(g, *((K, M) if ta else (M, K)))
    b = _randn(g, *((N, K) if tb else (K, N)))
    assert bits_equal(ops.mm(a.cuda(), b.cuda(), ta, tb), oracle.mm(a, b, ta, tb))


@pytest.mark.parametrize("shape", [(256, 128, 9216), (37, 50, 2048), (5, 3, 4100), (64, 64, 2060), (1, 1, 2048),
                                   (130, 9, 3000)])
def test_mm_few_outputs_over_a_long_k(shape):
    """x W^T with few outputs and a long K runs on the chain kernel of the convolution weight gradient
    (one chain per thread, chunks padded with the chain's identity): same bits as the tiled kernel's."""
    from repdl_b200 import ops
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7919 + N * 104729 + K)
    a, b = _randn(g, M, K), _randn(g, N, K)
    a[0, : K // 2] = -1e-30  # products that underflow to -0 keep the accumulator at -0 through the padding
    b[0, : K // 2] = 1e-30
    a[0, K // 2:] = 0.0
    assert bits_equal(ops.mm(a.cuda(), b.cuda(), False, True), oracle.mm(a, b, False, True))
    # the same operands in the other layouts take the tiled kernel
    assert bits_equal(ops.mm(a.cuda(), b.t().contiguous().cuda(), False, False), oracle.mm(a, b, False, True))


def test_chain_sums_random_shapes():
    from repdl_b200 import ops
    rnd = random.Random(5)
    g = torch.Generator().manual_seed(5)
    for _ in range(25 * SCALE):
        N, C, H, W = rnd.randint(1, 70), rnd.randint(1, 9), rnd.randint(1, 33), rnd.randint(1, 33)
        x = _randn(g, N, C, H, W)
        for avg in (False, True):
            assert bits_equal(ops.sum4d_dim023(x.cuda(), False, avg), oracle.sum4d_dim023(x, False, avg)), (N, C, H, W)
        M, K = rnd.randint(1, 300), rnd.randint(1, 5000)
        y = _randn(g, M, K)
        assert bits_equal(ops.sum2d_dim0(y.cuda()), oracle.sum2d_dim0(y)), (M, K)
        assert bits_equal(ops.sum2d_dim1(y.cuda()), oracle.sum2d_dim1(y)), (M, K)


def test_sum1d_random_chains():
    """Long single chains (the summarised path with its opened nodes, tiles and leaves) over element
    distributions chosen to move the running sum through binades in different ways."""
    from repdl_b200 import ops
    rnd = random.Random(11)
    g = torch.Generator().manual_seed(11)
    for it in range(24 * SCALE):
        n = rnd.randint(1 << 16, 1 << 21)
        kind = it % 8
        if kind == 0:      # zero-mean: the sum hovers around zero and keeps changing binade
            x = torch.randn(n, generator=g)
        elif kind == 1:    # drifting upwards through many binades
            x = torch.rand(n, generator=g) * 10.0 ** rnd.randint(-3, 3)
        elif kind == 2:    # heavy tails
            x = torch.randn(n, generator=g) * torch.exp(3 * torch.randn(n, generator=g))
        elif kind == 3:    # exact ties: halves of the ulp of the running sum
            x = torch.randint(-3, 4, (n,), generator=g).float() * 2.0 ** rnd.randint(-30, -10) + 1e-3
        elif kind == 4:    # a few huge elements among small ones (and a cancellation)
            x = torch.randn(n, generator=g) * 1e-3
            idx = torch.randint(0, n, (8,), generator=g)
            x[idx] = torch.tensor([1e20, -1e20, 3e7, -3e7, 1e30, -1e30, 5e3, -5e3])
        elif kind == 5:    # subnormal and tiny values
            x = torch.randn(n, generator=g) * 1e-40
        elif kind == 6:    # constant: the sum saturates where the element is below half an ulp
            x = torch.full((n,), rnd.choice([1.0, 0.1, 3.0e-5]))
        else:              # sign flips in blocks
            x = torch.rand(n, generator=g) * torch.sign(torch.sin(torch.arange(n) / rnd.randint(50, 50000)))
        for avg in (False, True):
            assert bits_equal(ops.sum1d(x.cuda(), avg), oracle.sum1d(x, avg)), (it, kind, n)
