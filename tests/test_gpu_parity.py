"""GPU: every operator of librepdl_b200.so against the CPU oracle and the reference's golden
fixtures, bit for bit.  All calls go through the C ABI (repdl_b200.ops -> ctypes)."""
import json
import os

import pytest
import torch

import oracle
from cases import build_cases, run_case, sha

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = build_cases()


def golden(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def bits_equal(a, b):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.shape != b.shape:
        print("shape", a.shape, b.shape)
        return False
    ai, bi = a.view(torch.int32).reshape(-1), b.view(torch.int32).reshape(-1)
    if torch.equal(ai, bi):
        return True
    bad = (ai != bi).nonzero().view(-1)
    print("%d of %d elements differ; first:" % (bad.numel(), ai.numel()),
          [(int(i), "%08x" % (ai[i].item() & 0xFFFFFFFF), "%08x" % (bi[i].item() & 0xFFFFFFFF))
           for i in bad[:8]])
    return False


@pytest.fixture(scope="module")
def ops():
    from repdl_b200 import ops as o
    return o


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_small_case(ops, case):
    got = run_case(ops, case, to_device="cuda")
    want = run_case(oracle, case)
    assert got.is_cuda
    assert bits_equal(got, want), case[0]
    g = golden("small_cases.json")[case[0]]
    assert list(got.shape) == g["shape"] and sha(got) == g["sha256"]


def test_unaligned_pointers(ops):
    """Device pointers that are only 4-byte aligned take the scalar paths."""
    g = torch.Generator().manual_seed(21)
    x = (torch.rand(100003, generator=g) * 40 - 20)
    xd = x.cuda()
    for off in (1, 2, 3):
        v, vd = x[off:off + 90001].contiguous(), xd[off:off + 90001]
        assert vd.data_ptr() % 16 != 0
        assert bits_equal(ops.exp(vd), oracle.exp(v))
        assert bits_equal(ops.log(vd.abs()), oracle.log(v.abs()))  # no NaN in v: abs() is exact
        assert bits_equal(ops.sqrt(vd.abs()), oracle.sqrt(v.abs()))
        assert bits_equal(ops.div(vd, 10.0), oracle.div(v, 10.0))
    a = torch.randn(65 * 36 + 1, generator=g)
    b = torch.randn(36 * 44 + 3, generator=g)
    am, bm = a[1:].view(65, 36), b[3:].view(36, 44)
    amd, bmd = a.cuda()[1:].view(65, 36), b.cuda()[3:].view(36, 44)
    assert bits_equal(ops.mm(amd, bmd), oracle.mm(am.contiguous(), bm.contiguous()))
    r = torch.randn(33 * 64 + 1, generator=g)
    assert bits_equal(ops.sum2d_dim1(r.cuda()[1:].view(33, 64)), oracle.sum2d_dim1(r[1:].view(33, 64)))
    # a long chain (summarised path) that starts 4 bytes past a 16-byte boundary and ends mid-node
    c = torch.randn(250001, generator=g) * 300.0
    assert bits_equal(ops.sum1d(c.cuda()[1:]), oracle.sum1d(c[1:].contiguous()))


def test_results_do_not_depend_on_run(ops):
    g = torch.Generator().manual_seed(22)
    a, b = torch.randn(513, 300, generator=g).cuda(), torch.randn(300, 257, generator=g).cuda()
    first = ops.mm(a, b)
    for _ in range(3):
        assert torch.equal(first, ops.mm(a, b))


def test_config1_mm_1024(ops):
    from repdl_b200 import workloads
    a, b = workloads.mm_square(1024, 0)
    got = ops.mm(a.cuda(), b.cuda())
    assert bits_equal(got, oracle.mm(a, b))
    path = os.path.join(GOLDEN, "configs.json")
    if os.path.exists(path):
        assert sha(got) == golden("configs.json")["c1_mm_1024"]["sha256"]
    # all four layouts of the same product give the same bits
    at, bt = a.t().contiguous().cuda(), b.t().contiguous().cuda()
    assert torch.equal(got, ops.mm(at, b.cuda(), transA=True))
    assert torch.equal(got, ops.mm(a.cuda(), bt, transB=True))
    assert torch.equal(got, ops.mm(at, bt, transA=True, transB=True))


def test_config2_first_chunks(ops):
    """Config 2 on its first two 2^24-element chunks, against the oracle run live."""
    from repdl_b200 import workloads
    gold = golden("configs.json")["c2_crmath_2p28"]["chunks"] if os.path.exists(
        os.path.join(GOLDEN, "configs.json")) else None
    for ci, x in enumerate(workloads.crmath_chunks(1 << 25, 1)):
        # |x| is taken on the CPU, as in the reference's CPU run: torch's CUDA abs() returns the
        # canonical NaN 0x7FFFFFFF for NaN inputs and would change the input bits
        xd, xad = x.cuda(), x.abs().cuda()
        res = {"div10": ops.div(xd, 10.0), "sqrt_abs": ops.sqrt(xad),
               "exp": ops.exp(xd.view(4096, 4096)).view(-1), "log_abs": ops.log(xad)}
        want = {"div10": oracle.div(x, 10.0), "sqrt_abs": oracle.sqrt(x.abs()),
                "exp": oracle.exp(x), "log_abs": oracle.log(x.abs())}
        for k in res:
            assert bits_equal(res[k], want[k]), (ci, k)
            if gold:
                assert sha(res[k]) == gold[ci][k], (ci, k)


def test_config3_pieces(ops):
    """Config 3 recipe on one 2^24 chunk: the 1-D chain and 4096 row chains."""
    from repdl_b200 import workloads
    x = next(iter(workloads.sum_chunks(1 << 24, 2)))
    xd = x.cuda()
    assert bits_equal(ops.sum1d(xd), oracle.sum1d(x))
    assert bits_equal(ops.sum1d(xd, average=True), oracle.sum1d(x, average=True))
    assert bits_equal(ops.sum2d_dim1(xd.view(4096, 4096)), oracle.sum2d_dim1(x.view(4096, 4096)))
    assert bits_equal(ops.sum2d_dim0(xd.view(4096, 4096)), oracle.sum2d_dim0(x.view(4096, 4096)))


def test_mm_linearity_in_rows(ops):
    """Size-independent property used at full size: any row block of C equals the product of the
    same row block of A with B (rows are independent chains), so sharding by rows keeps the bits."""
    g = torch.Generator().manual_seed(23)
    a, b = (torch.rand(2048, 1024, generator=g) * 2 - 1).cuda(), (torch.rand(1024, 2048, generator=g) * 2 - 1).cuda()
    full = ops.mm(a, b)
    for lo, hi in [(0, 256), (256, 1024), (1024, 1029), (1029, 2048)]:
        assert torch.equal(full[lo:hi], ops.mm(a[lo:hi], b))


def test_sqrt_sweep_of_the_input_domain(ops):
    """Every 1021st fp32 bit pattern (4.2 M values: denormals, both signs, infinities, NaNs) and every
    pattern of three binades: the branch-free square root equals the oracle's correctly rounded one.
    (On the device it was compared with sqrt.rn.f32 for every non-negative pattern.)"""
    bits = torch.arange(0, 1 << 32, 1021, dtype=torch.int64)
    dense = torch.cat([torch.arange(lo, lo + (3 << 23), dtype=torch.int64) for lo in (0, 0x3F000000)])
    for b in (bits, dense):
        x = (b & 0xFFFFFFFF).to(torch.uint32).view(torch.float32)
        assert bits_equal(ops.sqrt(x.cuda()), oracle.sqrt(x))


def test_scalar_division_with_subnormal_quotients(ops):
    """x / d for divisors whose quotients reach rounding midpoints of the subnormal range (the
    kernel multiplies by a double reciprocal and must fall back to the exact division there):
    every x bit pattern below 2^26 (all quotients subnormal or tiny), both signs, and a strided
    sweep of the whole domain."""
    low = torch.arange(0, 1 << 26, dtype=torch.int64)
    wide = torch.arange(0, 1 << 32, 4093, dtype=torch.int64)
    for d in (98.0, 150.0, 154.0, 182.0, -186.0, 198.0, 10.0):
        for b in (low, low | 0x80000000, wide):
            x = (b & 0xFFFFFFFF).to(torch.uint32).view(torch.float32)
            assert bits_equal(ops.div(x.cuda(), d), oracle.div(x, d)), d
    x = torch.tensor([147 * 2.0 ** -149], dtype=torch.float32)  # 1.5 ulp: ties to even
    assert ops.div(x.cuda(), 98.0).cpu().view(torch.int32).item() == 2


def test_conv_backward_rejects_inconsistent_shapes(ops):
    """The backward kernels index grad_output with extents derived from H, W / KH, KW: a grad_output
    of any other shape is refused on the host instead of being read out of bounds."""
    x = torch.zeros(2, 3, 8, 8, device="cuda")
    k = torch.zeros(4, 3, 3, 3, device="cuda")
    good = torch.zeros(2, 4, 6, 6, device="cuda")
    ops.conv2d_grad_input(x.shape, k, good, (1, 1), (0, 0))
    ops.conv2d_grad_kernel(x, k.shape, good, (1, 1), (0, 0))
    for bad in (torch.zeros(2, 4, 7, 6, device="cuda"), torch.zeros(2, 5, 6, 6, device="cuda")):
        with pytest.raises(ValueError):
            ops.conv2d_grad_input(x.shape, k, bad, (1, 1), (0, 0))
        with pytest.raises(ValueError):
            ops.conv2d_grad_kernel(x, k.shape, bad, (1, 1), (0, 0))
    with pytest.raises(ValueError):
        ops.conv2d_grad_kernel(x, k.shape, torch.zeros(3, 4, 6, 6, device="cuda"), (1, 1), (0, 0))
    with pytest.raises(ValueError):
        ops.conv2d(x, torch.zeros(4, 3, 9, 9, device="cuda"), (1, 1), (0, 0), 1)  # kernel larger than the image
    with pytest.raises(ValueError):
        ops.conv2d(x, k, (0, 1), (0, 0), 1)


def test_mm_from_host_pipeline_equals_one_launch(ops):
    """The pipelined host-operand step (row blocks uploaded, multiplied and downloaded on three
    streams) gives the bits of the one-launch product, twice in a row on the same buffers."""
    from repdl_b200.dist import ShardedMM, mm_from_host
    M, N, K = 4096, 640, 300
    g = torch.Generator().manual_seed(77)
    a = (torch.rand(M, K, generator=g) * 2 - 1)
    b = (torch.rand(K, N, generator=g) * 2 - 1)
    want = ops.mm(a.cuda(), b.cuda())
    sh = ShardedMM(M, N, K, device="cuda")
    a_host, b_host = a.pin_memory(), b.pin_memory()
    a_dev, b_dev = torch.zeros(M, K, device="cuda"), torch.zeros(K, N, device="cuda")
    c_host = torch.zeros(M, N).pin_memory()
    for rep in range(2):
        sh.C.zero_()
        c_host.zero_()
        sh.kernel_launches = 0
        c = mm_from_host(sh, a_host, b_host, a_dev, b_dev, c_host, chunks=8)
        torch.cuda.synchronize()
        assert sh.kernel_launches == 8
        assert torch.equal(c.view(torch.int32), want.view(torch.int32))
        assert torch.equal(c_host.view(torch.int32), want.cpu().view(torch.int32))


def test_mm_from_host_wave_aligned_blocks_and_column_parts(ops):
    """A problem large enough for the unequal, wave-aligned row blocks, with B uploaded by column parts
    (strided copies) and the first block multiplied part by part: bits of the one-launch product."""
    from repdl_b200.dist import ShardedMM, mm_from_host, _row_blocks
    M, N, K = 6150, 2048, 72
    blocks = _row_blocks(M, N, 8, torch.cuda.get_device_properties(0).multi_processor_count)
    assert blocks[0][0] == 0 and blocks[-1][1] == M and all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
    assert len({r1 - r0 for r0, r1 in blocks}) > 1  # not the equal split
    g = torch.Generator().manual_seed(78)
    a = (torch.rand(M, K, generator=g) * 2 - 1)
    b = (torch.rand(K, N, generator=g) * 2 - 1)
    want = ops.mm(a.cuda(), b.cuda())
    sh = ShardedMM(M, N, K, device="cuda")
    a_host, b_host = a.pin_memory(), b.pin_memory()
    a_dev, b_dev = torch.zeros(M, K, device="cuda"), torch.zeros(K, N, device="cuda")
    c_host = torch.zeros(M, N).pin_memory()
    for rep in range(2):
        sh.C.zero_(), b_dev.zero_(), c_host.zero_()
        sh.kernel_launches = 0
        c = mm_from_host(sh, a_host, b_host, a_dev, b_dev, c_host, chunks=8)
        torch.cuda.synchronize()
        assert sh.kernel_launches == len(blocks) + 3
        assert torch.equal(b_dev.cpu(), b)
        assert torch.equal(c.view(torch.int32), want.view(torch.int32))
        assert torch.equal(c_host.view(torch.int32), want.cpu().view(torch.int32))


def test_cross_entropy_gradient_in_one_launch(ops):
    """ops.cross_entropy_grad equals the reference's backward composition (softmax, one_hot, subtraction,
    two scalings) evaluated with the oracle's softmax on the CPU, bit for bit."""
    g = torch.Generator().manual_seed(91)
    for M, N, gscale in ((256, 10, 1.0), (37, 5, 0.3), (1, 1, -2.0), (300, 129, 1.0)):
        x = torch.randn(M, N, generator=g) * 6
        t = torch.randint(0, N, (M,), generator=g)
        gl = torch.tensor(gscale)
        want = oracle.softmax(x) - torch.nn.functional.one_hot(t, N)
        want *= 1.0 / M
        want *= gl
        assert bits_equal(ops.cross_entropy_grad(x.cuda(), t.cuda(), gl.cuda()), want)


def test_strided_copy_entry_point(ops):
    """repdl_b200_copy2d: a column block of a pinned host matrix to the device, device to device, and back;
    bad arguments are refused before anything is queued."""
    from repdl_b200._cabi import lib
    g = torch.Generator().manual_seed(5)
    h = torch.rand(37, 50, generator=g).pin_memory()
    d = torch.zeros(37, 64, device="cuda")
    d2 = torch.zeros(40, 20, device="cuda")
    back = torch.zeros(37, 20).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.repdl_b200_copy2d(d.data_ptr() + 4 * 8, 4 * 64, h.data_ptr() + 4 * 30, 4 * 50, 4 * 20, 37, 0, st) == 0
    assert lib.repdl_b200_copy2d(d2.data_ptr(), 4 * 20, d.data_ptr() + 4 * 8, 4 * 64, 4 * 20, 37, 2, st) == 0
    assert lib.repdl_b200_copy2d(back.data_ptr(), 4 * 20, d2.data_ptr(), 4 * 20, 4 * 20, 37, 1, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(back, h[:, 30:50]) and torch.equal(d[:, 8:28].cpu(), h[:, 30:50])
    assert float(d[:, :8].abs().sum()) == 0.0 and float(d[:, 28:].abs().sum()) == 0.0 and float(d2[37:].abs().sum()) == 0.0
    assert lib.repdl_b200_copy2d(d.data_ptr(), 4 * 10, h.data_ptr(), 4 * 50, 4 * 20, 37, 0, st) < 0   # pitch < width
    assert lib.repdl_b200_copy2d(d.data_ptr(), 4 * 64, h.data_ptr(), 4 * 50, 4 * 20, 37, 7, st) < 0   # direction
    assert lib.repdl_b200_copy2d(None, 4 * 64, h.data_ptr(), 4 * 50, 4 * 20, 37, 0, st) < 0
    assert lib.repdl_b200_copy2d(None, 4 * 64, None, 4 * 50, 0, 37, 0, st) == 0                       # nothing to copy


def test_config3_full_chain_and_rows(ops):
    """Config 3 at full size: the 2^30-element chain (checked against the reference's running
    state after every quarter and at the end) and the [65536, 4096] row sums."""
    path = os.path.join(GOLDEN, "configs.json")
    if not os.path.exists(path):
        pytest.skip("configs.json not generated")
    from repdl_b200 import workloads
    gold = golden("configs.json")
    states = gold["c3_sum1d_2p30"]["state_after_chunk_hex"]
    x = torch.empty(1 << 30, dtype=torch.float32, device="cuda")
    for ci, chunk in enumerate(workloads.sum_chunks(1 << 30, 2)):
        x[ci << 24:(ci + 1) << 24] = chunk.cuda()

    def hexof(t):
        return "%08x" % (t.cpu().view(torch.int32).item() & 0xFFFFFFFF)
    for nchunks in (1, 16, 32, 48, 64):
        assert hexof(ops.sum1d(x[:nchunks << 24])) == states[nchunks - 1], nchunks
    assert hexof(ops.sum1d(x)) == gold["c3_sum1d_2p30"]["result_hex"] == "c975c2b7"
    rows = ops.sum2d_dim1(x[:1 << 28].view(65536, 4096))
    assert sha(rows) == gold["c3_sum_rows_65536x4096"]["sha256"]
