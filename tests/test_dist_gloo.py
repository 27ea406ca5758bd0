"""CPU, world_size 2 over gloo: the row-sharding and gathering logic of repdl_b200.dist.ShardedMM
with the oracle standing in for the GPU product.  Each rank must end with the full C, bit-identical
to the unsharded product (rows are independent chains, so sharding keeps the bits)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from repdl_b200.dist import ShardedMM
        g = torch.Generator().manual_seed(7)
        M, N, K = 96, 50, 33
        a = torch.rand(M, K, generator=g) * 2 - 1
        b = torch.rand(K, N, generator=g) * 2 - 1

        def mm_into(a_rows, bb, c_rows):
            c_rows.copy_(oracle.mm(a_rows.contiguous(), bb))

        sh = ShardedMM(M, N, K, device="cpu", mode="nccl", mm_into=mm_into)
        assert sh.world == world and sh.Mp == M // world and sh.mode == "nccl"
        c = sh(a[sh.row0:sh.row0 + sh.Mp], b)
        full = oracle.mm(a, b)
        ok = torch.equal(c.view(torch.int32), full.view(torch.int32))
        # a rank that passes a wrong M is rejected before any communication
        try:
            ShardedMM(M + 1, N, K, device="cpu", mode="nccl", mm_into=mm_into)
            ok = False
        except ValueError:
            pass
        # host-operand step: every rank uploads 1/world of B's rows and the ranks gather the rest
        # (K = 34 divides by the world size; K = 33 above takes the upload-everything path)
        from repdl_b200.dist import mm_from_host
        for K2 in (34, 33):
            a2 = torch.rand(M, K2, generator=g) * 2 - 1
            b2 = torch.rand(K2, N, generator=g) * 2 - 1
            sh2 = ShardedMM(M, N, K2, device="cpu", mode="nccl", mm_into=mm_into)
            a_dev, b_dev = torch.zeros(sh2.Mp, K2), torch.full((K2, N), float("nan"))
            c_host = torch.zeros(sh2.Mp, N)
            c2 = mm_from_host(sh2, a2[sh2.row0:sh2.row0 + sh2.Mp], b2, a_dev, b_dev, c_host)
            full2 = oracle.mm(a2, b2)
            ok = ok and torch.equal(c2.view(torch.int32), full2.view(torch.int32))
            ok = ok and torch.equal(c_host.view(torch.int32),
                                    full2[sh2.row0:sh2.row0 + sh2.Mp].view(torch.int32))
            ok = ok and torch.equal(b_dev.view(torch.int32), b2.view(torch.int32))
        # the product block by block (what the pipelined host-operand step issues): same full C
        sh3 = ShardedMM(M, N, K, device="cpu", mode="nccl", mm_into=mm_into)
        mine = a[sh3.row0:sh3.row0 + sh3.Mp]
        sh3.begin_step()
        for r0, r1 in ((0, 7), (7, 40), (40, sh3.Mp)):
            sh3.rows_into_all(mine[r0:r1], b, r0)
        sh3.end_step()
        ok = ok and sh3.kernel_launches == 3 and torch.equal(sh3.C.view(torch.int32), full.view(torch.int32))
        # convolution sharded by batch: every rank ends with all images, bit-identical
        from repdl_b200.dist import ShardedConv2d
        x = torch.randn(6, 3, 9, 8, generator=g)
        k = torch.randn(4, 3, 3, 3, generator=g)

        def conv_into(xp, kk, op):
            op.copy_(oracle.conv2d(xp.contiguous(), kk, (2, 1), (1, 1), 1))

        sc = ShardedConv2d(x.shape, k.shape, (2, 1), (1, 1), 1, device="cpu", conv_into=conv_into)
        y = sc(x[sc.n0:sc.n0 + sc.Np], k)
        ok = ok and torch.equal(y.view(torch.int32), oracle.conv2d(x, k, (2, 1), (1, 1), 1).view(torch.int32))
        try:
            ShardedConv2d((7, 3, 9, 8), k.shape, device="cpu", conv_into=conv_into)
            ok = False
        except ValueError:
            pass
        q.put((rank, ok, sh.kernel_launches))
    finally:
        dist.destroy_process_group()


def _leaver(rank, world, port, q):
    """Rank 1 fails on the host before the gather; rank 0 must get an error from its collective
    within the process group's timeout instead of waiting for ever."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    import oracle
    from repdl_b200.dist import ShardedMM
    a, b = torch.rand(8, 5), torch.rand(5, 6)
    sh = ShardedMM(8, 6, 5, device="cpu", mode="nccl",
                   mm_into=lambda x, y, c: c.copy_(oracle.mm(x.contiguous(), y)))
    sh(a[sh.row0:sh.row0 + sh.Mp], b)  # one good step first: both ranks are really connected
    def leave(code):  # flush the queue's feeder thread, then go without tearing anything down
        q.close()
        q.join_thread()
        os._exit(code)

    if rank == 1:
        q.put((1, "left", 0.0))
        leave(3)  # the failure: this rank is gone, with nothing of its own in flight
    t0 = time.time()
    try:
        sh(a[sh.row0:sh.row0 + sh.Mp], b)
        q.put((0, "no error", time.time() - t0))
    except Exception as e:  # gloo reports the lost peer (or the timeout) as a RuntimeError
        q.put((0, "error: " + type(e).__name__, time.time() - t0))
    leave(0)  # skip the process-group teardown, which would wait for the lost peer


def test_sharded_mm_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, 1), (1, True, 1)]


def test_a_rank_that_leaves_before_the_gather_is_an_error_not_a_hang():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 30500 + os.getpid() % 1000
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict((r, (what, dt)) for r, what, dt in (q.get(timeout=90) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
    assert res[1][0] == "left"
    assert res[0][0].startswith("error"), res
    assert res[0][1] < 60.0, res


def test_single_process_is_local():
    sys.path.insert(0, ROOT)
    import oracle
    from repdl_b200.dist import ShardedMM
    a, b = torch.rand(8, 5), torch.rand(5, 6)
    sh = ShardedMM(8, 6, 5, device="cpu", mm_into=lambda x, y, c: c.copy_(oracle.mm(x.contiguous(), y)))
    assert sh.mode == "local"
    assert torch.equal(sh(a, b), oracle.mm(a, b))
