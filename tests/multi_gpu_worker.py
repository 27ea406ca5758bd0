"""Worker for tests/test_gpu_multi.py: run under torchrun, one rank per GPU.  Every rank computes the
row-sharded product in both gather modes and compares the full result, bit for bit, with the
product it computes alone on its own GPU."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from repdl_b200 import ops
    from repdl_b200.dist import ShardedMM
    M, N, K = 2048, 1536, 1000
    g = torch.Generator().manual_seed(31)
    a = (torch.rand(M, K, generator=g) * 2 - 1).to(dev)
    b = (torch.rand(K, N, generator=g) * 2 - 1).to(dev)
    alone = ops.mm(a, b)
    # a second pair of operands: consecutive calls reuse the result buffer with DIFFERENT contents,
    # and the previous result is read on the stream right up to the next call (no barrier here:
    # ordering the peers' stores against that read is the product's job)
    a2 = (torch.rand(M, K, generator=g) * 2 - 1).to(dev)
    alone2 = ops.mm(a2, b)
    out = {"rank": rank}
    for mode in ("nccl", "auto"):
        sh = ShardedMM(M, N, K, device=dev, mode=mode)
        flags = []
        for rep in range(6):
            src, want = (a, alone) if rep % 2 == 0 else (a2, alone2)
            c = sh(src[sh.row0:sh.row0 + sh.Mp].contiguous(), b)
            flags.append((c == want).all())  # queued on the stream; the next call follows at once
        torch.cuda.synchronize()
        out["%s_0" % mode] = out["%s_1" % mode] = all(bool(f) for f in flags)
        out[mode + "_mode"] = sh.mode
        if hasattr(sh, "p2p_error"):
            out["p2p_error"] = sh.p2p_error
    # the host-operand step: A panel and 1/world of B uploaded, B gathered over NVLink, C panel back
    from repdl_b200.dist import mm_from_host
    a_host = a[sh.row0:sh.row0 + sh.Mp].cpu().pin_memory()
    b_host = b.cpu().pin_memory()
    a_dev, b_dev = torch.zeros_like(a_host, device=dev), torch.zeros_like(b_host, device=dev)
    c_host = torch.zeros(sh.Mp, N).pin_memory()
    dist.barrier()
    c = mm_from_host(sh, a_host, b_host, a_dev, b_dev, c_host)
    torch.cuda.synchronize()
    out["from_host"] = bool(torch.equal(c, alone)) and bool(
        torch.equal(c_host, alone[sh.row0:sh.row0 + sh.Mp].cpu())) and bool(torch.equal(b_dev, b))
    # a panel tall enough for the step to run in row blocks (each multiplied when it has arrived, its rows
    # of C sent back while the next one is multiplied), twice on the same buffers
    Mb, Kb = 4096 * world, 200
    ab = (torch.rand(Mb, Kb, generator=g) * 2 - 1).to(dev)
    bb = (torch.rand(Kb, N, generator=g) * 2 - 1).to(dev)
    alone_b = ops.mm(ab, bb)
    shb = ShardedMM(Mb, N, Kb, device=dev, mode="auto")
    ab_host = ab[shb.row0:shb.row0 + shb.Mp].cpu().pin_memory()
    bb_host = bb.cpu().pin_memory()
    ab_dev, bb_dev = torch.zeros_like(ab_host, device=dev), torch.zeros_like(bb_host, device=dev)
    cb_host = torch.zeros(shb.Mp, N).pin_memory()
    ok = True
    for rep in range(2):
        cb_host.zero_()
        shb.kernel_launches = 0
        cb = mm_from_host(shb, ab_host, bb_host, ab_dev, bb_dev, cb_host)
        torch.cuda.synchronize()
        ok = ok and shb.kernel_launches >= 2 and bool(torch.equal(cb, alone_b)) and bool(
            torch.equal(cb_host, alone_b[shb.row0:shb.row0 + shb.Mp].cpu()))
    out["from_host_blocks"] = ok
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
