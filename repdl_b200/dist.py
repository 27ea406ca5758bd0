"""Row-sharded matrix multiplication across the GPUs of one node.

microsoft/RepDL has no multi-GPU code; this is the one distributed strategy the operator backend
needs: A is partitioned by rows, B is replicated, every rank computes its own row panel of C with
the single-GPU kernel (no reduction is ever split, so the bits are those of a one-GPU run), and
the panels are all-gathered so that every rank ends with the full C.

`ShardedMM` owns the buffers of one problem size and offers two ways of moving the panels:
  * "nccl": torch.distributed all_gather_into_tensor (NCCL over NVLink), written in place into the
            full C, optionally pipelined stripe by stripe behind the compute;
  * "p2p" : the GEMM epilogue itself stores every finished tile into all ranks' C buffers over
            NVLink (peer pointers from torch symmetric memory), followed by one barrier.
"""
import torch
import torch.distributed as dist

from . import ops
from ._cabi import check, lib


class ShardedMM:
    def __init__(self, M, N, K, group=None, device=None, mode="nccl", stripes=1):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if M % self.world:
            raise ValueError("M must be divisible by the number of ranks")
        self.M, self.N, self.K = M, N, K
        self.Mp = M // self.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.mode = mode if self.world > 1 else "local"
        self.stripes = stripes if (self.Mp % max(stripes, 1) == 0) else 1
        self.C = torch.empty((M, N), dtype=torch.float32, device=self.device)
        self.comm_stream = torch.cuda.Stream(self.device) if self.world > 1 else None
        self.kernel_launches = 0

    @property
    def row0(self):
        return self.rank * self.Mp

    def _mm_into(self, a_rows, b, c_rows):
        """c_rows[:] = a_rows @ b through the C ABI, on the current stream."""
        st = torch.cuda.current_stream(self.device).cuda_stream
        check(lib.repdl_b200_mm(a_rows.data_ptr(), b.data_ptr(), c_rows.data_ptr(), a_rows.shape[0],
                                self.N, self.K, 0, 0, a_rows.stride(0), b.stride(0),
                                c_rows.stride(0), st), "mm")
        self.kernel_launches += 1

    def __call__(self, a_panel, b):
        """a_panel: this rank's [M/world, K] rows of A; b: [K, N].  Returns the full [M, N] C."""
        C, Mp = self.C, self.Mp
        mine = C[self.row0:self.row0 + Mp]
        if self.world == 1:
            self._mm_into(a_panel, b, mine)
            return C
        if self.stripes <= 1:
            self._mm_into(a_panel, b, mine)
            dist.all_gather_into_tensor(C, mine, group=self.group)
            return C
        # stripe pipeline: stripe s is gathered on the communication stream while stripe s + 1
        # is being computed.  Each stripe is a [world, rows, N] strided view of C, which NCCL
        # cannot write in place, so stripes are gathered as one send/recv group per stripe.
        cur = torch.cuda.current_stream(self.device)
        rows = Mp // self.stripes
        for s in range(self.stripes):
            lo = self.row0 + s * rows
            self._mm_into(a_panel[s * rows:(s + 1) * rows], b, C[lo:lo + rows])
            ev = torch.cuda.Event()
            ev.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                outs = [C[r * Mp + s * rows: r * Mp + (s + 1) * rows] for r in range(self.world)]
                dist.all_gather(outs, C[lo:lo + rows], group=self.group)
        cur.wait_stream(self.comm_stream)
        return C


def mm_from_host(sharded, a_host_panel, b_host, a_dev, b_dev, c_host_panel):
    """End-to-end step with HOST operands: pinned A panel and B go to the device, the sharded
    product runs, and this rank's panel of C comes back to pinned host memory."""
    a_dev.copy_(a_host_panel, non_blocking=True)
    b_dev.copy_(b_host, non_blocking=True)
    C = sharded(a_dev, b_dev)
    c_host_panel.copy_(C[sharded.row0:sharded.row0 + sharded.Mp], non_blocking=True)
    return C
