"""Row-sharded matrix multiplication (and batch-sharded convolution) across the GPUs of one node.

microsoft/RepDL has no multi-GPU code; this is the one distributed strategy the operator backend
needs: A is partitioned by rows, B is replicated, every rank computes its own row panel of C with
the single-GPU kernel (no reduction is ever split, so the bits are those of a one-GPU run), and
the panels are gathered so that every rank ends with the full C.

`ShardedMM` owns the buffers of one problem size and offers two ways of moving the panels:
  * "p2p" : the GEMM epilogue itself stores every finished tile into all ranks' C buffers over
            NVLink (peer pointers from torch symmetric memory; plain stores, no multicast), so the
            gather overlaps the math tile by tile; one barrier afterwards makes the result visible;
  * "nccl": torch.distributed all_gather_into_tensor (NCCL over NVLink) written in place into the
            full C after the local panel is done -- the baseline.
"auto" tries "p2p" and falls back to "nccl" when symmetric memory cannot be set up.

Lifetime of the result.  `ShardedMM` returns its own buffer C, the same one on every call.  In
"p2p" mode the OTHER ranks write into it, so each call begins with a small all-reduce that no
rank's stream passes before every rank's stream has reached it: whatever a rank queued on its
stream to read the previous result (before making this call) has finished by the time any peer
starts to overwrite it.  Work on other streams, or on the host after the call returns, must be
ordered by the caller, as with any buffer that the next call reuses.

The panel product itself is injectable (`mm_into`), which lets the partitioning and gathering logic
be exercised on CPU ranks over gloo with any reference implementation of the product.
"""
import ctypes

import torch
import torch.distributed as dist


def _cabi_mm_into(a_rows, b, c_rows):
    from ._cabi import check, lib
    st = torch.cuda.current_stream(a_rows.device).cuda_stream
    check(lib.repdl_b200_mm(a_rows.data_ptr(), b.data_ptr(), c_rows.data_ptr(), a_rows.shape[0],
                            b.shape[1], a_rows.shape[1], 0, 0, a_rows.stride(0), b.stride(0),
                            c_rows.stride(0), st), "mm")


class ShardedMM:
    def __init__(self, M, N, K, group=None, device=None, mode="auto", mm_into=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if M % self.world:
            raise ValueError("M (%d) must be divisible by the number of ranks (%d)" % (M, self.world))
        self.M, self.N, self.K = M, N, K
        self.Mp = M // self.world
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.mm_into = mm_into or _cabi_mm_into
        self.kernel_launches = 0
        self.C = None
        self._peer_ptrs = None
        if self.world == 1:
            self.mode = "local"
        elif mode in ("auto", "p2p") and self.device.type == "cuda" and mm_into is None:
            try:
                self._setup_p2p()
                self.mode = "p2p"
            except Exception as e:  # symmetric memory unavailable: use the NCCL path
                if mode == "p2p":
                    raise
                self.mode, self.p2p_error = "nccl", repr(e)
        else:
            self.mode = "nccl"
        if self.C is None:
            self.C = torch.empty((M, N), dtype=torch.float32, device=self.device)

    # -- layout ----------------------------------------------------------------------------------
    @property
    def row0(self):
        return self.rank * self.Mp

    def my_rows(self):
        return self.C[self.row0:self.row0 + self.Mp]

    # -- p2p -------------------------------------------------------------------------------------
    def _setup_p2p(self):
        import torch.distributed._symmetric_memory as symm_mem
        grp = self.group if self.group is not None else dist.group.WORLD
        self.C = symm_mem.empty((self.M, self.N), dtype=torch.float32, device=self.device)
        self._hdl = symm_mem.rendezvous(self.C, grp)
        ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != self.C.data_ptr():
            raise RuntimeError("unexpected symmetric-memory layout")
        self._peer_ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def _p2p(self, a_panel, b):
        from ._cabi import check, lib
        # no peer may start storing into this rank's C before this rank has finished with the
        # previous result: nothing passes this collective until every rank's stream has reached it
        dist.all_reduce(self._flag, group=self.group)
        st = torch.cuda.current_stream(self.device).cuda_stream
        check(lib.repdl_b200_mm_allgather(a_panel.data_ptr(), b.data_ptr(), self._peer_ptrs,
                                          self.world, self.row0, self.Mp, self.N, self.K, 0, 0,
                                          a_panel.stride(0), b.stride(0), self.C.stride(0), st),
              "mm_allgather")
        self.kernel_launches += 1
        # every rank's kernel (and with it its stores into this rank's C) has completed once this
        # collective has: it is ordered after the kernel on each rank's stream
        dist.all_reduce(self._flag, group=self.group)

    # -- the product, block by block (for callers that pipeline it with copies) ---------------------
    def begin_step(self):
        """Before the first rows_into_all() of a step: in p2p mode no peer may store into this rank's
        C before this rank has finished with the previous result."""
        if self.mode == "p2p":
            dist.all_reduce(self._flag, group=self.group)

    def rows_into_all(self, a_rows, b, r0):
        """The product of rows [r0, r0 + len(a_rows)) of this rank's panel: into every rank's C in
        p2p mode, into this rank's C otherwise (end_step() then gathers)."""
        if self.mode == "p2p":
            from ._cabi import check, lib
            st = torch.cuda.current_stream(self.device).cuda_stream
            check(lib.repdl_b200_mm_allgather(a_rows.data_ptr(), b.data_ptr(), self._peer_ptrs, self.world,
                                              self.row0 + r0, a_rows.shape[0], self.N, self.K, 0, 0,
                                              a_rows.stride(0), b.stride(0), self.C.stride(0), st),
                  "mm_allgather")
        else:
            self.mm_into(a_rows, b, self.my_rows()[r0:r0 + a_rows.shape[0]])
        self.kernel_launches += 1

    def end_step(self):
        """After the last rows_into_all() of a step: the whole of C is on every rank when the stream
        has passed this point."""
        if self.mode == "p2p":
            dist.all_reduce(self._flag, group=self.group)
        elif self.world > 1:
            dist.all_gather_into_tensor(self.C, self.my_rows(), group=self.group)

    # -- the product -----------------------------------------------------------------------------
    def __call__(self, a_panel, b):
        """a_panel: this rank's [M/world, K] rows of A; b: [K, N].  Returns the full [M, N] C."""
        if self.mode == "p2p":
            self._p2p(a_panel, b)
            return self.C
        self.mm_into(a_panel, b, self.my_rows())
        self.kernel_launches += 1
        if self.world > 1:
            dist.all_gather_into_tensor(self.C, self.my_rows(), group=self.group)
        return self.C


class ShardedConv2d:
    """conv2d with the batch partitioned over the ranks (images are independent chains, microsoft/RepDL
    backend/cpu/convolution.cpp:24, so the bits are those of a one-GPU run): every rank convolves its
    N/world images with the replicated kernel and the outputs are all-gathered in place (NCHW is
    batch-major, so a rank's images are one contiguous block of the result).

    `conv_into(x_part, kernel, out_part)` is injectable like ShardedMM's product, which lets the
    partitioning be exercised on CPU ranks over gloo."""

    def __init__(self, input_shape, kernel_shape, stride=(1, 1), padding=(0, 0), groups=1, group=None,
                 device=None, conv_into=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        N, IC, H, W = input_shape
        OC, _, KH, KW = kernel_shape
        if N % self.world:
            raise ValueError("batch (%d) must be divisible by the number of ranks (%d)" % (N, self.world))
        self.stride, self.padding, self.groups = tuple(stride), tuple(padding), groups
        OH = (H + 2 * self.padding[0] - KH) // self.stride[0] + 1
        OW = (W + 2 * self.padding[1] - KW) // self.stride[1] + 1
        if OH <= 0 or OW <= 0:
            raise ValueError("the kernel does not fit into the padded image")
        self.Np = N // self.world
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.out = torch.empty((N, OC, OH, OW), dtype=torch.float32, device=device)
        self.conv_into = conv_into or self._ops_conv_into
        self.kernel_launches = 0

    def _ops_conv_into(self, x_part, kernel, out_part):
        from . import ops
        out_part.copy_(ops.conv2d(x_part, kernel, self.stride, self.padding, self.groups))

    @property
    def n0(self):
        return self.rank * self.Np

    def my_images(self):
        return self.out[self.n0:self.n0 + self.Np]

    def __call__(self, x_part, kernel):
        """x_part: this rank's [N/world, IC, H, W] images; kernel: [OC, IC/groups, KH, KW].  Returns
        the full [N, OC, OH, OW] output on every rank."""
        if x_part.shape[0] != self.Np:
            raise ValueError("expected %d images per rank, got %d" % (self.Np, x_part.shape[0]))
        self.conv_into(x_part, kernel, self.my_images())
        self.kernel_launches += 1
        if self.world > 1:
            dist.all_gather_into_tensor(self.out, self.my_images(), group=self.group)
        return self.out


_copy_streams = {}


def _side_streams(device):
    key = torch.device(device).index
    if key not in _copy_streams:
        _copy_streams[key] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
    return _copy_streams[key]


def _dense2d(*tensors):
    return all(t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] for t in tensors)


def _copy_cols_h2d(dst, src, c0, c1, stream):
    """Columns [c0, c1) of a pinned host matrix to the same columns of a device matrix, on `stream`."""
    from ._cabi import check, lib
    check(lib.repdl_b200_copy2d(dst.data_ptr() + 4 * c0, 4 * dst.stride(0), src.data_ptr() + 4 * c0,
                                4 * src.stride(0), 4 * (c1 - c0), dst.shape[0], 0, stream.cuda_stream), "copy2d")


def _equal_blocks(rows, chunks):
    step = -(-rows // chunks)
    return [(r0, min(rows, r0 + step)) for r0 in range(0, rows, step)]


def _row_blocks(rows, n_cols, chunks, sms):
    """Row blocks [(r0, r1), ...] for the pipelined host-operand step.

    Equal blocks waste the last wave of every launch (2048 rows of 16384 columns are 6.9 waves of
    192 x 128 tiles on 148 SMs: 4 % lost eight times).  So block heights are chosen in units of the
    192-row tile to fill whole waves, with a smaller first block (its upload is not hidden) and a
    smaller last block (its download is not hidden).  Small problems keep equal blocks."""
    unit = 192
    units = -(-rows // unit)   # the last unit may be partial
    if units < 4 * chunks:
        return _equal_blocks(rows, chunks)
    tiles_per_unit = -(-n_cols // 128)
    waves = lambda r: -(-r * tiles_per_unit // sms)                      # launches of r units
    loss = lambda r: waves(r) - r * tiles_per_unit / sms                  # idle fraction of its last wave
    target = units / chunks
    edge = min(range(max(1, int(0.3 * target)), max(2, int(0.9 * target)) + 1), key=lambda r: (loss(r) / r, r))
    inner_sizes = sorted(range(max(1, int(0.7 * target)), int(1.6 * target) + 1), key=lambda r: (loss(r) / r, -r))
    best = None
    for mid in inner_sizes[:4]:
        left = units - 2 * edge
        if left < 0:
            continue
        n_mid, rest = divmod(left, mid)
        sizes = [edge] + [mid] * n_mid + ([rest] if rest else []) + [edge]
        cost = sum(waves(r) for r in sizes) + 0.5 * len(sizes)
        if best is None or cost < best[0]:
            best = (cost, sizes)
    if best is None:
        return _equal_blocks(rows, chunks)
    out, r0 = [], 0
    for r in best[1]:
        out.append((r0 * unit, min(rows, (r0 + r) * unit)))
        r0 += r
    return out


def mm_from_host(sharded, a_host_panel, b_host, a_dev, b_dev, c_host_panel, chunks=8):
    """End-to-end step with HOST operands: pinned A panel and B go to the device, the sharded
    product runs, and this rank's panel of C comes back to pinned host memory.

    One GPU: the step is a pipeline over about `chunks` row blocks of A (heights that fill whole waves
    of the product's tiles, see _row_blocks).  The first block of A goes up first, then B in four
    or eight column parts, each multiplied with that block as soon as it has arrived, then the other blocks of
    A; block i is multiplied when it is there, and its rows of C go back on a second copy stream
    while block i + 1 is multiplied.  What stays exposed is the first block of A, a quarter of B and
    the last download.  (Every element of C is its own chain over the whole of K, so the bits are
    those of the one-launch product.)

    Several GPUs: every rank has the same B in host memory, so each uploads only its 1/world of B's
    rows and the ranks all-gather B over NVLink -- world times less PCIe traffic for B than uploading
    it everywhere.  The slice of B goes first on a copy stream and the A panel behind it in row blocks,
    so that A arrives while B is being gathered; every block is multiplied when it is there (into
    all ranks' C in the fused mode) and its rows of C go back to the host while the next block is
    multiplied.
    """
    dev = a_dev.device
    if sharded.world > 1:
        kp = b_dev.shape[0] // sharded.world
        if dev.type == "cuda" and b_dev.shape[0] % sharded.world == 0 and b_dev.is_contiguous():
            lo = sharded.rank * kp
            cur = torch.cuda.current_stream(dev)
            up, down = _side_streams(dev)
            # row blocks of this rank's panel: multiplied as they arrive, their rows of C sent back while
            # the next block is multiplied (a rank's own rows of C are written by its own kernel)
            Mp = a_dev.shape[0]
            nblocks = 4 if Mp >= 8192 else (2 if Mp >= 2048 else 1)
            blocks = _row_blocks(Mp, b_dev.shape[1], nblocks,
                                 torch.cuda.get_device_properties(dev).multi_processor_count) if nblocks > 1 else [(0, Mp)]
            up.wait_stream(cur)  # the buffers may still be in use by what the caller queued before
            down.wait_stream(cur)
            a_there = []
            with torch.cuda.stream(up):
                b_dev[lo:lo + kp].copy_(b_host[lo:lo + kp], non_blocking=True)
                b_there = torch.cuda.Event()
                b_there.record(up)
                for r0, r1 in blocks:
                    a_dev[r0:r1].copy_(a_host_panel[r0:r1], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(up)
                    a_there.append(ev)
            cur.wait_event(b_there)
            dist.all_gather_into_tensor(b_dev, b_dev[lo:lo + kp], group=sharded.group)
            sharded.begin_step()
            mine = sharded.my_rows()
            for (r0, r1), ev in zip(blocks, a_there):
                cur.wait_event(ev)
                sharded.rows_into_all(a_dev[r0:r1], b_dev, r0)
                done = torch.cuda.Event()
                done.record(cur)
                down.wait_event(done)
                with torch.cuda.stream(down):
                    c_host_panel[r0:r1].copy_(mine[r0:r1], non_blocking=True)
            sharded.end_step()
            cur.wait_stream(down)
            return sharded.C
        elif b_dev.shape[0] % sharded.world == 0 and b_dev.is_contiguous():
            lo = sharded.rank * kp
            a_dev.copy_(a_host_panel, non_blocking=True)
            b_dev[lo:lo + kp].copy_(b_host[lo:lo + kp], non_blocking=True)
            dist.all_gather_into_tensor(b_dev, b_dev[lo:lo + kp], group=sharded.group)
        else:
            a_dev.copy_(a_host_panel, non_blocking=True)
            b_dev.copy_(b_host, non_blocking=True)
        C = sharded(a_dev, b_dev)
        c_host_panel.copy_(sharded.my_rows(), non_blocking=True)
        return C
    rows = a_dev.shape[0]
    if dev.type != "cuda" or chunks <= 1 or rows // chunks < 256:
        a_dev.copy_(a_host_panel, non_blocking=True)
        b_dev.copy_(b_host, non_blocking=True)
        C = sharded(a_dev, b_dev)
        c_host_panel.copy_(sharded.my_rows(), non_blocking=True)
        return C
    cur = torch.cuda.current_stream(dev)
    up, down = _side_streams(dev)
    N = b_dev.shape[1]
    blocks = _row_blocks(rows, N, chunks, torch.cuda.get_device_properties(dev).multi_processor_count)
    # the first block's product runs by column parts of B, each as soon as it has arrived
    parts = (8 if N % 4096 == 0 else 4) if N % 2048 == 0 and _dense2d(b_dev, b_host) else 1
    up.wait_stream(cur)      # the buffers may still be in use by what the caller queued before
    down.wait_stream(cur)
    a_there, b_there = [], []
    with torch.cuda.stream(up):
        for i, (r0, r1) in enumerate(blocks):
            a_dev[r0:r1].copy_(a_host_panel[r0:r1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(up)
            a_there.append(ev)
            if i == 0:
                w = N // parts
                for j in range(parts):
                    if parts == 1:
                        b_dev.copy_(b_host, non_blocking=True)
                    else:
                        _copy_cols_h2d(b_dev, b_host, j * w, (j + 1) * w, up)
                    ev = torch.cuda.Event()
                    ev.record(up)
                    b_there.append(ev)
    C = sharded.C
    for i, (r0, r1) in enumerate(blocks):
        cur.wait_event(a_there[i])
        if i == 0:
            w = N // parts
            for j in range(parts):
                cur.wait_event(b_there[j])
                sharded.mm_into(a_dev[r0:r1], b_dev[:, j * w:(j + 1) * w], C[r0:r1, j * w:(j + 1) * w])
                sharded.kernel_launches += 1
        else:
            sharded.mm_into(a_dev[r0:r1], b_dev, C[r0:r1])
            sharded.kernel_launches += 1
        done = torch.cuda.Event()
        done.record(cur)
        down.wait_event(done)
        with torch.cuda.stream(down):
            c_host_panel[r0:r1].copy_(C[r0:r1], non_blocking=True)
    cur.wait_stream(down)    # the caller's stream order covers the whole step
    return C
