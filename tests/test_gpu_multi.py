"""GPU (2 or more devices): the row-sharded product gives, on every rank, the bits of the
single-GPU product -- through NCCL's all-gather and through the GEMM epilogue that stores its tiles
into the peers' buffers."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_sharded_mm_matches_single_gpu():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29611",
           os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-3000:])
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    ranks = json.loads(line[len("RESULT "):])
    assert len(ranks) == world
    for r in ranks:
        for key in ("nccl_0", "nccl_1", "auto_0", "auto_1", "from_host", "from_host_blocks"):
            assert r[key], (r, key)
        # the GPUs of one B200 node reach each other's memory: "auto" must really have taken the
        # epilogue-store path, not quietly fallen back to NCCL
        assert r["auto_mode"] == "p2p", r
