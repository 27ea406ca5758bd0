"""Seeded synthetic inputs of the five benchmark configurations.

Inputs are always drawn on the CPU with torch generators (CUDA generators produce different
streams) and then copied to the device, so that a CPU run of the reference and a GPU run of this
package see identical bits.  The reference ships no dataset for these operators; these synthetic
tensors ARE the workload.
"""
import torch

CHUNK = 1 << 24


def mm_square(n=1024, seed=0):
    """Config 1: A, B ~ U[-1, 1) (x*2-1 is exact in fp32), drawn after torch.manual_seed(seed)."""
    g = torch.Generator().manual_seed(seed)
    a = torch.rand(n, n, generator=g) * 2 - 1
    b = torch.rand(n, n, generator=g) * 2 - 1
    return a, b


def mm_large(n=16384, seed=4):
    """Config 5: same distribution, generator seed 4."""
    return mm_square(n, seed)


def crmath_chunks(n_total=1 << 28, seed=1):
    """Config 2, yielded in chunks of 2^24: 90% U[-88, 88) drawn in fp64 then rounded to fp32 (an
    fp32 torch.rand has only 2^24 distinct values), 10% uniformly random fp32 bit patterns
    (subnormals, +-0, inf, NaN with payloads)."""
    g = torch.Generator().manual_seed(seed)
    done = 0
    while done < n_total:
        n = min(CHUNK, n_total - done)
        u = (torch.rand(n, generator=g, dtype=torch.float64) * 176 - 88).float()
        m = torch.rand(n, generator=g) < 0.1
        bits = torch.randint(-2 ** 31, 2 ** 31, (n,), generator=g, dtype=torch.int64)
        bits = bits.to(torch.int32).view(torch.float32)
        yield torch.where(m, bits, u)
        done += n


def sum_chunks(n_total=1 << 30, seed=2):
    """Config 3, yielded in chunks of 2^24: lognormal(0, 2) magnitudes with a random sign."""
    g = torch.Generator().manual_seed(seed)
    done = 0
    while done < n_total:
        n = min(CHUNK, n_total - done)
        v = torch.empty(n).log_normal_(0, 2, generator=g)
        s = torch.randint(0, 2, (n,), generator=g).float() * 2 - 1
        yield v * s
        done += n


def sum_rows(rows=65536, cols=4096, seed=2):
    """Config 3, row-wise case: the first rows*cols values of the same stream as a matrix."""
    return torch.cat(list(sum_chunks(rows * cols, seed))).view(rows, cols)


def cnn_batch(batch=256, seed=3):
    """Config 4: torch.manual_seed(seed); build the model FIRST (default init consumes the global
    generator), then call this for images U[0,1) [batch,1,28,28] and labels in 0..9."""
    x = torch.rand(batch, 1, 28, 28)
    y = torch.randint(0, 10, (batch,))
    return x, y


def cnn_torch_model():
    """The torch.nn.Sequential of config 4 (convert with from_torch_module of either package)."""
    nn = torch.nn
    return nn.Sequential(
        nn.Conv2d(1, 32, 3), nn.ReLU(), nn.Conv2d(32, 64, 3), nn.ReLU(), nn.MaxPool2d(2),
        nn.Flatten(), nn.Linear(9216, 128), nn.ReLU(), nn.Linear(128, 10))
