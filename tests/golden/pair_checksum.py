"""Order-independent checksum of an undirected pair set, computable with wrap-around 64-bit arithmetic both in numpy (the
generator, on the CPU oracle's and the reference's lists) and in torch on the device (the test, on the exported list)."""
import numpy as np

M1 = 0x9E3779B1
M2 = 0x85EBCA77
MASK = (1 << 64) - 1


def checksum_numpy(a, b):
    """a < b: int arrays of atom ids. Returns (count, sum1, sum2) as Python ints, the sums modulo 2^64."""
    a = np.asarray(a).astype(np.uint64)
    b = np.asarray(b).astype(np.uint64)
    one = np.uint64(1)
    with np.errstate(over="ignore"):
        s1 = int(np.sum((a + one) * (b + one), dtype=np.uint64))
        s2 = int(np.sum((a * np.uint64(M1) + b) * (b * np.uint64(M2) + a + one), dtype=np.uint64))
    return int(len(a)), s1 & MASK, s2 & MASK


def checksum_torch(a, b, chunk=1 << 26):
    """The same sums from int64 device tensors (two's-complement wrap-around equals arithmetic modulo 2^64)."""
    s1 = s2 = 0
    for k in range(0, a.numel(), chunk):
        x, y = a[k:k + chunk], b[k:k + chunk]
        s1 += int(((x + 1) * (y + 1)).sum().item())
        s2 += int(((x * M1 + y) * (y * M2 + x + 1)).sum().item())
    return int(a.numel()), s1 & MASK, s2 & MASK
