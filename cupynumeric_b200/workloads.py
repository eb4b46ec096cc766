"""Seeded synthetic inputs with the shapes, sizes and value distributions of the five benchmark
configurations of the SORT path.  No public dataset is involved: every array comes from
``numpy.random.default_rng(seed)``.  Each generator takes the element count (or shape) so that
tests can draw reduced sizes from the same distribution."""
from __future__ import annotations

import numpy as np

C1_N = 1 << 24
C2_N = 1 << 28
C3_SHAPE = (65536, 4096)
C4_N_PER_GPU = 1 << 28
C5_N_PER_GPU = 1 << 28


def c1_int32_uniform(n: int = C1_N, seed: int = 101) -> np.ndarray:
    """1-D int32 keys uniform over the full int32 range; plain sort."""
    rng = np.random.default_rng(seed)
    return rng.integers(-2**31, 2**31, n, dtype=np.int32)


def c2_float32_nan_dups(n: int = C2_N, seed: int = 202) -> np.ndarray:
    """1-D float32 ~N(0,1) with 1 % exact duplicates and 0.1 % NaN at seeded positions; stable
    argsort with int64 indices."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(n, dtype=np.float32)
    k = n // 100
    if k:
        d = rng.choice(n, k, replace=False)
        a[d] = a[rng.integers(0, n, k)]
    k = n // 1000
    if k:
        a[rng.choice(n, k, replace=False)] = np.nan
    return a


def c3_float64_rows(shape: tuple[int, int] = C3_SHAPE, seed: int = 303) -> np.ndarray:
    """2-D float64 uniform [0,1); sorted along axis -1 (independent rows)."""
    rng = np.random.default_rng(seed)
    return rng.random(shape, dtype=np.float64)


def c4_int64_zipf_shard(n: int = C4_N_PER_GPU, rank: int = 0, seed: int = 404) -> np.ndarray:
    """One rank's shard of the 1-D int64 distributed sort: Zipf(a=1.2) clipped to [0, 2^40),
    heavy duplicates.  The global array is the shards in rank order."""
    rng = np.random.default_rng(seed + rank)
    out = np.empty(n, dtype=np.int64)
    step = 1 << 24
    for lo in range(0, n, step):  # bounded temporary memory
        m = min(step, n - lo)
        out[lo:lo + m] = np.minimum(rng.zipf(1.2, m), 2**40 - 1)
    return out


def c5_uint64_nearly_sorted_shard(n_per_rank: int = C5_N_PER_GPU, rank: int = 0, nranks: int = 1,
                                  seed: int = 505) -> np.ndarray:
    """One rank's shard of the nearly sorted uint64 array: ascending 0..N-1 (N = n_per_rank *
    nranks) with N/100 random pair swaps applied one after the other; stable argsort.

    Every rank draws the same swap list and applies the swaps that touch its own range, reading
    the partner's current value from a sparse overlay, so the global array never has to exist in
    one process."""
    n = n_per_rank * nranks
    rng = np.random.default_rng(seed)
    k = n // 100
    ii = rng.integers(0, n, k)
    jj = rng.integers(0, n, k)
    lo, hi = rank * n_per_rank, (rank + 1) * n_per_rank
    if nranks == 1:
        a = np.arange(n, dtype=np.uint64)
        _apply_swaps(a, ii, jj)
        return a
    # sparse simulation of the sequential swaps: only touched positions live in the dict
    touched: dict[int, int] = {}
    for i, j in zip(ii.tolist(), jj.tolist()):
        vi, vj = touched.get(i, i), touched.get(j, j)
        touched[i], touched[j] = vj, vi
    a = np.arange(lo, hi, dtype=np.uint64)
    pos = np.fromiter((p for p in touched if lo <= p < hi), dtype=np.int64)
    if pos.size:
        a[pos - lo] = np.fromiter((touched[int(p)] for p in pos), dtype=np.uint64, count=pos.size)
    return a


def _apply_swaps(a: np.ndarray, ii: np.ndarray, jj: np.ndarray) -> None:
    """Sequential pair swaps a[i], a[j] = a[j], a[i] in order; vectorised in blocks whose indices
    are all distinct, which leaves the sequential result unchanged."""
    k, pos = len(ii), 0
    block = 4096
    while pos < k:
        end = min(pos + block, k)
        bi, bj = ii[pos:end], jj[pos:end]
        both = np.concatenate([bi, bj])
        if np.unique(both).size == both.size:
            tmp = a[bi].copy()
            a[bi] = a[bj]
            a[bj] = tmp
        else:
            for i, j in zip(bi.tolist(), bj.tolist()):
                a[i], a[j] = a[j], a[i]
        pos = end


# ------------------------------------------------------------------------------------------------
# The same five distributions drawn on the GPU with torch's seeded generator: the full-size
# benchmark configurations (2^28 keys per GPU) take minutes to draw with NumPy on the host and a
# second on the device.  Same shapes, sizes and value distributions; a different random stream.
# ------------------------------------------------------------------------------------------------
def _gen(device, seed: int):
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def c1_int32_uniform_device(n: int, device, seed: int = 101):
    import torch

    return torch.randint(-2**31, 2**31, (n,), dtype=torch.int64, device=device, generator=_gen(device, seed)).to(torch.int32)


def c2_float32_nan_dups_device(n: int, device, seed: int = 202):
    import torch

    g = _gen(device, seed)
    a = torch.randn(n, dtype=torch.float32, device=device, generator=g)
    k = n // 100
    if k:
        dst = torch.randint(0, n, (k,), device=device, generator=g)
        src = torch.randint(0, n, (k,), device=device, generator=g)
        a[dst] = a[src]
    k = n // 1000
    if k:
        a[torch.randint(0, n, (k,), device=device, generator=g)] = float("nan")
    return a


def c3_float64_rows_device(shape, device, seed: int = 303):
    import torch

    return torch.rand(shape, dtype=torch.float64, device=device, generator=_gen(device, seed))


def c4_int64_zipf_shard_device(n: int, rank: int, device, seed: int = 404, a: float = 1.2):
    """Zipf(a) by rejection from the continuous envelope (Devroye's method, the one NumPy uses),
    clipped to [1, 2^40 - 1]."""
    import torch

    g = _gen(device, seed + rank)
    am1, b = a - 1.0, 2.0 ** (a - 1.0)
    out = torch.empty(n, dtype=torch.int64, device=device)
    chunk = 1 << 24
    for lo in range(0, n, chunk):
        m = min(chunk, n - lo)
        part = torch.empty(m, dtype=torch.float64, device=device)
        todo = torch.arange(m, device=device)
        while todo.numel():
            u = 1.0 - torch.rand(todo.numel(), dtype=torch.float64, device=device, generator=g)
            v = torch.rand(todo.numel(), dtype=torch.float64, device=device, generator=g)
            x = torch.floor(u ** (-1.0 / am1))
            tm1 = torch.expm1(am1 * torch.log1p(1.0 / x))            # T - 1, T = (1 + 1/x)^(a-1)
            ok = (x >= 1) & (v * x * tm1 / (b - 1.0) <= (tm1 + 1.0) / b)
            part[todo[ok]] = x[ok]
            todo = todo[~ok]
        out[lo:lo + m] = torch.clamp(part, max=float(2**40 - 1)).to(torch.int64)
    return out


def c5_uint64_nearly_sorted_shard_device(n_per_rank: int, rank: int, nranks: int, device, seed: int = 505):
    """This rank's range of the ascending array 0..N-1 (N = n_per_rank * nranks) after N/100
    random pair swaps.  Every rank draws the same pair list; pairs that share a position with
    another pair are dropped, which makes the result independent of the order of application
    (and so identical on every rank) and keeps the global array a permutation of 0..N-1.
    Returned as int64 bit patterns of the uint64 keys (all values are below 2^63)."""
    import torch

    n = n_per_rank * nranks
    g = _gen(device, seed)
    k = n // 100
    ii = torch.randint(0, n, (k,), device=device, generator=g)
    jj = torch.randint(0, n, (k,), device=device, generator=g)
    both = torch.cat([ii, jj])
    order = torch.argsort(both)
    s = both[order]
    dup = torch.zeros(2 * k, dtype=torch.bool, device=device)
    if k:
        same = s[1:] == s[:-1]
        dup[order[1:][same]] = True
        dup[order[:-1][same]] = True
    keep = ~(dup[:k] | dup[k:])
    ii, jj = ii[keep], jj[keep]
    lo, hi = rank * n_per_rank, (rank + 1) * n_per_rank
    a = torch.arange(lo, hi, dtype=torch.int64, device=device)
    mi = (ii >= lo) & (ii < hi)
    a[ii[mi] - lo] = jj[mi]
    mj = (jj >= lo) & (jj < hi)
    a[jj[mj] - lo] = ii[mj]
    return a
