"""World-size-2 CPU test of the distributed sort's host logic over the gloo backend: where the
samples are taken, the weighted splitter selection and the destination rule come from the C ABI's
host entry points; the local sort of what a rank received is played by the oracle, the data
movement by gloo.  Checks that the rank-ordered concatenation is the global stable sort, that
indices are global, and that the splitters balance heavy duplicates."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def ordered_u64(a: np.ndarray) -> np.ndarray:
    """Order-preserving unsigned image of int64 / uint64 keys (what the library samples)."""
    if a.dtype == np.int64:
        return (a.view(np.uint64) ^ np.uint64(1 << 63))
    return a.astype(np.uint64)


def make_shard(kind: str, rank: int, n: int) -> np.ndarray:
    from cupynumeric_b200 import workloads as w

    if kind == "zipf":
        return w.c4_int64_zipf_shard(n, rank)
    if kind == "nearly_sorted":
        return w.c5_uint64_nearly_sorted_shard(n, rank, 2)
    if kind == "all_equal":
        return np.full(n, 7, dtype=np.int64)
    if kind == "one_empty":
        return np.arange(n, 0, -1, dtype=np.int64) if rank == 0 else np.empty(0, dtype=np.int64)
    raise ValueError(kind)


def worker(rank: int, world: int, port: int, kind: str, n: int, argsort: bool, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cupynumeric_b200 import _lib
        lib = _lib.lib()
        shard = make_shard(kind, rank, n)
        n_local = shard.size
        lens = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(lens, torch.tensor([n_local]))
        global_lo = int(sum(int(x) for x in lens[:rank]))

        okeys = ordered_u64(shard)

        # regular samples of the unsorted tile, exactly as the device kernel takes them
        s = lib.b2s_samples_per_rank()
        mine = np.zeros(s, dtype=_lib.SAMPLE_DTYPE)
        s_eff = min(s, n_local)
        for j in range(s):
            if j < s_eff:
                p = lib.b2s_host_sample_position(j, s_eff, n_local)
                mine[j] = (okeys[p], 0, p, lib.b2s_host_sample_weight(j, s_eff, n_local), rank, 0)
            else:
                mine[j] = (np.uint64(2**64 - 1), np.uint64(2**64 - 1), 0, 0, rank, 0)
        assert int(mine["weight"].sum()) == n_local
        gathered = [torch.zeros(mine.nbytes, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine.view(np.uint8)))
        samples = np.concatenate([g.numpy() for g in gathered]).view(_lib.SAMPLE_DTYPE).copy()
        splitters = np.zeros(world - 1, dtype=_lib.SAMPLE_DTYPE)
        assert lib.b2s_host_select_splitters(samples.ctypes.data, samples.size, world, splitters.ctypes.data) == 0

        # destination of every element of my tile; the pieces keep their input order
        dest = np.array([lib.b2s_host_bucket_of(splitters.ctypes.data, world - 1, rank, int(okeys[i]), 0, i)
                         for i in range(n_local)], dtype=np.int64)
        assert ((dest >= 0) & (dest < world)).all()
        idx = np.arange(n_local, dtype=np.int64) + global_lo
        send_counts = torch.tensor([int((dest == p).sum()) for p in range(world)])
        by_dest = np.argsort(dest, kind="stable")
        recv_counts = torch.zeros(world, dtype=torch.int64)
        dist.all_to_all_single(recv_counts, send_counts)
        recv_k = torch.zeros(int(recv_counts.sum()), dtype=torch.int64)
        recv_p = torch.zeros(int(recv_counts.sum()), dtype=torch.int64)
        dist.all_to_all_single(recv_k, torch.from_numpy(np.ascontiguousarray(shard[by_dest].view(np.int64))),
                               recv_counts.tolist(), send_counts.tolist())
        dist.all_to_all_single(recv_p, torch.from_numpy(np.ascontiguousarray(idx[by_dest])),
                               recv_counts.tolist(), send_counts.tolist())
        rk = recv_k.numpy().view(shard.dtype)
        # the pieces arrive in rank order, each in input order: a stable sort of what arrived is
        # this rank's part of the global stable sort
        m = np.argsort(rk, kind="stable")
        part = recv_p.numpy()[m] if argsort else rk[m]

        parts = [None] * world
        dist.all_gather_object(parts, part)
        shards = [None] * world
        dist.all_gather_object(shards, shard)
        if rank == 0:
            whole = np.concatenate(shards)
            got = np.concatenate(parts)
            want = np.argsort(whole, kind="stable") if argsort else np.sort(whole, kind="stable")
            ok = bool(np.array_equal(got, want.astype(got.dtype) if argsort else want))
            sizes = [len(p) for p in parts]
            ret.put((ok, sizes, whole.size))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,n,argsort", [("zipf", 20000, False), ("zipf", 20000, True),
                                           ("nearly_sorted", 16384, True), ("all_equal", 5000, True),
                                           ("one_empty", 3000, False), ("zipf", 100, True)])
def test_two_rank_sample_sort_over_gloo(kind, n, argsort):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29500 + (os.getpid() + hash((kind, n, argsort))) % 2000
    procs = [ctx.Process(target=worker, args=(r, 2, port, kind, n, argsort, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    ok, sizes, total = ret.get(timeout=10)
    assert ok, "rank-ordered concatenation differs from the global stable sort"
    assert sum(sizes) == total
    if kind in ("zipf", "all_equal", "nearly_sorted") and total >= 5000:
        # (rank, position) tie-breaking keeps the parts balanced even when one key dominates
        assert max(sizes) <= 0.55 * total, sizes


def rows_worker(rank: int, world: int, port: int, ret):
    """N-D arrays are tiled by rows: a sort along the last axis is local to every rank; a sort
    along the tiled axis makes every column a 1-D array spanning the ranks, which goes through
    the distributed sort and the move back into fixed extents.  The point task is played by the
    oracle, the two distributed calls by gloo stand-ins with the same contracts."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cupynumeric_b200._dist as dist_mod
        from cupynumeric_b200._thunk import _sort as sort_mod
        from cupynumeric_b200._thunk.deferred import DeferredArray, create_deferred_thunk
        from cupynumeric_b200.runtime import runtime
        from oracle import np_task_sort

        def fake_local(tile, argsort, stable, index_offset=0, out=None):
            a = tile.numpy()
            res = np_task_sort(a, a.shape[-1], argsort, index_offset=index_offset, ndim_is_1=a.ndim == 1)
            return torch.from_numpy(np.ascontiguousarray(res.reshape(a.shape)))

        def fake_dist_sort(tile, argsort, global_lo):
            """Same contract as dist_sort_1d: returns (this rank's part, its global start); the
            parts are deliberately uneven."""
            shards = [None] * world
            dist.all_gather_object(shards, tile.numpy().copy())
            whole = np.concatenate(shards)
            res = np.argsort(whole, kind="stable").astype(np.int64) if argsort else np.sort(whole, kind="stable")
            cut = [0, max(1, whole.size // 3), whole.size][rank:rank + 2]
            return torch.from_numpy(res[cut[0]:cut[1]].copy()), cut[0]

        def fake_rebalance(part, part_start, out, out_start):
            parts = [None] * world
            dist.all_gather_object(parts, (int(part_start), part.numpy().copy()))
            whole = np.concatenate([p for _, p in sorted(parts, key=lambda t: t[0])])
            out.copy_(torch.from_numpy(whole[out_start:out_start + out.numel()].copy()))

        def fake_dist_sort_nd(tile, argsort):
            """Same contract as dist_sort_nd: every rank holds a slice of every row; returns this
            rank's slice of every sorted row (values, or positions along the whole row)."""
            tiles = [None] * world
            dist.all_gather_object(tiles, tile.numpy().copy())
            full = np.concatenate(tiles, axis=1)
            res = np.argsort(full, axis=1, kind="stable").astype(np.int64) if argsort else np.sort(full, axis=1, kind="stable")
            lo = sum(t.shape[1] for t in tiles[:rank])
            return torch.from_numpy(res[:, lo:lo + tile.shape[1]].copy())

        sort_mod.local_sort_tile = fake_local
        dist_mod.dist_sort_1d = fake_dist_sort
        dist_mod.rebalance_1d = fake_rebalance
        dist_mod.dist_sort_nd = fake_dist_sort_nd
        assert runtime.num_procs == world
        whole = np.random.default_rng(9).integers(-50, 50, (8, 13)).astype(np.int32)
        block = whole[rank * 4:(rank + 1) * 4]
        out = create_deferred_thunk(block.shape, np.int64)
        out.sort(DeferredArray(torch.from_numpy(block.copy()), global_lo=rank * 4), argsort=True, axis=-1, kind="stable")
        ok_rows = bool(np.array_equal(out.base.numpy(), np.argsort(block, axis=-1, kind="stable")))
        ok_split = True
        for argsort in (False, True):
            res = create_deferred_thunk(block.shape, np.int64 if argsort else np.int32)
            res.sort(DeferredArray(torch.from_numpy(block.copy()), global_lo=rank * 4), argsort=argsort, axis=0, kind="stable")
            want = (np.argsort(whole, axis=0, kind="stable") if argsort else np.sort(whole, axis=0, kind="stable"))
            ok_split &= bool(np.array_equal(res.base.numpy(), want[rank * 4:(rank + 1) * 4]))
            ok_split &= res.global_lo == rank * 4 and res.tiled_axis == 0
        # fewer columns than ranks: each column takes the distributed 1-D sort and the move back
        thin = whole[:, :1]
        for argsort in (False, True):
            res = create_deferred_thunk((4, 1), np.int64 if argsort else np.int32)
            res.sort(DeferredArray(torch.from_numpy(thin[rank * 4:(rank + 1) * 4].copy()), global_lo=rank * 4), argsort=argsort,
                     axis=0, kind="stable")
            want = (np.argsort(thin, axis=0, kind="stable") if argsort else np.sort(thin, axis=0, kind="stable"))
            ok_split &= bool(np.array_equal(res.base.numpy(), want[rank * 4:(rank + 1) * 4]))
        ret.put((rank, ok_rows, ok_split))
    finally:
        dist.destroy_process_group()


def test_row_blocks_sort_locally_and_split_axis_goes_distributed():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=rows_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = sorted(ret.get(timeout=10) for _ in range(2))
    assert got == [(0, True, True), (1, True, True)]
