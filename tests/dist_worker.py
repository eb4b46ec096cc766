"""Child process of the multi-GPU test: one rank of a distributed sort through the public API,
checked against the oracle on rank 0.  Launched with torch.distributed.run."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    workload = sys.argv[1]
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 1 << 20
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    import cupynumeric_b200 as num
    from cupynumeric_b200 import workloads as w
    from cupynumeric_b200._dist import destroy_comm

    if workload == "recache":
        # several sorts of growing size in one process with a one-entry mapping table
        # (B2S_PEER_CACHE=1, set by the test): mappings of earlier calls get closed and replaced
        keep = []
        for m in (30_000, 400_000, 3_000_000, 30_000):
            shard = np.random.default_rng(m + rank).integers(-1000, 1000, m).astype(np.int32)
            shards = [None] * world
            dist.all_gather_object(shards, shard)
            res = num.argsort(num.array(shard, global_lo=rank * m), kind="stable")
            keep.append(res)                       # holds its block, so later calls get other blocks
            parts = [None] * world
            dist.all_gather_object(parts, res.to_numpy())
            assert np.array_equal(np.concatenate(parts), np.argsort(np.concatenate(shards), kind="stable")), m
        dist.barrier()
        if rank == 0:
            print("DIST_OK recache")
        destroy_comm()
        dist.destroy_process_group()
        return
    if workload == "search":
        # sort across the ranks, then look values up in the distributed result
        shard = np.random.default_rng(50 + rank).integers(-10_000, 10_000, 200_000).astype(np.int64)
        shards = [None] * world
        dist.all_gather_object(shards, shard)
        whole = np.sort(np.concatenate(shards), kind="stable")
        srt = num.sort(num.array(shard, global_lo=rank * shard.size))
        v = np.random.default_rng(7).integers(-11_000, 11_000, 5000).astype(np.int64)   # same on every rank
        for side in ("left", "right"):
            got = num.searchsorted(srt, v, side=side).to_numpy()
            assert np.array_equal(got, np.searchsorted(whole, v, side=side)), side
        # unique across the ranks: parts are sorted, disjoint and in rank order
        few = np.random.default_rng(60 + rank).integers(0, 50, 100_000).astype(np.int64)
        fews = [None] * world
        dist.all_gather_object(fews, few)
        uparts = [None] * world
        dist.all_gather_object(uparts, num.unique(num.array(few, global_lo=rank * few.size)).to_numpy())
        assert np.array_equal(np.concatenate(uparts), np.unique(np.concatenate(fews))), "distributed unique"
        dist.barrier()
        if rank == 0:
            print("DIST_OK search")
        destroy_comm()
        dist.destroy_process_group()
        return
    if workload == "split2d":
        # a (world*300, 7) int32 array tiled by rows; sort along axis 0 (the tiled axis) and flat
        rng = np.random.default_rng(100 + rank)
        block = rng.integers(-1000, 1000, (300, 7)).astype(np.int32)
        blocks = [None] * world
        dist.all_gather_object(blocks, block)
        whole = np.concatenate(blocks)
        arr = num.array(block, global_lo=rank * 300)
        got_s = num.sort(arr, axis=0).to_numpy()
        got_a = num.argsort(arr, axis=0, kind="stable").to_numpy()
        want_s, want_a = np.sort(whole, axis=0, kind="stable"), np.argsort(whole, axis=0, kind="stable")
        assert np.array_equal(got_s, want_s[rank * 300:(rank + 1) * 300]), "sort along the split axis"
        assert np.array_equal(got_a, want_a[rank * 300:(rank + 1) * 300]), "argsort along the split axis"
        flat = num.sort(arr, axis=None)
        parts = [None] * world
        dist.all_gather_object(parts, flat.to_numpy())
        assert np.array_equal(np.concatenate(parts), np.sort(whole, axis=None, kind="stable")), "flattened sort"
        assert flat.global_lo == sum(len(p) for p in parts[:rank]), "global start of the flattened part"
        rows = num.sort(arr, axis=1).to_numpy()
        assert np.array_equal(rows, np.sort(block, axis=1))
        dist.barrier()
        if rank == 0:
            print("DIST_OK split2d")
        destroy_comm()
        dist.destroy_process_group()
        return
    if workload == "c4":
        shard, argsort = w.c4_int64_zipf_shard(n, rank), False
    elif workload == "c5":
        shard, argsort = w.c5_uint64_nearly_sorted_shard(n, rank, world), True
    elif workload == "tiny":
        shard, argsort = np.random.default_rng(rank).integers(-5, 5, 1000).astype(np.int32), True
    elif workload == "mixed":   # a long tile (32-bit positions in the exchange) beside a short one (int64)
        m = 50000 if rank == 0 else 700
        shard, argsort = np.random.default_rng(7 + rank).integers(-40, 40, m).astype(np.int16), True
    elif workload == "c64":     # complex64 keys: one 8-byte (real, imaginary) radix key
        rng = np.random.default_rng(31 + rank)
        shard = (rng.integers(-30, 30, 60_000) + 1j * rng.integers(-30, 30, 60_000)).astype(np.complex64)
        argsort = True
    elif workload == "empty":   # only rank 0 holds data; everybody still takes part
        shard = np.arange(5000, 0, -1, dtype=np.int64) if rank == 0 else np.empty(0, dtype=np.int64)
        argsort = False
    else:
        shard, argsort = w.c2_float32_nan_dups(n, seed=202 + rank), True
    if rank == world - 1 and workload == "c4":
        shard = shard[: n // 3]  # ragged tiles
    lens = [None] * world
    dist.all_gather_object(lens, int(shard.size))
    lo = sum(lens[:rank])
    arr = num.array(shard, global_lo=lo)
    res = num.argsort(arr, kind="stable") if argsort else num.sort(arr)
    part = res.to_numpy()
    parts, shards, starts = [None] * world, [None] * world, [None] * world
    dist.all_gather_object(parts, part)
    dist.all_gather_object(shards, shard)
    dist.all_gather_object(starts, res.global_lo)
    if rank == 0:
        whole = np.concatenate(shards)
        got = np.concatenate(parts)
        want = np.argsort(whole, kind="stable") if argsort else np.sort(whole, kind="stable")
        assert got.shape == want.shape, (got.shape, want.shape)
        same = np.array_equal(got, want) if argsort else np.array_equal(got.view(np.uint8), want.view(np.uint8))
        assert same, "distributed result differs from the global stable sort"
        assert starts == [int(x) for x in np.cumsum([0] + [len(p) for p in parts])[:-1]], starts
        sizes = [len(p) for p in parts]
        if workload not in ("tiny", "empty", "mixed"):
            assert max(sizes) <= 1.2 * sum(sizes) / world + 16, sizes
        print("DIST_OK", workload, sizes)
    destroy_comm()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
