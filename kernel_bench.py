"""Micro-benchmarks of single kernels through the C ABI, with CUDA-event timing per kernel family.

    python kernel_bench.py merge --dtype int64 --runs 8 --log2 27 [--payload]
    python kernel_bench.py sort  --dtype float32 --log2 28 [--argsort] [--segment L]
    python kernel_bench.py select --dtype float32 --log2 28 [--argsort]      (partition by selection, kth = n/2)

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        kernel_bench.py dist --dtype float32 --log2 27 [--argsort]

    python kernel_bench.py dist-threads --ranks 8 --dtype float32 --log2 24 [--argsort]

`dist-threads` runs the distributed sort with its ranks as threads of this process on ONE GPU (the
thread form of the collectives): the partition kernels write into buffers of the same GPU, so this
shows their cost without NVLink, and it is a single process that a profiler can follow.
`merge` times b2s_kway_merge on `runs` sorted runs holding 2^log2 elements in all; `sort` times
b2s_local_sort; `dist` (one process per GPU) times the distributed 1-D sort of 2^log2 keys per GPU,
first without the per-kernel events (the step time), then with them (where the time goes).
B2S_DIST_P2P=0 selects the NCCL exchange.  Small cases of these commands are what the ncu summaries
under profiles/ capture.
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np
import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from cupynumeric_b200 import _lib  # noqa: E402
from cupynumeric_b200._thunk._sort import local_sort_tile  # noqa: E402

KINDS = ["hist", "scan", "sweep", "fixup", "segsort", "unit", "dist", "merge", "xchg"]


def _random(dtype: torch.dtype, n: int) -> torch.Tensor:
    if dtype.is_floating_point or dtype.is_complex:
        return torch.randn(n, device="cuda", dtype=dtype)
    info = torch.iinfo(dtype)
    return torch.randint(max(info.min, -2**62), min(info.max, 2**62), (n,), device="cuda", dtype=torch.int64).to(dtype)


def _report(lib, iters: int) -> str:
    out = []
    for k, name in enumerate(KINDS):
        tot, cnt = ctypes.c_double(), ctypes.c_ulonglong()
        lib.b2s_profile_read(k, ctypes.byref(tot), ctypes.byref(cnt))
        if cnt.value:
            out.append(f"{name} {tot.value / iters:.3f} ms ({cnt.value // iters} launches)")
    return ", ".join(out)


def bench_merge(args) -> None:
    lib = _lib.lib()
    dtype = getattr(torch, args.dtype)
    n_each = (1 << args.log2) // args.runs
    runs = [torch.sort(_random(dtype, n_each)).values for _ in range(args.runs)]
    pays = [torch.arange(n_each, device="cuda", dtype=torch.int64) + i * n_each for i in range(args.runs)] if args.payload else None
    total = n_each * args.runs
    kp = (ctypes.c_void_p * args.runs)(*[r.data_ptr() for r in runs])
    pp = (ctypes.c_void_p * args.runs)(*[p.data_ptr() for p in pays]) if pays else None
    lens = (ctypes.c_size_t * args.runs)(*([n_each] * args.runs))
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_kway_merge_workspace_bytes(total, args.runs, ctypes.byref(need)), "workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    out = torch.empty(total, dtype=torch.int64 if pays else dtype, device="cuda")
    code = _lib.DTYPE_CODE[np.dtype(args.dtype)]

    def call():
        _lib.check(lib.b2s_kway_merge(code, args.runs, kp, pp, lens, out.data_ptr(), ws.data_ptr(), ws.numel(),
                                      torch.cuda.current_stream().cuda_stream), "b2s_kway_merge")

    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    lib.b2s_profile_enable(1)
    for _ in range(args.iters):
        call()
    torch.cuda.synchronize()
    print(f"merge {args.dtype} runs={args.runs} total=2^{args.log2} payload={bool(pays)}: {_report(lib, args.iters)}")
    lib.b2s_profile_enable(0)


def bench_sort(args) -> None:
    lib = _lib.lib()
    dtype = getattr(torch, args.dtype)
    n = 1 << args.log2
    x = _random(dtype, n)
    if args.segment:
        x = x.reshape(-1, args.segment)
    out = torch.empty(x.shape, dtype=torch.int64 if args.argsort else dtype, device="cuda")
    for _ in range(args.warmup):
        local_sort_tile(x, args.argsort, True, out=out)
    torch.cuda.synchronize()
    lib.b2s_profile_enable(1)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iters):
        local_sort_tile(x, args.argsort, True, out=out)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.iters
    print(f"sort {args.dtype} n=2^{args.log2} segment={args.segment or n} argsort={args.argsort}: {ms:.3f} ms "
          f"-> {n / ms / 1e6:.1f} Gkeys/s; {_report(lib, args.iters)}")
    lib.b2s_profile_enable(0)


def bench_select(args) -> None:
    """b2s_partition_1d (radix select + three-block partition) at kth = n / 2."""
    lib = _lib.lib()
    dtype = getattr(torch, args.dtype)
    n = 1 << args.log2
    x = _random(dtype, n)
    out = torch.empty(n, dtype=torch.int64 if args.argsort else dtype, device="cuda")
    need = ctypes.c_size_t(0)
    _lib.check(lib.b2s_partition_workspace_bytes(ctypes.byref(need)), "b2s_partition_workspace_bytes")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    code = _lib.DTYPE_CODE[np.dtype(args.dtype)]
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        _lib.check(lib.b2s_partition_1d(code, x.data_ptr(), None if args.argsort else out.data_ptr(),
                                        out.data_ptr() if args.argsort else None, n, n // 2, 0, ws.data_ptr(), ws.numel(), stream),
                   "b2s_partition_1d")

    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    lib.b2s_profile_enable(1)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iters):
        call()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.iters
    print(f"select {args.dtype} n=2^{args.log2} kth=n/2 argsort={args.argsort}: {ms:.3f} ms -> {n / ms / 1e6:.1f} Gkeys/s; "
          f"{_report(lib, args.iters)}")
    lib.b2s_profile_enable(0)


def bench_dist(args) -> None:
    import os
    import time

    import torch.distributed as dist

    from cupynumeric_b200 import array, argsort, sort
    from cupynumeric_b200._dist import destroy_comm

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    lib = _lib.lib()
    dtype = getattr(torch, args.dtype)
    n = 1 << args.log2
    torch.manual_seed(1000 + rank)
    arr = array(_random(dtype, n), global_lo=rank * n)

    def call():
        return argsort(arr, kind="stable") if args.argsort else sort(arr)

    def timed(profile: bool) -> float:
        for _ in range(args.warmup):
            call()
        torch.cuda.synchronize()
        dist.barrier()
        lib.b2s_profile_enable(1 if profile else 0)
        t0 = time.perf_counter()
        for _ in range(args.iters):
            call()          # returns after its own final synchronisation
        torch.cuda.synchronize()
        dist.barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / args.iters * 1e3], device="cuda", dtype=torch.float64)
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return float(dt.item())

    ms = timed(False)
    timed(True)
    parts = _report(lib, args.iters)
    lib.b2s_profile_enable(0)
    if rank == 0:
        print(f"dist {args.dtype} 2^{args.log2}/GPU x{world} argsort={args.argsort}: {ms:.2f} ms/step -> "
              f"{n * world / ms / 1e6:.1f} Gkeys/s; rank 0 kernels: {parts}")
    destroy_comm()
    dist.destroy_process_group()


def bench_dist_threads(args) -> None:
    import threading

    lib = _lib.lib()
    nranks, n = args.ranks, 1 << args.log2
    dtype = getattr(torch, args.dtype)
    code = _lib.DTYPE_CODE[np.dtype(args.dtype)]
    torch.manual_seed(1)
    shards = [_random(dtype, n) for _ in range(nranks)]
    torch.cuda.synchronize()

    class Pool:
        def __init__(self):
            self.live = {}
            self.alloc_cb = _lib.ALLOC_FN(self._alloc)
            self.free_cb = _lib.FREE_FN(self._free)

        def _alloc(self, _ctx, nbytes):
            t = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device="cuda")
            self.live[t.data_ptr()] = t
            return t.data_ptr()

        def _free(self, _ctx, ptr):
            self.live.pop(ptr, None)

    def one_call():
        ops = (_lib.CommOps * nranks)()
        _lib.check(lib.b2s_thread_comm_create(nranks, ops), "b2s_thread_comm_create")
        status = [None] * nranks

        def rank_main(r):
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                pool = Pool()
                out_ptr, out_len, out_start = ctypes.c_void_p(), ctypes.c_size_t(), ctypes.c_int64()
                status[r] = lib.b2s_dist_sort_1d_ops(
                    code, shards[r].data_ptr(), n, r * n, int(args.argsort), ctypes.byref(ops[r]), r, nranks,
                    ctypes.cast(pool.alloc_cb, ctypes.c_void_p), ctypes.cast(pool.free_cb, ctypes.c_void_p), None, None, None,
                    ctypes.byref(out_ptr), ctypes.byref(out_len), ctypes.byref(out_start), stream.cuda_stream)

        threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(nranks)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for r in range(nranks):
            lib.b2s_thread_comm_destroy(ctypes.byref(ops[r]))
        assert all(s == 0 for s in status), status

    for _ in range(args.warmup):
        one_call()
    lib.b2s_profile_enable(1)
    for _ in range(args.iters):
        one_call()
    torch.cuda.synchronize()
    print(f"dist-threads {args.dtype} 2^{args.log2} x{nranks} ranks on one GPU argsort={args.argsort}; all ranks' kernels per call: "
          f"{_report(lib, args.iters)}")
    lib.b2s_profile_enable(0)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="what", required=True)
    m = sub.add_parser("merge")
    m.add_argument("--dtype", default="int64")
    m.add_argument("--runs", type=int, default=8)
    m.add_argument("--log2", type=int, default=27)
    m.add_argument("--payload", action="store_true")
    s = sub.add_parser("sort")
    s.add_argument("--dtype", default="float32")
    s.add_argument("--log2", type=int, default=28)
    s.add_argument("--argsort", action="store_true")
    s.add_argument("--segment", type=int, default=0)
    q = sub.add_parser("select")
    q.add_argument("--dtype", default="float32")
    q.add_argument("--log2", type=int, default=28)
    q.add_argument("--argsort", action="store_true")
    d = sub.add_parser("dist")
    d.add_argument("--dtype", default="float32")
    d.add_argument("--log2", type=int, default=27)
    d.add_argument("--argsort", action="store_true")
    t = sub.add_parser("dist-threads")
    t.add_argument("--ranks", type=int, default=8)
    t.add_argument("--dtype", default="float32")
    t.add_argument("--log2", type=int, default=24)
    t.add_argument("--argsort", action="store_true")
    for p in (m, s, q, d, t):
        p.add_argument("--iters", type=int, default=5)
        p.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    if args.what == "dist":
        import os

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        bench_dist(args)
        return
    torch.cuda.set_device(0)
    {"merge": bench_merge, "sort": bench_sort, "select": bench_select, "dist-threads": bench_dist_threads}[args.what](args)


if __name__ == "__main__":
    main()
