"""Benchmark of the SORT path: sorted Gkeys/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path (one SORT task) over one batch of seeded synthetic keys.
At one GPU the default workload is the 1-D float32 stable argsort of 2^28 keys (N(0,1) with 0.1 %
NaN and 1 % duplicates, int64 indices out).  ``value`` is measured with the input resident in HBM;
``e2e`` goes through the public API with pinned host buffers (upload of the keys and download of
the result inside the timed region).  ``--impl reference`` times the reference's CPU arithmetic
(Thrust OpenMP back-end, every host thread) on a bounded sample of the same workload.
Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used when MEASURED_PEAKS.json is absent

# DRAM bytes (read + write) of one onesweep launch per key, from the ncu capture summarised in
# profiles/ (scaled to a full launch by the number of keys); None until a capture exists.
NCU_TRAFFIC_BYTES_PER_KEY = {"c1": 7.77, "c2": 13.8}  # c2: mean of the four passes (10.8, 14.8, 14.8, 14.7)


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------------------------
# workloads: name -> description used by both arms
# ------------------------------------------------------------------------------------------------
def make_workload(name: str, rank: int, nranks: int, scale_log2: int | None):
    """Returns dict(keys=np.ndarray (this rank's tile), argsort, segment, label, bytes_per_key,
    sweep_bytes_per_key, dtype)."""
    from cupynumeric_b200 import workloads as w

    if name == "c1":
        n = 1 << (scale_log2 or 24)
        return dict(keys=w.c1_int32_uniform(n, seed=101 + rank), argsort=False, label=f"1-D int32 sort, N=2^{n.bit_length()-1}, uniform full range, seed 101",
                    bytes_per_key=36.0, sweep_bytes_per_key=8.0, dtype="i32")
    if name == "c2":
        n = 1 << (scale_log2 or 28)
        # rank 0 holds the configuration's own array; further ranks draw fresh shards of the same distribution
        return dict(keys=w.c2_float32_nan_dups(n, seed=202 + rank), argsort=True,
                    label=f"1-D float32 stable argsort -> int64, N=2^{n.bit_length()-1}, N(0,1) + 0.1% NaN + 1% duplicates, seed 202",
                    bytes_per_key=88.0, sweep_bytes_per_key=21.0, dtype="f32")
    if name == "c3":
        rows = (1 << (scale_log2 or 16)) // nranks
        a = w.c3_float64_rows((rows, 4096), seed=303 + rank)
        return dict(keys=a, argsort=False, label=f"2-D float64 ({rows * nranks}, 4096) sort along axis -1, uniform [0,1), row blocks per GPU",
                    bytes_per_key=16.0, sweep_bytes_per_key=16.0, dtype="f64")
    if name == "c4":
        n = 1 << (scale_log2 or 28)
        return dict(keys=w.c4_int64_zipf_shard(n, rank), argsort=False,
                    label=f"1-D int64 distributed sort, 2^{n.bit_length()-1} keys/GPU, Zipf(1.2) clipped to [0,2^40)",
                    bytes_per_key=136.0 if nranks == 1 else 152.0, sweep_bytes_per_key=16.0, dtype="i64")
    if name == "c5":
        n = 1 << (scale_log2 or 28)
        return dict(keys=w.c5_uint64_nearly_sorted_shard(n, rank, nranks), argsort=True,
                    label=f"1-D uint64 distributed stable argsort, 2^{n.bit_length()-1} keys/GPU, ascending with 1% pair swaps",
                    bytes_per_key=248.0 if nranks == 1 else 272.0, sweep_bytes_per_key=31.0, dtype="u64")
    raise SystemExit(f"unknown workload {name}")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_time(keys: np.ndarray, argsort: bool, sample: int, steps: int, warmup: int):
    """Times the reference's CPU arithmetic (OpenMP back-end, all host threads) on the first
    ``sample`` keys (whole rows for 2-D inputs).  Returns (Gkeys/s, seconds per step, threads)."""
    from oracle import num_threads, thrust_task_sort

    if keys.ndim == 2:
        rows = max(1, min(keys.shape[0], sample // keys.shape[1]))
        part, segment, one_d = keys[:rows], keys.shape[1], False
    else:
        part, segment, one_d = keys[:sample], min(sample, keys.size), True
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        thrust_task_sort(part, segment, argsort, ndim_is_1=one_d, backend="omp")
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    per = float(np.mean(times))
    return part.size / per / 1e9, per, num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload, 0, 1, args.scale_log2)
    sample = 1 << args.cpu_sample_log2
    gk, per, threads = cpu_reference_time(wl["keys"], wl["argsort"], sample, args.steps, min(args.warmup, 1))
    n = min(sample, wl["keys"].size)
    line = {
        "impl": "reference", "metric": "sorted Gkeys/s", "value": gk, "unit": "Gkeys/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": wl["label"], "sample": f"first {n} keys of the workload per step"},
        "cpu_baseline": {"value": gk, "unit": "Gkeys/s", "cores": threads, "kind": "port",
                         "sample": f"thrust::omp::par stable sort of the first {n} keys, {args.steps} steps"},
        "e2e": {"value": gk, "unit": "Gkeys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist

    import cupynumeric_b200 as num
    from cupynumeric_b200 import _lib
    from cupynumeric_b200._thunk._sort import local_sort_tile

    nranks = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if nranks > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = _lib.lib()

    wl = make_workload(args.workload, rank, nranks, args.scale_log2)
    host = wl["keys"]
    n_local = host.size
    distributed = nranks > 1 and host.ndim == 1
    arr = num.array(host, global_lo=rank * n_local if host.ndim == 1 else 0)
    tile = arr.torch()
    out = torch.empty(tile.shape, dtype=torch.int64 if wl["argsort"] else tile.dtype, device=tile.device)

    def step():
        if distributed:
            r = num.argsort(arr, kind="stable") if wl["argsort"] else num.sort(arr)
            return r
        return local_sort_tile(tile, wl["argsort"], True, index_offset=0, out=out)

    def barrier():
        if nranks > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = lib.b2s_launch_count(-1)
    lib.b2s_profile_enable(1)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    launches = lib.b2s_launch_count(-1) - launches0
    kind = _lib.K_SEGSORT if host.ndim == 2 else _lib.K_SWEEP
    tot, cnt = ctypes.c_double(0), ctypes.c_ulonglong(0)
    lib.b2s_profile_read(kind, ctypes.byref(tot), ctypes.byref(cnt))
    lib.b2s_profile_enable(0)
    if nranks > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_keys = n_local * nranks
    value = total_keys * args.steps / (ms * 1e-3) / 1e9

    # ---- end to end through the public API with pinned host buffers ----
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    pinned_in = torch.from_numpy(host.view(np.int32 if host.dtype.itemsize == 4 else np.int64)).pin_memory()
    host_in = pinned_in.numpy().view(host.dtype)
    res_dtype = np.int64 if wl["argsort"] else host.dtype
    e2e_ms, h2d, d2h = None, int(host.nbytes), None
    if not distributed:
        pinned_out = torch.empty(host.shape, dtype=torch.int64 if res_dtype == np.int64 else pinned_in.dtype).pin_memory()
        host_out = pinned_out.numpy().view(res_dtype)
        d2h = int(host_out.nbytes)

        def e2e_step():
            a = num.array(host_in)
            r = num.argsort(a, kind="stable") if wl["argsort"] else num.sort(a)
            r.to_numpy(out=host_out)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    else:
        # each rank's part of the result has its own length: a pinned buffer with head-room
        cap = int(n_local * 1.5) + 1024
        pinned_out = torch.empty(cap, dtype=torch.int64 if res_dtype == np.int64 else pinned_in.dtype).pin_memory()
        host_out = pinned_out.numpy().view(res_dtype)
        got = [0]

        def e2e_step():
            a = num.array(host_in, global_lo=rank * n_local)
            r = num.argsort(a, kind="stable") if wl["argsort"] else num.sort(a)
            got[0] = r.size
            r.to_numpy(out=host_out[: r.size])

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        d2h = int(got[0]) * np.dtype(res_dtype).itemsize
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = total_keys * e2e_steps / (e2e_ms * 1e-3) / 1e9

    if rank != 0:
        if nranks > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_hbm_peak()
    launches_k = int(cnt.value)
    roofline = None
    if launches_k:
        avg_ms = tot.value / launches_k
        # algorithmic bytes of one launch of the dominant kernel: keys one launch processes x bytes per key
        keys_one_launch = n_local
        achieved = wl["sweep_bytes_per_key"] * keys_one_launch / (avg_ms * 1e-3) / 1e9
        traffic_pk = NCU_TRAFFIC_BYTES_PER_KEY.get(args.workload)
        roofline = {"bound": "hbm", "kernel": "segsort_kernel" if host.ndim == 2 else "onesweep_kernel",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_source": f"of {peak_kind}", "avg_launch_ms": avg_ms, "launches_timed": launches_k,
                    "algorithmic_bytes_per_launch": wl["sweep_bytes_per_key"] * keys_one_launch,
                    "traffic": traffic_pk * keys_one_launch if traffic_pk else None}
    job_gbs = wl["bytes_per_key"] * n_local * args.steps / (ms * 1e-3) / 1e9

    cpu = None
    if nranks == 1 and not args.no_cpu_baseline:
        sample = 1 << args.cpu_sample_log2
        gk, per, threads = cpu_reference_time(host, wl["argsort"], sample, 1, 0)
        cpu = {"value": gk, "unit": "Gkeys/s", "cores": threads, "kind": "port",
               "sample": f"thrust::omp::par stable sort of the first {min(sample, host.size)} keys of the workload, 1 step ({per:.2f} s)"}

    line = {
        "metric": "sorted Gkeys/s", "value": value, "unit": "Gkeys/s", "n_gpus": nranks, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": wl["label"], "keys_per_gpu": n_local,
                   "l2": "inputs larger than the 126 MB L2, no flush needed" if host.nbytes > (126 << 20)
                   else "input smaller than L2; every step re-reads it after the sort's own temporaries evicted it"},
        "roofline": roofline,
        "job_roofline": {"algorithmic_bytes_per_key": wl["bytes_per_key"], "achieved": job_gbs, "peak": peak,
                         "unit": "GB/s", "frac": job_gbs / peak, "peak_source": f"of {peak_kind}",
                         "frac_of_8TBs": job_gbs / 8000.0},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "Gkeys/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    print(json.dumps(line))
    if nranks > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--scale-log2", type=int, default=None, help="log2 of the key count (per GPU); default: the configuration's size")
    ap.add_argument("--cpu-sample-log2", type=int, default=25)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload is None:
        args.workload = "c2"
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
