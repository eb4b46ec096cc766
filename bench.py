"""Benchmark of the SORT path: sorted Gkeys/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path (one SORT task through the public API) over one batch of
seeded synthetic keys.  The headline workload (``value``) is the 1-D float32 stable argsort of
2^28 keys per GPU (N(0,1) with 0.1 % NaN and 1 % duplicates, int64 indices out); with several
GPUs the same workload is sharded, 2^28 keys per GPU, and goes through the distributed sort.
``value`` is measured with the input resident in HBM; ``e2e`` goes through the same API with
pinned host buffers (upload of the keys and download of the result inside the timed region).

Every number is backed by a check made in the same run (``verified``): first the same step at a
reduced size against the CPU oracle (bit for bit; with several GPUs the rank-ordered concatenation
against the oracle's global stable sort), then the full-size result of the warm-up on the device
(sorted in the sort's total order, neighbouring ranks in order, element count, multiset /
permutation fingerprints, stability of every tie).  A failed check ends the run with exit code 1.

``configs`` carries the other benchmark configurations beside the headline, each timed and checked
the same way, with its roofline (the larger of the HBM floor and the NVLink floor), the dominant
kernel's event-timed share and, on one GPU, the CCCL library sort the reference's GPU variant
calls (``cub_baseline``, measurement infrastructure under ``oracle/``).

``--impl reference`` times the reference's CPU arithmetic (Thrust OpenMP back-end, every host
thread) on the headline workload.  Prints one JSON line (rank 0).
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

FALLBACK_HBM_GBS = 6650.0   # used when MEASURED_PEAKS.json is absent
NVLINK_GBS = 900.0          # per direction per GPU, the figure the roofline is defined on
L2_BYTES = 126 << 20

# name -> description.  hbm_bytes: algorithmic bytes per key on one GPU / on several (the second
# adds the k-way merge); nvlink_bytes: bytes per key that cross NVLink per direction, before the
# (P-1)/P factor; sweep_bytes: algorithmic bytes per key of one launch of the dominant kernel.
CONFIGS = {
    "c1": dict(label="1-D int32 sort, N=2^{log2} per GPU, keys uniform over the full int32 range", dtype="i32", log2=24,
               argsort=False, hbm_bytes=(36.0, 36.0), nvlink_bytes=4.0, sweep_bytes=8.0, kernel="onesweep_kernel",
               multi="distributed"),
    "c2": dict(label="1-D float32 stable argsort -> int64, N=2^{log2} per GPU, N(0,1) + 0.1% NaN + 1% duplicates",
               dtype="f32", log2=28, argsort=True, hbm_bytes=(88.0, 108.0), nvlink_bytes=12.0, sweep_bytes=21.0,
               kernel="onesweep_kernel", multi="distributed"),
    "c3": dict(label="2-D float64 ({rows}, 4096) sort along axis -1, uniform [0,1), row blocks per GPU", dtype="f64",
               log2=28, argsort=False, hbm_bytes=(16.0, 16.0), nvlink_bytes=0.0, sweep_bytes=16.0,
               kernel="segmerge_kernel", multi="rows"),
    "c4": dict(label="1-D int64 distributed sort, 2^{log2} keys per GPU, Zipf(1.2) clipped to [0,2^40)", dtype="i64",
               log2=28, argsort=False, hbm_bytes=(136.0, 152.0), nvlink_bytes=8.0, sweep_bytes=16.0,
               kernel="onesweep_kernel", multi="distributed"),
    "c5": dict(label="1-D uint64 distributed stable argsort -> int64, 2^{log2} keys per GPU, ascending with 1% pair swaps",
               dtype="u64", log2=28, argsort=True, hbm_bytes=(248.0, 272.0), nvlink_bytes=16.0, sweep_bytes=31.0,
               kernel="onesweep_kernel", multi="distributed"),
}


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic_bytes_per_key():
    """DRAM bytes per key of one launch of the dominant kernel, from the committed ncu summaries."""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json")))["bytes_per_key_per_launch"]
    except Exception:
        return {}


# ------------------------------------------------------------------------------------------------
# inputs
# ------------------------------------------------------------------------------------------------
def config_label(name, log2, nranks):
    c = CONFIGS[name]
    return c["label"].format(log2=log2, rows=(1 << log2) // 4096)


def device_input(name, log2, rank, nranks, device):
    """This rank's tile of the configuration, drawn on the GPU."""
    from cupynumeric_b200 import workloads as w

    n = 1 << log2
    if name == "c1":
        return w.c1_int32_uniform_device(n, device, seed=101 + rank)
    if name == "c2":
        return w.c2_float32_nan_dups_device(n, device, seed=202 + rank)
    if name == "c3":
        rows = (n // 4096) // nranks
        return w.c3_float64_rows_device((rows, 4096), device, seed=303 + rank)
    if name == "c4":
        return w.c4_int64_zipf_shard_device(n, rank, device)
    if name == "c5":
        import torch
        return w.c5_uint64_nearly_sorted_shard_device(n, rank, nranks, device).view(torch.uint64)
    raise SystemExit(f"unknown workload {name}")


def host_input(name, log2, rank, nranks):
    """The same tile from the NumPy generators (reduced-size checks, reference arm)."""
    from cupynumeric_b200 import workloads as w

    n = 1 << log2
    if name == "c1":
        return w.c1_int32_uniform(n, seed=101 + rank)
    if name == "c2":
        return w.c2_float32_nan_dups(n, seed=202 + rank)
    if name == "c3":
        return w.c3_float64_rows(((n // 4096) // nranks, 4096), seed=303 + rank)
    if name == "c4":
        return w.c4_int64_zipf_shard(n, rank)
    if name == "c5":
        return w.c5_uint64_nearly_sorted_shard(n, rank, nranks)
    raise SystemExit(f"unknown workload {name}")


# ------------------------------------------------------------------------------------------------
# checks (torch ops on the device are the checker here, never the thing measured)
# ------------------------------------------------------------------------------------------------
_MIN64 = -(1 << 63)


def ordered_i64(t):
    """int64 tensor whose signed order is the sort's total order of ``t``: integers by value,
    floats as -inf < .. < -0.0 == +0.0 < .. < +inf < NaN (all NaNs equal)."""
    import torch

    if t.dtype == torch.uint64:
        return t.view(torch.int64) ^ _MIN64
    if t.dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool, torch.uint16, torch.uint32):
        if t.dtype == torch.uint16:
            return t.view(torch.int16).to(torch.int64) & 0xFFFF
        if t.dtype == torch.uint32:
            return t.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        return t.to(torch.int64)
    if t.dtype in (torch.float16, torch.float32, torch.float64):
        v = t.to(torch.float64).view(torch.int64) if t.dtype != torch.float64 else t.view(torch.int64)
        o = torch.where(v < 0, (~v) ^ _MIN64, v)
        o = torch.where(t == 0, torch.zeros_like(o), o)
        return torch.where(t != t, torch.full_like(o, (1 << 63) - 1), o)
    raise TypeError(t.dtype)


def _mix(x, c):
    """A 64-bit mixing function in wrapping int64 arithmetic."""
    x = x * c
    x = x ^ (x >> 31)
    x = x * -7046029254386353131
    return x ^ (x >> 29)


def fingerprint(x_i64):
    """Order-independent 2 x 64-bit fingerprint of a multiset of int64 values (wrapping sums)."""
    import torch

    return torch.stack([_mix(x_i64, -4417276706812531889).sum(), _mix(x_i64 ^ 0x5DEECE66D, 7640891576956012809).sum()])


def check_full(name, tile, result, result_lo, rank, nranks, dist):
    """Properties of a full-size result that together pin it: returns (ok, detail).  ``tile`` is
    this rank's input, ``result`` this rank's part of the output, ``result_lo`` its global start."""
    import torch

    c = CONFIGS[name]
    dev = tile.device
    multi = nranks > 1 and c["multi"] == "distributed"

    def allsum(v):
        if multi:
            dist.all_reduce(v)
        return v

    detail = {}
    if tile.ndim == 2:  # independent rows: every row sorted, every row a permutation of its input
        o_out = ordered_i64(result)
        sorted_ok = bool((o_out[:, 1:] >= o_out[:, :-1]).all())
        same = bool((_mix(tile.view(torch.int64), -4417276706812531889).sum(1) ==
                     _mix(result.view(torch.int64), -4417276706812531889).sum(1)).all())
        detail = {"rows_sorted": sorted_ok, "rows_same_multiset": same}
        return sorted_ok and same, detail

    n_in = torch.tensor([tile.numel()], dtype=torch.int64, device=dev)
    n_out = torch.tensor([result.numel()], dtype=torch.int64, device=dev)
    total_in, total_out = int(allsum(n_in)), int(allsum(n_out))
    detail["count"] = total_in == total_out
    o_in = ordered_i64(tile)
    if not c["argsort"]:
        o_out = ordered_i64(result)
        detail["sorted"] = bool((o_out[1:] >= o_out[:-1]).all()) if o_out.numel() > 1 else True
        bits = lambda t: t.view({1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]).to(torch.int64)
        detail["same_multiset"] = bool((allsum(fingerprint(bits(tile))) == allsum(fingerprint(bits(result)))).all())
        first = o_out[:1] if o_out.numel() else torch.zeros(1, dtype=torch.int64, device=dev)
        last = o_out[-1:] if o_out.numel() else torch.zeros(1, dtype=torch.int64, device=dev)
        edge = torch.cat([first, last, n_out * 0 + result.numel()])
    else:
        # the keys of the whole array, so that every index of my part can be looked up
        if multi:
            parts = [torch.empty_like(o_in) for _ in range(nranks)]
            dist.all_gather(parts, o_in)
            o_all = torch.cat(parts)
            del parts
        else:
            o_all = o_in
        idx = result
        in_range = bool(((idx >= 0) & (idx < total_in)).all()) if idx.numel() else True
        detail["indices_in_range"] = in_range
        if not in_range:
            return False, detail
        ko = o_all[idx]
        if idx.numel() > 1:
            detail["sorted_and_stable"] = bool(((ko[1:] > ko[:-1]) | ((ko[1:] == ko[:-1]) & (idx[1:] > idx[:-1]))).all())
        else:
            detail["sorted_and_stable"] = True
        mine = torch.arange(result_lo, result_lo + idx.numel(), dtype=torch.int64, device=dev)
        detail["permutation"] = bool((allsum(fingerprint(idx)) == allsum(fingerprint(mine))).all())
        first = torch.stack([ko[0], idx[0]]) if idx.numel() else torch.zeros(2, dtype=torch.int64, device=dev)
        last = torch.stack([ko[-1], idx[-1]]) if idx.numel() else torch.zeros(2, dtype=torch.int64, device=dev)
        edge = torch.cat([first, last, n_out * 0 + idx.numel()])
        del o_all, ko
    if multi:
        edges = [torch.empty_like(edge) for _ in range(nranks)]
        dist.all_gather(edges, edge)
        rows = [e.tolist() for e in edges]
        ok, prev = True, None
        start = 0
        for r, e in enumerate(rows):
            cnt = e[-1]
            if r == rank and start != result_lo:
                ok = False  # the reported global start must be the sum of the lower ranks' lengths
            start += cnt
            if cnt == 0:
                continue
            half = (len(e) - 1) // 2
            lo_key, hi_key = tuple(e[:half]), tuple(e[half:2 * half])
            if prev is not None and not (prev <= lo_key if not c["argsort"] else prev < lo_key):
                ok = False
            prev = hi_key
        detail["ranks_in_order"] = ok
    return all(detail.values()), detail


def check_small(name, rank, nranks, dist, num, log2=20):
    """The step at a reduced size against the CPU oracle, bit for bit (rank 0 compares)."""
    from oracle import thrust_task_sort

    c = CONFIGS[name]
    if name == "c3":
        log2 = 12 + 8  # 256 rows in all
    shard = host_input(name, log2, rank, nranks)
    multi = nranks > 1 and c["multi"] == "distributed"
    lo = rank * shard.shape[0] if multi else 0
    arr = num.array(shard, global_lo=lo)
    res = num.argsort(arr, kind="stable") if c["argsort"] else num.sort(arr)
    got = res.to_numpy()
    if not multi:
        seg = shard.shape[-1]
        want_k, want_i = thrust_task_sort(shard, seg, c["argsort"], ndim_is_1=shard.ndim == 1)
        want = want_i if c["argsort"] else want_k
        ok = np.array_equal(got.reshape(-1).view(np.uint8), want.reshape(-1).view(np.uint8))
        if nranks > 1:
            flags = [None] * nranks
            dist.all_gather_object(flags, bool(ok))
            ok = all(flags)
        return bool(ok)
    shards, parts, starts = [None] * nranks, [None] * nranks, [None] * nranks
    dist.all_gather_object(shards, shard)
    dist.all_gather_object(parts, got)
    dist.all_gather_object(starts, int(res.global_lo))
    ok = True
    if rank == 0:
        whole = np.concatenate(shards)
        want_k, want_i = thrust_task_sort(whole, whole.size, c["argsort"])
        want = want_i if c["argsort"] else want_k
        cat = np.concatenate(parts)
        ok = cat.shape == want.shape and np.array_equal(cat.view(np.uint8), want.view(np.uint8))
        ok = ok and starts == [int(x) for x in np.cumsum([0] + [len(p) for p in parts])[:-1]]
    flag = [bool(ok)]
    dist.broadcast_object_list(flag, src=0)
    return flag[0]


# ------------------------------------------------------------------------------------------------
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


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline
# ------------------------------------------------------------------------------------------------
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_reference_time(keys: np.ndarray, argsort: bool, steps: int, warmup: int, budget_s: float):
    """Times the reference's CPU arithmetic (OpenMP back-end, all host threads) on ``keys`` (whole
    rows for 2-D inputs).  Stops early when ``budget_s`` is spent.  Returns (Gkeys/s, seconds per
    step, threads, steps timed)."""
    from oracle import num_threads, set_num_threads, thrust_task_sort

    set_num_threads(host_threads())  # launchers export OMP_NUM_THREADS=1 to their children
    segment, one_d = (keys.shape[1], False) if keys.ndim == 2 else (keys.size, True)
    times, t_start = [], time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        thrust_task_sort(keys, segment, argsort, ndim_is_1=one_d, backend="omp")
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if times and time.perf_counter() - t_start + dt > budget_s:
            break
    if not times:
        times = [dt]
    per = float(np.mean(times))
    return keys.size / per / 1e9, per, num_threads(), len(times)


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    name = args.workload
    log2 = args.scale_log2 or CONFIGS[name]["log2"]
    keys = host_input(name, log2, 0, 1)
    gk, per, threads, done = cpu_reference_time(keys, CONFIGS[name]["argsort"], args.steps, args.warmup, args.reference_budget_s)
    line = {
        "impl": "reference", "metric": "sorted Gkeys/s", "value": gk, "unit": "Gkeys/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": CONFIGS[name]["dtype"], "data": "synthetic",
        "config": {"workload": config_label(name, log2, 1), "keys_per_step": int(keys.size),
                   "note": "one host runs the CPU arm whatever --gpus says: all keys of one GPU's shard per step"},
        "cpu_baseline": {"value": gk, "unit": "Gkeys/s", "cores": threads, "kind": "port",
                         "sample": f"thrust::omp::par stable sort of all {keys.size} keys of the workload, {done} steps"},
        "e2e": {"value": gk, "unit": "Gkeys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
KINDS = ["hist", "scan", "sweep", "fixup", "segsort", "unit", "dist", "merge", "xchg"]


class Bench:
    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import cupynumeric_b200 as num
        from cupynumeric_b200 import _lib

        self.args, self.torch, self.dist, self.num = args, torch, dist, num
        self.nranks = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.nranks > 1:
            dist.init_process_group("nccl", device_id=self.device)
        self.lib = _lib.lib()
        self.peak, self.peak_kind = measured_hbm_peak()
        self.flush_buf = None

    def barrier(self):
        if self.nranks > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.nranks > 1:
            t = self.torch.tensor([ms], device=self.device, dtype=self.torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def flush_l2(self):
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(256 << 20, dtype=self.torch.uint8, device=self.device)
        self.flush_buf.zero_()

    def kernel_breakdown(self, steps):
        out = {}
        for k, nm in enumerate(KINDS):
            tot, cnt = ctypes.c_double(0), ctypes.c_ulonglong(0)
            self.lib.b2s_profile_read(k, ctypes.byref(tot), ctypes.byref(cnt))
            if cnt.value:
                out[nm] = {"ms_per_step": tot.value / steps, "launches_per_step": cnt.value / steps,
                           "avg_launch_ms": tot.value / cnt.value}
                # launches that did work: a radix pass the routing skipped returns after a few
                # microseconds and must not dilute the average the roofline is taken from
                ms = (ctypes.c_float * cnt.value)()
                got = ctypes.c_size_t(0)
                self.lib.b2s_profile_durations(k, ms, cnt.value, ctypes.byref(got))
                work = [x for x in ms if x >= 0.2 * max(ms)]
                out[nm]["working_launches_per_step"] = len(work) / steps
                out[nm]["avg_working_launch_ms"] = sum(work) / len(work)
        return out

    def run_config(self, name, log2, headline=False):
        """Times one configuration; returns its record."""
        torch, num, args = self.torch, self.num, self.args
        c = CONFIGS[name]
        nranks, rank = self.nranks, self.rank
        multi = nranks > 1 and c["multi"] == "distributed"
        rec = {"workload": config_label(name, log2, nranks), "multi_gpu": c["multi"] if nranks > 1 else "one GPU"}

        small_ok = True if args.no_verify else check_small(name, rank, nranks, self.dist, num)
        tile = device_input(name, log2, rank, nranks, self.device)
        n_local = tile.numel()
        arr = num.array(tile, global_lo=rank * n_local if multi else 0)
        flush = tile.numel() * tile.element_size() <= L2_BYTES

        def step():
            return num.argsort(arr, kind="stable") if c["argsort"] else num.sort(arr)

        res = None
        for _ in range(args.warmup):
            res = step()
        self.barrier()
        full_ok, detail = (True, {}) if args.no_verify else check_full(name, tile, res.torch(), res.global_lo if multi else 0,
                                                                        rank, nranks, self.dist)
        del res
        sampler = ClockSampler(self.local_rank) if (headline and rank == 0) else None
        if sampler:
            sampler.start()
        launches0 = self.lib.b2s_launch_count(-1)
        self.barrier()
        ms = 0.0
        if flush:
            for _ in range(args.steps):
                self.flush_l2()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                ms += e0.elapsed_time(e1)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                step()
            e1.record()
            self.barrier()
            ms = e0.elapsed_time(e1)
        self.barrier()
        clocks = sampler.stop() if sampler else None
        launches = int(self.lib.b2s_launch_count(-1) - launches0)
        ms = self.max_over_ranks(ms) / args.steps
        # the same steps once more with one CUDA-event pair around every launch: where the time goes
        psteps = max(1, min(args.steps, 5))
        self.lib.b2s_profile_enable(1)
        for _ in range(psteps):
            if flush:
                self.flush_l2()
            step()
        torch.cuda.synchronize()
        kernels = self.kernel_breakdown(psteps)
        self.lib.b2s_profile_enable(0)
        self.barrier()
        kernels_rank = rank
        if nranks > 1:
            # the step ends when the slowest rank ends: report the rank with the most device time
            every = [None] * nranks
            self.dist.all_gather_object(every, kernels)
            busy = [sum(k["ms_per_step"] for k in ks.values()) for ks in every]
            kernels_rank = max(range(nranks), key=lambda r: busy[r])
            kernels = every[kernels_rank]

        total_keys = n_local * nranks
        gkeys = total_keys / (ms * 1e-3) / 1e9
        hbm_bytes = c["hbm_bytes"][1 if multi else 0]
        t_hbm = hbm_bytes * n_local / (self.peak * 1e9)
        t_nvl = c["nvlink_bytes"] * (nranks - 1) / nranks * n_local / (NVLINK_GBS * 1e9) if multi else 0.0
        floor = max(t_hbm, t_nvl)
        rec.update({
            "keys_per_gpu": n_local, "ms_per_step": ms, "gkeys_per_s": gkeys,
            "verified": {"ok": bool(small_ok and full_ok), "oracle_bit_exact_at_reduced_size": bool(small_ok),
                         "full_size_properties": detail},
            "roofline": {"bound": "hbm" if t_hbm >= t_nvl else "nvlink", "hbm_bytes_per_key": hbm_bytes,
                         "nvlink_bytes_per_key_per_direction": c["nvlink_bytes"] * (nranks - 1) / nranks if multi else 0.0,
                         "floor_ms": floor * 1e3, "frac": floor * 1e3 / ms, "hbm_peak_gbs": self.peak,
                         "peak_source": f"of {self.peak_kind}", "nvlink_gbs": NVLINK_GBS,
                         "frac_of_8TBs": (max(hbm_bytes * n_local / 8e12, t_nvl)) * 1e3 / ms},
            "kernels": kernels, "kernels_of_rank": kernels_rank, "gpu_launches_per_step": launches / args.steps,
            "l2": "input smaller than L2: a 256 MB buffer is written between timed steps" if flush
                  else "input larger than the 126 MB L2, no flush needed",
        })
        if multi:
            rec["exchange"] = os.environ.get("B2S_DIST_P2P", "1") != "0" and "peer" or "nccl"
        dom = {"onesweep_kernel": "sweep", "segmerge_kernel": "segsort"}[c["kernel"]]
        if dom in kernels:
            avg_ms = kernels[dom]["avg_working_launch_ms"]
            achieved = c["sweep_bytes"] * n_local / (avg_ms * 1e-3) / 1e9
            traffic = ncu_traffic_bytes_per_key().get(name)
            rec["dominant_kernel"] = {"bound": "hbm", "kernel": c["kernel"], "achieved": achieved, "peak": self.peak,
                                      "unit": "GB/s", "frac": achieved / self.peak, "peak_source": f"of {self.peak_kind}",
                                      "avg_launch_ms": avg_ms, "launches_per_step": kernels[dom]["working_launches_per_step"],
                                      "launches": "passes that moved data (a pass the routing skipped returns at once and is left out)",
                                      "algorithmic_bytes_per_launch": c["sweep_bytes"] * n_local,
                                      "traffic": traffic * n_local if traffic else None}
        if nranks == 1 and not args.no_cub:
            rec["cub_baseline"] = self.cub_baseline(tile, c["argsort"], flush)
        rec["_clocks"], rec["_launches"], rec["_tile"] = clocks, launches, tile
        return rec

    def cub_baseline(self, tile, argsort, flush):
        """The CCCL library sort the reference's GPU variant calls, on the same tile, under the same
        cache protocol as the timed steps (L2 flushed before every step when the input fits L2)."""
        try:
            from oracle import cub_baseline as cb
            if not cb.available():
                return {"unavailable": "oracle/libcub_baseline.so is not built"}
            ms, _ = cb.time_sort(tile, argsort, steps=max(1, min(self.args.steps, 5)), warmup=2,
                                 between=self.flush_l2 if flush else None)
            ours = self.direct_call_ms(tile, argsort, flush, steps=max(1, min(self.args.steps, 5)), warmup=2)
            return {"ms_per_step": ms, "gkeys_per_s": tile.numel() / (ms * 1e-3) / 1e9,
                    "ours_same_protocol_ms": ours,
                    "l2": "flushed before every step" if flush else "input larger than L2",
                    "timed": "direct C call with preallocated buffers (no allocation, no Python dispatch inside the interval)",
                    "what": "cub::DeviceRadixSort / DeviceSegmentedRadixSort (+ index fill for argsort), CCCL of the CUDA toolkit"}
        except Exception as e:  # the baseline is optional evidence, not part of the product
            return {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    def direct_call_ms(self, tile, argsort, flush, steps, warmup):
        """b2s_local_sort timed the way the library baseline is: the C entry point itself, output and
        workspace allocated beforehand."""
        torch, lib = self.torch, self.lib
        from cupynumeric_b200 import _lib
        from cupynumeric_b200._thunk.deferred import to_numpy_dtype
        code = _lib.DTYPE_CODE[to_numpy_dtype(tile.dtype)]
        volume, segment = tile.numel(), tile.shape[-1]
        need = ctypes.c_size_t(0)
        _lib.check(lib.b2s_workspace_bytes(code, volume, segment, int(argsort), ctypes.byref(need)), "b2s_workspace_bytes")
        ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device=tile.device)
        out = torch.empty(tile.shape, dtype=torch.int64 if argsort else tile.dtype, device=tile.device)
        stream = torch.cuda.current_stream().cuda_stream

        def call():
            _lib.check(lib.b2s_local_sort(code, tile.data_ptr(), None if argsort else out.data_ptr(),
                                          out.data_ptr() if argsort else None, volume, segment, 0, int(tile.ndim == 1), 1,
                                          ws.data_ptr(), ws.numel(), stream), "b2s_local_sort")

        for _ in range(warmup):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if flush:
            ms = 0.0
            for _ in range(steps):
                self.flush_l2()
                e0.record()
                call()
                e1.record()
                torch.cuda.synchronize()
                ms += e0.elapsed_time(e1)
            return ms / steps
        e0.record()
        for _ in range(steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def run_e2e(self, name, log2, tile):
        """The same step through the public API with pinned host buffers on both sides."""
        torch, num, args = self.torch, self.num, self.args
        c = CONFIGS[name]
        nranks, rank = self.nranks, self.rank
        multi = nranks > 1 and c["multi"] == "distributed"
        n_local = tile.numel()
        sview = {torch.uint64: torch.int64, torch.uint32: torch.int32, torch.uint16: torch.int16}.get(tile.dtype, tile.dtype)
        pinned_in = torch.empty(tile.shape, dtype=sview, pin_memory=True)
        pinned_in.copy_(tile.view(sview))
        np_dtype = {"i32": np.int32, "f32": np.float32, "f64": np.float64, "i64": np.int64, "u64": np.uint64}[c["dtype"]]
        host_in = pinned_in.numpy().view(np_dtype)
        res_dtype = np.int64 if c["argsort"] else np_dtype
        cap = int(n_local * 1.5) + 1024 if multi else n_local
        pinned_out = torch.empty(cap if tile.ndim == 1 else tile.shape, dtype=torch.int64 if c["argsort"] else sview, pin_memory=True)
        host_out = pinned_out.numpy().view(res_dtype)
        got = [n_local]

        def e2e_step():
            a = num.array(host_in, global_lo=rank * n_local if multi else 0)
            r = num.argsort(a, kind="stable") if c["argsort"] else num.sort(a)
            got[0] = r.size
            r.to_numpy(out=host_out[: r.size] if tile.ndim == 1 else host_out)

        steps = max(1, min(args.steps, args.e2e_steps))
        e2e_step()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            e2e_step()
        e1.record()
        self.barrier()
        ms = self.max_over_ranks(e0.elapsed_time(e1)) / steps
        h2d, d2h = int(host_in.nbytes), int(got[0]) * np.dtype(res_dtype).itemsize
        return {"value": n_local * nranks / (ms * 1e-3) / 1e9, "unit": "Gkeys/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": steps, "ms_per_step": ms,
                "host_copy_gbs_per_rank": (h2d + d2h) / (ms * 1e-3) / 1e9,
                "note": "per rank: pinned host -> device copy of the keys, the sort, device -> pinned host copy of the result; "
                        "all ranks of one box share the host's memory and PCIe root"}


def run_ours(args):
    b = Bench(args)
    torch, dist = b.torch, b.dist
    name = args.workload
    log2 = args.scale_log2 or CONFIGS[name]["log2"]
    head = b.run_config(name, log2, headline=True)
    tile = head.pop("_tile")
    clocks, launches = head.pop("_clocks"), head.pop("_launches")
    e2e = b.run_e2e(name, log2, tile)
    n_local = tile.numel()
    cpu = None
    if b.nranks == 1 and b.rank == 0 and not args.no_cpu_baseline:
        sample = min(1 << args.cpu_sample_log2, n_local)
        host = tile.reshape(-1)[:sample].cpu()
        host = host.numpy() if host.dtype != torch.uint64 else host.view(torch.int64).numpy().view(np.uint64)
        if tile.ndim == 2:
            host = host.reshape(-1, tile.shape[1])
        gk, per, threads, _ = cpu_reference_time(host, CONFIGS[name]["argsort"], 1, 0, 60.0)
        cpu = {"value": gk, "unit": "Gkeys/s", "cores": threads, "kind": "port",
               "sample": f"thrust::omp::par stable sort of the first {host.size} keys of the workload, 1 step ({per:.2f} s)"}
    del tile
    torch.cuda.empty_cache()

    configs = {}
    if not args.no_configs:
        for other in [x for x in args.configs.split(",") if x and x != name]:
            rec = b.run_config(other, args.scale_log2 or CONFIGS[other]["log2"])
            for k in ("_tile", "_clocks", "_launches"):
                rec.pop(k, None)
            configs[other] = rec
            torch.cuda.empty_cache()

    all_ok = head["verified"]["ok"] and all(r["verified"]["ok"] for r in configs.values())
    if b.rank == 0:
        dom = head.get("dominant_kernel")
        line = {
            "metric": "sorted Gkeys/s", "value": head["gkeys_per_s"], "unit": "Gkeys/s", "n_gpus": b.nranks,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": CONFIGS[name]["dtype"], "data": "synthetic",
            "config": {"workload": head["workload"], "keys_per_gpu": n_local, "l2": head["l2"],
                       "multi_gpu": head["multi_gpu"], "exchange": head.get("exchange")},
            "verified": head["verified"],
            "roofline": dom,
            "job_roofline": head["roofline"],
            "kernels": head["kernels"],
            "cub_baseline": head.get("cub_baseline"),
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
            "configs": configs,
        }
        print(json.dumps(line))
    if b.nranks > 1:
        dist.barrier()
        try:
            from cupynumeric_b200._dist import destroy_comm
            destroy_comm()
        except Exception:
            pass
        dist.destroy_process_group()
    if not all_ok:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--scale-log2", type=int, default=None, help="log2 of the key count per GPU; default: the configuration's size")
    ap.add_argument("--configs", default="c1,c3,c4,c5", help="configurations reported beside the headline")
    ap.add_argument("--cpu-sample-log2", type=int, default=28, help="log2 of the keys the CPU baseline sorts (the first keys of the workload; 28 = all of the headline workload, about 8 s on 16 threads)")
    ap.add_argument("--reference-budget-s", type=float, default=150.0, help="the reference arm stops starting new steps after this")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true")
    ap.add_argument("--no-cub", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--lean", action="store_true", help="headline only: no other configurations, checks or baselines (profiling runs)")
    args = ap.parse_args()
    if args.lean:
        args.no_cpu_baseline = args.no_configs = args.no_cub = args.no_verify = True
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
