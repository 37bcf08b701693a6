#!/usr/bin/env python
"""Benchmark of the encrypted-aggregation hot path on B200.

  python bench.py --gpus N --steps K --warmup W [--workload ntt|hmult|krum] [--impl reference]

One "step" is one pass of the workload over one batch of seeded synthetic input.  The
line printed by rank 0 follows the driver's contract: `value` is device-timed throughput
with inputs resident in HBM, `e2e` the same metric through the C ABI with host buffers
(host<->device copies inside the timed region), `roofline` the dominant kernel against the
measured HBM peak, `cpu_baseline` the CPU checker timed on a bounded sample of the same
workload on this box's host cores.

Workloads (bench_workloads.py):
  krum   encrypted-Krum distance round (lancelot_b200/krum.py), the default; its line also carries short runs of
         the other two as the sub-records "hmult" and "ntt"
  hmult  multiply + relinearize + rescale, N = 2^16, L = 24, dnum = 3 (8 special primes)
  ntt    batched NTT + INTT, N = 2^16, 24 fifty-bit primes, 128 polynomials per step
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs.  Uses NVML in-process
    (a query costs microseconds); falls back to the nvidia-smi command line when the module is missing."""

    def __init__(self, index=0, period=0.25):
        self.index, self.period = index, period
        self.sm, self.sm_max, self.reasons = [], None, set()
        self._stop = threading.Event()
        self._t = None

    def _run_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
        names = {"hw_slowdown": getattr(pynvml, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(pynvml, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
            try:
                mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
            except Exception:
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            for nm, bit in names.items():
                if mask & bit:
                    self.reasons.add(nm)
            self._stop.wait(self.period)

    def _run_smi(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                r = [x.strip() for x in out.split(",")]
                if r and r[0].isdigit():
                    self.sm.append(int(r[0]))
                    self.sm_max = int(r[1])
                    for i, nm in enumerate(names):
                        if len(r) > 2 + i and r[2 + i].lower().startswith("active"):
                            self.reasons.add(nm)
            except Exception:
                pass
            self._stop.wait(1.0)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------

def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, wl):
    """CPU arm: the checker under oracle/ (a restatement of the reference's algorithm; the reference's own CPU
    path is OpenFHE, which cannot be installed here) with every host core, on a bounded sample per step.  Rank 0
    alone runs it.  Neither torch nor the CUDA library is imported on this path."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    vals, walls = [], []
    sample, used = "", threads
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        v, sample, used = wl.cpu_sample(threads)
        if i >= args.warmup:
            vals.append(v)
            walls.append(time.perf_counter() - t0)
    value = sum(vals) / len(vals)
    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            # a step of this arm is one bounded sample; ms_per_step is its wall time, value the whole workload it stands for
            "ms_per_step": 1e3 * sum(walls) / len(walls), "higher_is_better": wl.higher_is_better, "scaling": getattr(wl, "scaling", "weak"),
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(), "impl": "reference",
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": used, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def kernel_table(report, peak):
    """per-kernel rows of the diagnostic timer, largest share first"""
    total = sum(r["ms"] for r in report.values()) or 1.0
    rows = []
    for name, r in sorted(report.items(), key=lambda kv: -kv[1]["ms"]):
        row = {"kernel": name, "launches": r["launches"], "ms": round(r["ms"], 3), "share": round(r["ms"] / total, 4)}
        if r["bytes"] > 0 and r["ms"] > 0:
            gbs = r["bytes"] / (r["ms"] * 1e-3) / 1e9
            row.update(algorithmic_bytes=r["bytes"], gbs=round(gbs, 1), frac_of_hbm=round(gbs / peak, 4))
        rows.append(row)
    return rows


def roofline_from(rows, peak, peak_kind, traffic_table):
    """the roofline entry of the kernel with the largest share of the step among those with stated algorithmic bytes"""
    for row in rows:
        if "gbs" not in row:
            continue
        per_launch = row["algorithmic_bytes"] / row["launches"]
        traffic = None
        cap = traffic_table.get(row["kernel"])
        if cap:
            traffic = int(per_launch * cap["dram_bytes"] / cap["algorithmic_bytes"])
        return {"bound": "hbm", "achieved": row["gbs"], "peak": peak, "unit": "GB/s", "frac": row["gbs"] / peak, "traffic": traffic,
                "kernel": row["kernel"], "peak_kind": "of " + peak_kind, "share_of_step": row["share"], "launches_per_step": row["launches"],
                "algorithmic_bytes_per_launch": per_launch, "avg_launch_ms": row["ms"] / row["launches"],
                "how": "CUDA events recorded in front of every launch during one instrumented repeat of the timed step"}
    return None


def short_run(cls, batch, timed, steps, peak, device, threads, with_cpu):
    """a short run of another headline workload on this GPU: metric value, its dominant kernel against the HBM peak,
    and (on one GPU) its CPU baseline"""
    from lancelot_b200 import cabi
    wl = cls(batch=batch)
    wl.setup_gpu(device)
    for _ in range(3):
        wl.step_gpu()
    ms, _ = timed(wl.step_gpu, steps)
    ok = wl.check_gpu()
    cabi.kernel_timing(True)
    wl.step_gpu()
    rows = kernel_table(cabi.kernel_report(), peak)
    cabi.kernel_timing(False)
    value = wl.units_per_step() / (ms * 1e-3 / steps)
    out = {"metric": wl.metric, "value": value, "unit": wl.unit, "config": wl.config()["workload"], "steps": steps, "parity_check": ok,
           "algorithmic_gbs": wl.algorithmic_bytes_per_step() / (ms * 1e-3 / steps) / 1e9,
           "frac_of_hbm": wl.algorithmic_bytes_per_step() / (ms * 1e-3 / steps) / 1e9 / peak, "kernels": rows[:4]}
    if hasattr(wl, "butterfly_roofs"):
        out["arithmetic_roof_gbs"] = wl.butterfly_roofs()
    if with_cpu:
        v, sample, used = wl.cpu_sample(threads)
        out["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": used, "kind": "port", "sample": sample}
    return out


def run_gpu(args, wl, default_line):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from lancelot_b200 import cabi
    import bench_workloads
    wl.setup_gpu(local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        stream = torch.cuda.current_stream()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        extra = None
        for _ in range(steps):
            extra = fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, extra

    warm = max(args.warmup, 3)
    for _ in range(warm):
        wl.step_gpu()
    with ClockSampler(local) as clocks:
        ms, _ = timed(wl.step_gpu, args.steps)
    ok = wl.check_gpu()
    launches = wl.launches_per_step
    if hasattr(wl, "profile_phases"):  # one extra, untimed pass with per-phase synchronisation for the breakdown
        wl.profile_phases = True
        wl.step_gpu()
        wl.profile_phases = False
    # one instrumented repeat of the same step: an event in front of every launch gives per-kernel device times
    peak, peak_kind = measured_peaks()
    barrier()
    cabi.kernel_timing(True)
    wl.step_gpu()
    rows = kernel_table(cabi.kernel_report(), peak)
    cabi.kernel_timing(False)
    for _ in range(warm):
        wl.step_e2e()
    ms_e2e, io = timed(wl.step_e2e, args.steps)
    pair = wl.time_pair_tile(timed) if hasattr(wl, "time_pair_tile") and world == 1 else None
    roofs = wl.butterfly_roofs() if hasattr(wl, "butterfly_roofs") and world == 1 else None

    line = None
    if rank == 0:
        units = wl.units_per_step() * (world if getattr(wl, "scaling", "weak") == "weak" else 1)
        sec = ms * 1e-3 / args.steps
        sec_e2e = ms_e2e * 1e-3 / args.steps
        if wl.higher_is_better:
            value, e2e_value = units / sec, units / sec_e2e
        else:
            value, e2e_value = sec, sec_e2e
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms / args.steps, "higher_is_better": wl.higher_is_better, "scaling": getattr(wl, "scaling", "weak"),
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
                "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": io[0], "d2h_bytes_per_step": io[1]},
                "gpu_launches": args.steps * launches,
                "roofline": roofline_from(rows, peak, peak_kind, bench_workloads.NCU_TRAFFIC),
                "kernels": rows[:8], "cpu_baseline": None, "clocks": clocks.summary(), "parity_check": ok}
        if roofs:
            line["arithmetic_roof_gbs"] = roofs
        if pair:
            pair["peak"] = peak
            pair["frac"] = pair["achieved"] / peak
            cap = bench_workloads.NCU_TRAFFIC.get("krum_tile_kernel")
            pair["traffic"] = int(pair["bytes_per_launch"] * cap["dram_bytes"] / cap["algorithmic_bytes"]) if cap else None
            line["roofline_pair_kernel"] = pair
        if getattr(wl, "breakdown", None):
            line["breakdown"] = wl.breakdown
        if hasattr(wl, "rel_err"):
            line["max_rel_err_vs_float64_plaintext"] = wl.rel_err
        if hasattr(wl, "abs_err"):
            line["max_abs_err_vs_float64_plaintext"] = wl.abs_err
            line["first_chunk_bit_exact_vs_oracle"] = wl.bit_exact
    # the other two headline metrics, from short runs of their workloads on this same GPU (default line, one GPU)
    if default_line and world == 1:
        del wl
        torch.cuda.empty_cache()
        threads = host_threads()
        line["hmult"] = short_run(bench_workloads.HmultWorkload, 8, timed, 3, peak, local, threads, True)
        torch.cuda.empty_cache()
        line["ntt"] = short_run(bench_workloads.NttWorkload, 128, timed, 3, peak, local, threads, True)
        wl = bench_workloads.WORKLOADS[args.workload_name]() if args.batch is None else bench_workloads.WORKLOADS[args.workload_name](batch=args.batch)
    if rank == 0:
        if world == 1:
            v, sample, used = wl.cpu_sample(host_threads())
            line["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": used, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="krum (default), hmult or ntt")
    ap.add_argument("--batch", type=int, default=None)
    args = ap.parse_args()
    import bench_workloads
    name = args.workload or os.environ.get("LB_BENCH_WORKLOAD") or "krum"
    args.workload_name = name
    cls = bench_workloads.WORKLOADS[name]
    wl = cls(batch=args.batch) if args.batch else cls()
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        # the default line (no --workload) also carries the other two headline metrics as sub-records
        run_gpu(args, wl, default_line=args.workload is None and name == "krum" and args.batch is None)


if __name__ == "__main__":
    main()
