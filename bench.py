#!/usr/bin/env python
"""Benchmark of the encrypted-aggregation hot path on B200.

  python bench.py --gpus N --steps K --warmup W [--workload ntt|hmult|krum] [--impl reference]

One "step" is one pass of the workload over one batch of seeded synthetic input.  The
line printed by rank 0 follows the driver's contract: `value` is device-timed throughput
with inputs resident in HBM, `e2e` the same metric through the C ABI with host buffers
(host<->device copies inside the timed region), `roofline` the dominant kernel against the
measured HBM peak, `cpu_baseline` the CPU checker timed on a bounded sample of the same
workload on this box's host cores.

Workloads (BASELINE.json configs):
  ntt    batched NTT + INTT, N = 2^16, 24 fifty-bit primes, 128 polynomials per step
  hmult  multiply + relinearize + rescale, N = 2^16, L = 24, dnum = 3 (8 special primes)
  krum   encrypted-Krum distance round (see lancelot_b200/krum.py)
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
# workloads
# ------------------------------------------------------------------------------------------

class NttWorkload:
    """configs[1]: batched NTT/INTT sweep at N = 2^16 over 24 fifty-bit primes."""
    name = "ntt"
    metric = "ntt_hbm_gbs"
    unit = "GB/s"
    higher_is_better = True
    dtype = "u64"

    def __init__(self, batch=128, logn=16, limbs=24):
        self.batch, self.logn, self.limbs = batch, logn, limbs
        self.N = 1 << logn

    def config(self):
        return {"workload": "C2 batched NTT+INTT, N=2^16, 24 x 50-bit primes, %d polynomials per step" % self.batch,
                "l2": "inputs (%.1f GiB per step) exceed the 126 MB L2" % (self.batch * self.limbs * self.N * 8 / 2 ** 30)}

    def moduli(self):
        from lancelot_b200 import cabi
        return cabi.coeff_modulus_create(self.N, [50] * self.limbs)

    def algorithmic_bytes_per_step(self):
        # 16 bytes per coefficient per transform, forward + inverse
        return 2 * 16 * self.N * self.limbs * self.batch

    def setup_gpu(self, device):
        import torch
        from lancelot_b200 import cabi
        self.ctx = cabi.Context(self.logn, self.moduli(), 0, device=device)
        g = torch.Generator(device="cuda:%d" % device)
        g.manual_seed(1234)
        # residues uniform below 2^49 < q_i for every 50-bit prime
        self.data = torch.randint(0, 1 << 49, (self.batch, self.limbs, self.N), dtype=torch.int64, device="cuda:%d" % device, generator=g)
        self.orig = self.data.clone()
        self.host = torch.empty_like(self.data, device="cpu").pin_memory()
        self.host.copy_(self.data)
        self.host_out = torch.empty_like(self.host).pin_memory()
        self.launches_per_step = 2

    def step_gpu(self):
        self.ctx.ntt_forward(self.data, self.batch, self.limbs, 0)
        self.ctx.ntt_inverse(self.data, self.batch, self.limbs, 0)

    def step_e2e(self):
        self.data.copy_(self.host, non_blocking=True)
        self.step_gpu()
        self.host_out.copy_(self.data, non_blocking=True)
        return self.host.numel() * 8, self.host_out.numel() * 8

    def check_gpu(self):
        import torch
        return bool(torch.equal(self.data, self.orig))

    def units_per_step(self):
        return self.algorithmic_bytes_per_step() / 1e9  # GB

    def roofline_kernel_bytes(self):
        # one launch transforms the whole batch once
        return 16 * self.N * self.limbs * self.batch

    @property
    def ncu_traffic_bytes(self):
        # dram read + write of one captured 16-polynomial launch was 404.1 MB for 402.7 MB of
        # algorithmic bytes; traffic grows with the limb count, so scale that ratio
        return int(self.roofline_kernel_bytes() * 404.1 / 402.7)

    def int_roof(self):
        """arithmetic ceiling of the transform: the register-only butterfly rate converted to transform traffic"""
        per_limb = (self.N // 2) * self.logn
        to_gbs = lambda rate: rate / per_limb * 16 * self.N / 1e9
        rate = self.ctx.butterfly_rate()  # the variant this workload's primes take
        names = ["int_strict", "int_lazy", "fp64_strict", "fp64_lazy"]
        return {"butterflies_per_s": rate, "equivalent_transform_gbs": to_gbs(rate),
                "variants_gbs": {n: to_gbs(self.ctx.butterfly_rate(i)) for i, n in enumerate(names)},
                "note": "min(HBM, arithmetic) roof for the NTT is equivalent_transform_gbs"}

    def cpu_sample(self, threads):
        """forward + inverse of one polynomial (24 limbs) on the CPU checker"""
        import numpy as np
        from oracle import binding
        o = binding.Oracle(self.logn, self.moduli(), 0)
        rng = np.random.default_rng(0)
        data = rng.integers(0, 1 << 49, (self.limbs, self.N), dtype=np.uint64)
        reps = 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < 4.0 or reps < 2:
            f = o.ntt_rows(data, 1, self.limbs, 0)
            b = o.ntt_rows(f, 1, self.limbs, 0, inverse=True)
            reps += 1
        dt = time.perf_counter() - t0
        assert np.array_equal(b, data)
        gb = reps * 2 * 16 * self.N * self.limbs / 1e9
        return gb / dt, "%d x (NTT+INTT of 1 polynomial, 24 limbs)" % reps


WORKLOADS = {"ntt": NttWorkload}


def load_workloads():
    try:
        from lancelot_b200 import bench_workloads
        WORKLOADS.update(bench_workloads.WORKLOADS)
    except ImportError:
        pass


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------

def run_reference(args, wl):
    """CPU arm: the checker (a port of the reference's algorithm; the reference's own CPU path
    is OpenFHE, which is not installable here) on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    vals = []
    sample = ""
    for i in range(args.warmup + args.steps):
        v, sample = wl.cpu_sample(threads)
        if i >= args.warmup:
            vals.append(v)
    if wl.higher_is_better:
        value = sum(vals) / len(vals)
    else:
        value = sum(vals) / len(vals)
    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": None, "higher_is_better": wl.higher_is_better, "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic", "config": wl.config(), "impl": "reference",
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_gpu(args, wl):
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

    for _ in range(max(args.warmup, 3)):
        wl.step_gpu()
    with ClockSampler(local) as clocks:
        ms, _ = timed(wl.step_gpu, args.steps)
    ok = wl.check_gpu()
    if hasattr(wl, "profile_phases"):  # one extra, untimed pass with per-phase synchronisation for the breakdown
        wl.profile_phases = True
        wl.step_gpu()
        wl.profile_phases = False
    for _ in range(max(args.warmup, 3)):
        wl.step_e2e()
    ms_e2e, io = timed(wl.step_e2e, args.steps)

    # dominant kernel alone, for the roofline entry
    peak, peak_kind = measured_peaks()
    kms, kname = wl.time_dominant_kernel(timed) if hasattr(wl, "time_dominant_kernel") else (ms / (args.steps * wl.launches_per_step), "step average")
    achieved = wl.roofline_kernel_bytes() / (kms * 1e-3) / 1e9

    if rank == 0:
        units = wl.units_per_step() * world
        sec = ms * 1e-3 / args.steps
        sec_e2e = ms_e2e * 1e-3 / args.steps
        if wl.higher_is_better:
            value, e2e_value = units / sec, units / sec_e2e
        else:
            value, e2e_value = sec, sec_e2e
        threads = host_threads()
        os.environ.setdefault("OMP_NUM_THREADS", str(threads))
        cpu = None
        if world == 1:
            v, sample = wl.cpu_sample(threads)
            cpu = {"value": v, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample}
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms / args.steps, "higher_is_better": wl.higher_is_better, "scaling": getattr(wl, "scaling", "weak"),
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
                "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": io[0], "d2h_bytes_per_step": io[1]},
                "gpu_launches": args.steps * wl.launches_per_step,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": getattr(wl, "ncu_traffic_bytes", None), "kernel": kname, "peak_kind": "of " + peak_kind},
                "cpu_baseline": cpu, "clocks": clocks.summary(), "parity_check": ok}
        if hasattr(wl, "int_roof"):
            line["int_roof"] = wl.int_roof()
        if hasattr(wl, "int_roof_gbs"):
            line["roofline"]["arithmetic_roof_gbs"] = wl.int_roof_gbs
            line["roofline"]["frac_of_arithmetic_roof"] = achieved / wl.int_roof_gbs
        if hasattr(wl, "pair_kernel"):
            wl.pair_kernel["peak"] = peak
            wl.pair_kernel["frac"] = wl.pair_kernel["achieved"] / peak
            line["roofline_pair_kernel"] = wl.pair_kernel
        if getattr(wl, "breakdown", None):
            line["breakdown"] = wl.breakdown
        if hasattr(wl, "rel_err"):
            line["max_rel_err_vs_float64_plaintext"] = wl.rel_err
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--batch", type=int, default=None)
    args = ap.parse_args()
    load_workloads()
    name = args.workload or os.environ.get("LB_BENCH_WORKLOAD") or ("krum" if "krum" in WORKLOADS else "ntt")
    cls = WORKLOADS[name]
    wl = cls(batch=args.batch) if args.batch else cls()
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_gpu(args, wl)


if __name__ == "__main__":
    main()
