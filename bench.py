#!/usr/bin/env python
"""Benchmark of the matmult hot path on B200.  Workload: BASELINE.json's configs[1] (the second of its five
configurations, the one the metric is quoted on): batched Float16 matmult, A[64,2048,2048] . B[64,2048,2048] with B
passed as a transposed view, fp32 accumulation.  One step = one pass of the whole batch.  With N GPUs every rank owns
its own 64-item slice of a 64*N-item batch (weak scaling, no collective on the data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --configs [--cpu] [--only c1,c3i8,...]      # one JSON line per other configuration

Prints ONE JSON line (rank 0).  `value` is device-resident throughput, `e2e` goes through the C-ABI
host-buffer entry point with pinned host buffers (copies inside the timed region), `roofline` compares the
GEMM kernel with the measured tensor-core peak, `cpu_baseline` is the CPU oracle timed on this box's cores.
Secondary blocks on the same line: `sustained` (the same launch repeated for at least two seconds, against the
sustained cuBLAS figure), `target_8192` (the 8192^3 Float16 / BFloat16 target shape) and, with more than one GPU,
`mlp_n_sharded` (configs[3]: the BFloat16 MLP step with every GEMM split over its output columns, strong scaling,
checked against the unsharded step).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, M, K, N = 64, 2048, 2048, 2048
FLOPS_PER_ITEM = 2.0 * M * K * N
WORKLOAD = ("batched matmult Float16 A[64,2048,2048] x B[64,2048,2048]^T-view, fp32 accumulate "
            "(BASELINE.json configs[1], the second of the five configurations)")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM kernel: not measured by this run (a profiler
# cannot run inside a timed benchmark) but taken from a stored ncu capture of the same kernel on 8 items (134.3 MB
# read + 43.0 MB written), scaled to the items of the run: the traffic grows in proportion to the items.
NCU_DRAM_TRAFFIC_BYTES_PER_ITEM = (134.298880e6 + 43.018240e6) / 8


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops_burst": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0)),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def cpu_kernel():
    """(function(a, b_stored) -> C, kind, threads): the reference's own matmult kernel compiled from its sources
    (oracle/_ref, built by oracle/build_ref.py where the reference tree is present and carried along otherwise) when
    it is available, else the restatement of it in oracle/oracle.cpp.  Both use the host threads the reference would
    (its cap is 21)."""
    from oracle import oracle
    oracle.build()
    threads = oracle.default_threads()
    try:
        if oracle.reference_lib() is not None:
            return (lambda a, bs: oracle.reference_matmult(a, bs, False, True)), "reference", threads
    except OSError:
        pass
    return (lambda a, bs: oracle.matmult(a, bs, False, True, threads=threads)), "port", threads


def run_reference(args, rank, world):
    """The reference's own CPU implementation of this path on the box's host cores: its matmult kernel compiled from
    its own sources (oracle/_ref; the un-vendored simde / oneTBB / half headers are replaced by stand-ins, see
    oracle/build_ref.py), or the restatement where that library is missing.  One step = `sample` items of the batch."""
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle
    kernel, kind, threads = cpu_kernel()
    sample = 2
    rng = np.random.default_rng(3)
    a = (rng.standard_normal((sample, M, K)) * 0.1).astype(np.float16)
    bs = (rng.standard_normal((sample, N, K)) * 0.1).astype(np.float16)
    for _ in range(max(1, min(args.warmup, 2))):
        kernel(a[:1], bs[:1])
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        kernel(a, bs)
    dt = (time.perf_counter() - t0) / steps
    tflops = sample * FLOPS_PER_ITEM / dt / 1e12
    line = {
        "impl": "reference", "metric": "matmult TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "%d of %d batch items per step" % (sample, BATCH)},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": "%d of %d batch items (2048^3 each) per step, %d threads of %d hardware threads"
                                   % (sample, BATCH, threads, oracle.hardware_threads())},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline():
    import numpy as np
    kernel, kind, threads = cpu_kernel()
    rng = np.random.default_rng(3)
    a = (rng.standard_normal((1, M, K)) * 0.1).astype(np.float16)
    bs = (rng.standard_normal((1, N, K)) * 0.1).astype(np.float16)
    kernel(a, bs)                                                  # warm-up (page faults, thread start)
    t0 = time.perf_counter()
    kernel(a, bs)
    one = time.perf_counter() - t0
    items = int(max(1, min(64, 10.0 / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(items):
        kernel(a, bs)
    dt = time.perf_counter() - t0
    return {"value": items * FLOPS_PER_ITEM / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": "%d of %d batch items (2048^3 each), %.1f s of CPU time on %d threads"
                      % (items, BATCH, dt, threads)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--items", type=int, default=BATCH,
                    help="batch items per GPU (default: the full 64); smaller values are for profiler captures only")
    ap.add_argument("--no-extras", action="store_true", help="skip the sustained / target_8192 / mlp_n_sharded blocks")
    ap.add_argument("--configs", action="store_true", help="time the other configurations instead (one JSON line each)")
    ap.add_argument("--cpu", action="store_true", help="with --configs: also time the CPU oracle on a bounded sample of each row")
    ap.add_argument("--only", default="", help="with --configs: comma-separated row names")
    args = ap.parse_args()
    if args.configs:
        from neurotensor_b200 import bench_configs
        cpu_oracle = None
        if args.cpu:                                  # the oracle is test infrastructure: it is handed in from here
            from oracle import oracle as cpu_oracle
            cpu_oracle.build()
        return bench_configs.run(steps=min(args.steps, 20), only=args.only, oracle=cpu_oracle)
    rank, world, local_rank = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return 0
    warmup = max(3, args.warmup)

    import torch
    from neurotensor_b200 import _lib, api, partition
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # this rank's slice of the global batch (weak scaling: 64 items per rank)
    start, count = partition.shard_range(args.items * world, world, rank)
    gen = torch.Generator(device="cuda").manual_seed(3 + rank)
    a = (torch.randn((count, M, K), generator=gen, device="cuda") * 0.1).half()
    bs = (torch.randn((count, N, K), generator=gen, device="cuda") * 0.1).half()
    b = bs.transpose(-1, -2)                       # non-contiguous view: strides, no copy
    c = torch.empty((count, M, N), dtype=torch.float16, device="cuda")

    def step():
        api.gemm(a, b, c)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    _lib.check(_lib.lib().ntb200_check_device_status(None))
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    clocks = sampler.finish()
    launches = _lib.launch_count() - launches0
    ms = ev0.elapsed_time(ev1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    total_items = args.items * world
    value = total_items * FLOPS_PER_ITEM / (ms_per_step * 1e-3) / 1e12
    route = _lib.last_route()

    # ---- end to end: HOST buffers through ntb200_matmult_host (H2D of A and B, D2H of C every step)
    e2e = None
    if not args.no_e2e:
        ha = torch.empty((count, M, K), dtype=torch.float16).pin_memory()
        hb = torch.empty((count, N, K), dtype=torch.float16).pin_memory()
        hc = torch.empty((count, M, N), dtype=torch.float16).pin_memory()
        ha.copy_(a)
        hb.copy_(bs)
        e_steps = max(1, min(args.steps, 20))
        for _ in range(2):
            api.matmult_host(ha, hb, hc, False, True, accumulate=False)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            api.matmult_host(ha, hb, hc, False, True, accumulate=False)   # synchronous: returns with C on the host
        torch.cuda.synchronize()
        e_ms = (time.perf_counter() - t0) * 1e3 / e_steps
        if dist is not None:
            t = torch.tensor([e_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        ok = bool(torch.equal(hc[0].cuda(), c[0]))
        e2e = {"value": total_items * FLOPS_PER_ITEM / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(ha.numel() + hb.numel()) * 2, "d2h_bytes_per_step": int(hc.numel()) * 2,
               "ms_per_step": e_ms, "steps": e_steps, "matches_device_result": ok,
               "api": "ntb200_matmult_host (C ABI, pinned host buffers)"}

    peaks = measured_peaks()
    extras = {}
    if not args.no_extras and args.items == BATCH:
        # ---- the 8192^3 target shape, Float16 and BFloat16 (every rank runs its own copy; rank 0's numbers are reported)
        target = {}
        for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
            ta = (torch.randn((8192, 8192), generator=gen, device="cuda") * 0.1).to(dt)
            tb = (torch.randn((8192, 8192), generator=gen, device="cuda") * 0.1).to(dt)
            tc = torch.empty((8192, 8192), dtype=dt, device="cuda")
            for _ in range(3):
                api.gemm(ta, tb, tc)
            torch.cuda.synchronize()
            ev0.record()
            for _ in range(20):
                api.gemm(ta, tb, tc)
            ev1.record()
            torch.cuda.synchronize()
            t_ms = ev0.elapsed_time(ev1) / 20
            tf = 2.0 * 8192 ** 3 / (t_ms * 1e-3) / 1e12
            target[name] = {"ms": t_ms, "tflops": tf, "frac_of_burst_peak": tf / peaks["tflops_burst"], "route": _lib.last_route()}
            del ta, tb, tc
        target["peak"] = peaks["tflops_burst"]
        target["note"] = "20 launches after 3 warm-ups, operands (403 MB) exceed the L2"
        extras["target_8192"] = target
        # ---- more than one GPU: the N-sharded MLP step (strong scaling) through the C-ABI partitioner
        if world > 1:
            try:
                from neurotensor_b200 import bench_mlp_sharded
                # measure() agrees between the ranks on every failure it can meet (peer mapping, a flag exchange that
                # ran out of time) and then times the NCCL gather instead, saying so in the record
                rec = bench_mlp_sharded.measure(rank, world, dist, steps=20, check=True)
                chk = rec.get("check") or {}
                extras["mlp_n_sharded"] = {"workload": "BASELINE.json configs[3]: BFloat16 MLP 8192 x (4096 -> 16384 -> 4096), forward + backward, "
                                                       "every GEMM split over its output columns", "scaling": "strong",
                                           "ms_per_step": rec["ms_per_step"], "tflops": rec["tflops"], "gather": rec["gather"],
                                           "kernels_per_step": rec["kernels_per_step_rank0"],
                                           "matches_unsharded": bool(chk.get("bit_identical", False)),
                                           "unsharded_ms_per_step_same_gpu": chk.get("unsharded_ms_per_step_same_gpu"),
                                           "strong_scaling_efficiency": chk.get("strong_scaling_efficiency"), "check": chk,
                                           "forward_schedule": rec.get("forward_schedule"),
                                           "forward_schedule_trial_ms": rec.get("forward_schedule_trial_ms")}
                if rec.get("fused_gather_unavailable"):
                    extras["mlp_n_sharded"]["fused_gather_unavailable"] = rec["fused_gather_unavailable"]
            except Exception as exc:   # noqa: BLE001 - a failure every rank meets alike must not cost the headline line
                extras["mlp_n_sharded"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
                torch.cuda.synchronize()

        # ---- the same launch repeated for at least two seconds: what the GPU sustains under its power cap
        barrier()
        loop = max(50, int(2.2 / (ms_per_step * 1e-3)))
        sus_sampler = ClockSampler(local_rank)
        sus_sampler.start()
        ev0.record()
        for _ in range(loop):
            step()
        ev1.record()
        barrier()
        sus_clocks = sus_sampler.finish()
        sus_ms = ev0.elapsed_time(ev1)
        if dist is not None:
            t = torch.tensor([sus_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sus_ms = float(t.item())
        sus_tflops = count * FLOPS_PER_ITEM * loop / (sus_ms * 1e-3) / 1e12          # per GPU
        sus_peak = peaks["tflops_sustained"] or peaks["tflops_burst"]
        extras["sustained"] = {"seconds": sus_ms * 1e-3, "launches": loop, "tflops_per_gpu": sus_tflops,
                               "peak": sus_peak, "frac": sus_tflops / sus_peak,
                               "peak_source": "%s (sustained bf16 cuBLAS figure)" % peaks["source"], "clocks": sus_clocks}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    per_gpu_tflops = count * FLOPS_PER_ITEM / (ms_per_step * 1e-3) / 1e12
    timed_s = ms * 1e-3
    peak_kind = "sustained" if (timed_s > 1.0 and peaks["tflops_sustained"] > 0) else "burst"
    peak = peaks["tflops_sustained"] if peak_kind == "sustained" else peaks["tflops_burst"]
    line = {
        "metric": "matmult TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": total_items, "per_gpu_batch": count, "full_size": args.items == BATCH,
                   "parallelism": "batch-sharded x%d, no collective" % world,
                   "l2": "inputs (1.6 GB per step) exceed the 126 MB L2; no flush needed", "kernel": route},
        "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": per_gpu_tflops / peak, "traffic": NCU_DRAM_TRAFFIC_BYTES_PER_ITEM * count,
                     "traffic_source": "stored ncu profile of the same kernel on 8 items, scaled by the items per launch",
                     "peak_source": "%s (%s bf16 cuBLAS figure)" % (peaks["source"], peak_kind),
                     "algorithmic_flops_per_launch": count * FLOPS_PER_ITEM,
                     "algorithmic_bytes_per_launch": 3 * count * M * N * 2},
        "clocks": clocks, "gpu_launches": int(launches),
    }
    line.update(extras)
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
