"""Benchmark of the FP8 block-scaled GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-sweep]

One "step" is one GEMM of the headline workload M=8192, N=4608, K=7168 (e4m3fn a/b, fp32 block
scales, bf16 out). With N GPUs the columns of b/b_scale are sharded over the ranks (strong
scaling: the total problem is fixed), a/a_scale are replicated and c stays sharded; there is no
data-path collective. Rank 0 prints ONE JSON line.

--impl reference times the reference's own algorithm for this path on the host cores (the CPU
restatement of its dequantise-then-matmul script; the reference's HIP sources cannot be built
for a CUDA machine) on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HEADLINE = (8192, 4608, 7168)
METRIC = "FP8 block-scaled GEMM TFLOPS (M=8192,N=4608,K=7168; bf16 out)"
UNIT = "TFLOP/s"
NOMINAL_FP8_TFLOPS = 4500.0
FALLBACK_BF16_TFLOPS = 1590.0
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes of one launch of the headline GEMM on one GPU, from an ncu capture of that launch
# (dram__bytes_read.sum 113.7 MB + dram__bytes_write.sum 57.4 MB).
HEADLINE_DRAM_BYTES = 171_100_000
SWEEP_NK = ((1536, 7168), (3072, 1536), (576, 7168), (7168, 256), (7168, 2048), (4608, 7168), (7168, 2304),
            (512, 7168), (4096, 512))
SWEEP_M = (512, 2048, 8192, 16384)
NAMED_CONFIGS = ((2048, 576, 7168), (2048, 7168, 512), (2048, 7168, 256))


def algorithmic_bytes(m, n, k):
    """Bytes one GEMM must move: a, b, both scale tensors in, bf16 c out."""
    return m * k + n * k + 4 * m * (k // 128) + 4 * ((n + 127) // 128) * (k // 128) + 2 * m * n


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the first samples precede the warm-up: drop the leading quarter
        sm_load = sm[len(sm) // 4:] if len(sm) >= 4 else sm
        return {"sm_mhz": statistics.median(sm_load) if sm_load else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def gpu_inputs(m, n, k, seed, device):
    """Synthetic inputs of the contract's distributions, generated on the device for speed
    (a, b ~ N(0,1) in bf16 cast to e4m3fn; scales ~ U(0.01, 1))."""
    g = torch.Generator(device=device).manual_seed(seed)
    a = torch.randn(m, k, dtype=torch.bfloat16, device=device, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, dtype=torch.bfloat16, device=device, generator=g).to(torch.float8_e4m3fn)
    a_s = 0.01 + 0.99 * torch.rand(m, k // 128, dtype=torch.float32, device=device, generator=g)
    b_s = 0.01 + 0.99 * torch.rand((n + 127) // 128, k // 128, dtype=torch.float32, device=device, generator=g)
    return a, b, a_s, b_s


def time_launches(fn_list, steps, warmup):
    """Average device time in ms of one call, cycling through fn_list (rotating buffer sets)."""
    for i in range(warmup):
        fn_list[i % len(fn_list)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn_list[i % len(fn_list)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def spot_check(pkg, a, b, a_s, b_s, c, n_phase=0, rows=128):
    """Cheap on-device check of `rows` rows against an fp32 dequantise-then-matmul in torch
    (the full CPU-oracle parity runs in tests/); contract tolerance rtol=2e-2, atol=1e-3."""
    m, n = c.shape
    idx = torch.linspace(0, m - 1, min(rows, m), device=c.device).long()
    jb = (torch.arange(n, device=c.device) + n_phase) // 128
    a32 = a[idx].float() * a_s[idx].repeat_interleave(128, dim=1)
    b32 = b.float() * b_s[jb].repeat_interleave(128, dim=1)
    ref = (a32 @ b32.T).to(torch.bfloat16).float()
    got = c[idx].float()
    return bool(((got - ref).abs() <= 1e-3 + 2e-2 * ref.abs()).all().item())


def cpu_oracle_tflops(n, k, target_seconds, threads=None):
    """Times the CPU restatement of the reference's path on a row sample of the workload."""
    from oracle import fp8_mm_oracle as oracle
    from amd_developer_challenge_2025_b200.inputs import make_inputs

    if threads:
        torch.set_num_threads(threads)
    rows = 64
    a, b, a_s, b_s, _ = make_inputs(rows, n, k, seed=3)
    oracle.dequant_matmul(a, b, a_s, b_s)  # warm-up (thread pools, allocator)
    t0 = time.perf_counter()
    oracle.dequant_matmul(a, b, a_s, b_s)
    t_probe = time.perf_counter() - t0
    # the dequantisation of b is a fixed cost per call; scale rows so one call takes ~target/3 s
    rows = int(max(64, min(8192, rows * (target_seconds / 3.0) / max(t_probe, 1e-4))))
    rows = (rows // 64) * 64
    a, b, a_s, b_s, _ = make_inputs(rows, n, k, seed=4)
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < target_seconds and len(times) < 20):
        t0 = time.perf_counter()
        oracle.dequant_matmul(a, b, a_s, b_s)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return 2.0 * rows * n * k / t / 1e12, rows, torch.get_num_threads(), t


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    m, n, k = HEADLINE
    per_step = []
    rows_used = 0
    threads = 0
    total = args.warmup + args.steps
    budget = max(2.0, min(20.0, 120.0 / max(total, 1)))
    for i in range(total):
        tf, rows_used, threads, t = cpu_oracle_tflops(n, k, budget)
        if i >= args.warmup:
            per_step.append((tf, t))
    tf = statistics.median(x[0] for x in per_step)
    sample = f"rows 0..{rows_used - 1} of a (M sample {rows_used} of {m}), full N={n}, K={k}; torch CPU fp32"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(tf, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(2.0 * m * n * k / (tf * 1e12) * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (e4m3fn inputs dequantised on CPU)",
        "data": "synthetic",
        "config": {"workload": "fp8_block_scaled_gemm M=8192 N=4608 K=7168", "path": "CPU dequantise-then-matmul"},
        "cpu_baseline": {"value": round(tf, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(tf, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import amd_developer_challenge_2025_b200 as pkg
    from amd_developer_challenge_2025_b200.fp8_mm import check_device_status

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    m, n, k = HEADLINE if not args.shape else tuple(int(x) for x in args.shape.split(","))
    # The ranks form a grid of row blocks x column blocks of c (no collective either way); the grid is the one
    # whose slowest rank the library's cost model rates fastest (8 GPUs: 4 x 2, one wave of 256 x 256 pair
    # tiles per GPU, where 1 x 8 would leave each GPU 2.2 waves of narrower tiles).
    grid_m, grid_n = (tuple(int(x) for x in args.grid.split("x")) if args.grid else pkg.choose_grid(m, n, k, world))
    spec = pkg.grid_spec(m, n, world, rank, grid_m, grid_n)
    m_full, m = m, spec.m_local
    n_loc = spec.n_local
    set_bytes = m * k + n_loc * k + 2 * m * n_loc
    nsets = max(2, -(-(2 * L2_BYTES + 64 * 1024 * 1024) // set_bytes))
    sets = []
    for s in range(nsets):
        a, b, a_s, b_s = gpu_inputs(m_full, n, k, 1000 + s, dev)
        aa, bb, aas, bs = pkg.grid_inputs(a, b, a_s, b_s, spec)
        sets.append((aa.contiguous(), bb.contiguous(), aas.contiguous(), bs.contiguous(),
                     torch.empty(m, n_loc, dtype=torch.bfloat16, device=dev)))
        del a, b, a_s, b_s
    plan = pkg.describe(m, n_loc, k, spec.n_phase)
    fns = [(lambda t=t: pkg.fp8_mm(t[0], t[1], t[2], t[3], t[4], n_phase=spec.n_phase)) for t in sets]

    # correctness of what is about to be timed
    fns[0]()
    check_device_status(dev)
    ok = spot_check(pkg, *sets[0], n_phase=spec.n_phase)

    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    ms_local = time_launches(fns, args.steps, args.warmup)
    barrier()
    clocks = sampler.stop() if sampler else None  # samples cover the timed GEMM loop only
    ms = max_over_ranks(ms_local)
    check_device_status(dev)

    # The same GEMM with a and b in the harness's MN-major storage ([K][M], [K][N]), consumed in place.
    mn_ms = None
    if world == 1:
        from amd_developer_challenge_2025_b200.inputs import mn_major
        a0, b0, as0, bs0, c0 = sets[0]
        am, bm = mn_major(a0), mn_major(b0)
        mn_fn = lambda: pkg.fp8_mm(am, bm, as0, bs0, c0)
        mn_ms = time_launches([mn_fn], min(args.steps, 50), 3)
        check_device_status(dev)
        del am, bm

    # Grouped launch (expert GEMMs of an MoE layer): 8 groups of 1024 x 2048 x 7168 in one kernel, beside the same
    # eight problems as separate launches.
    grouped = None
    if world == 1 and not args.shape and not args.no_sweep:
        gg, gm, gn, gk = 8, 1024, 2048, 7168
        parts = [gpu_inputs(gm, gn, gk, 4000 + i, dev) for i in range(gg)]
        ga, gb, gas, gbs = (torch.stack([p_[j] for p_ in parts]) for j in range(4))
        gc = torch.empty(gg, gm, gn, dtype=torch.bfloat16, device=dev)
        del parts
        one = lambda: pkg.fp8_mm_grouped(ga, gb, gas, gbs, gc)
        sep = lambda: [pkg.fp8_mm(ga[i], gb[i], gas[i], gbs[i], gc[i]) for i in range(gg)]
        t_one = time_launches([one], 30, 3)
        t_sep = time_launches([sep], 30, 3)
        gc.fill_(float("nan"))
        one()  # what the check below looks at is the grouped launch's output
        check_device_status(dev)
        gflop = 2.0 * gg * gm * gn * gk
        grouped = {"groups": gg, "m": gm, "n": gn, "k": gk, "ms": round(t_one, 5),
                   "tflops": round(gflop / (t_one * 1e-3) / 1e12, 1),
                   "separate_launches_ms": round(t_sep, 5),
                   "pass": bool(spot_check(pkg, ga[3], gb[3], gas[3], gbs[3], gc[3], rows=64))}
        del ga, gb, gas, gbs, gc

    # Optional all-gather of the column shards of c (not part of the timed GEMM; reported beside it).
    gather_ms = None
    if dist is not None and n % grid_n == 0 and m_full % (128 * grid_m) == 0:
        gathered = torch.empty(world, m, n_loc, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            dist.all_gather_into_tensor(gathered, sets[0][4])
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(10):
            dist.all_gather_into_tensor(gathered, sets[0][4])
        g1.record()
        torch.cuda.synchronize()
        gather_ms = max_over_ranks(g0.elapsed_time(g1) / 10)
        del gathered

    # end to end through the public call with host buffers (pinned), copies inside the timed region
    ha, hb, has_, hbs = (t.cpu().pin_memory() for t in sets[0][:4])
    hc = torch.empty(m, n_loc, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        pkg.fp8_mm_host(ha, hb, has_, hbs, hc, device=dev, n_phase=spec.n_phase)
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        pkg.fp8_mm_host(ha, hb, has_, hbs, hc, device=dev, n_phase=spec.n_phase)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    _ = time.perf_counter() - t0
    barrier()
    h2d = sum(t.numel() * t.element_size() for t in (ha, hb, has_, hbs))
    d2h = hc.numel() * hc.element_size()

    flops = 2.0 * m_full * n * k
    value = flops / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    per_gpu_tflops = 2.0 * m * n_loc * k / (ms_local * 1e-3) / 1e12

    per_shape = []
    cpu_baseline = None
    if rank == 0 and world == 1:
        if not args.no_sweep and not args.shape:
            shapes = list(NAMED_CONFIGS) + [(mm, nn, kk) for mm in SWEEP_M for (nn, kk) in SWEEP_NK]
            for (mm, nn, kk) in shapes:
                # enough rotating input/output sets that consecutive launches do not find their
                # operands in L2 (capped at 12 sets), one CUDA graph of one launch per set
                set_b = mm * kk + nn * kk + 2 * mm * nn
                nset = max(2, min(12, -(-(2 * L2_BYTES) // set_b)))
                ins = [gpu_inputs(mm, nn, kk, mm + nn + kk + i, dev) for i in range(nset)]
                outs = [torch.empty(mm, nn, dtype=torch.bfloat16, device=dev) for _ in range(nset)]
                pkg.fp8_mm(*ins[0], outs[0])
                good = spot_check(pkg, *ins[0], outs[0], rows=64)
                graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        for t, o in zip(ins, outs):
                            pkg.fp8_mm(*t, o)
                torch.cuda.synchronize()
                reps = max(3, 48 // nset)
                t_ms = time_launches([graph.replay], reps, 2) / nset
                pl = pkg.describe(mm, nn, kk)
                tf = 2.0 * mm * nn * kk / (t_ms * 1e-3) / 1e12
                gbs = algorithmic_bytes(mm, nn, kk) / (t_ms * 1e-3) / 1e9
                per_shape.append({
                    "m": mm, "n": nn, "k": kk, "us": round(t_ms * 1e3, 2), "tflops": round(tf, 1),
                    "pct_fp8_peak_measured": round(100 * tf / fp8_peak, 1),
                    "pct_fp8_peak_nominal": round(100 * tf / NOMINAL_FP8_TFLOPS, 1),
                    "gbs": round(gbs, 1), "pct_hbm_measured": round(100 * gbs / peaks["hbm_gbs"], 1),
                    "plan": f"{'2x' if pl.cta_pair else ''}128x{pl.block_n} split{pl.split_k} st{pl.stages}",
                    "pass": good})
                del ins, outs, graph
            check_device_status(dev)
        tf_cpu, rows_used, threads, _t = cpu_oracle_tflops(n, k, 12.0)
        cpu_baseline = {"value": round(tf_cpu, 4), "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"M sample {rows_used} of {m} rows, full N={n}, K={k}; torch CPU fp32 "
                                  f"dequantise-then-matmul"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "e4m3fn x e4m3fn -> fp32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": f"fp8_block_scaled_gemm M={m_full} N={n} K={k}",
                       "sharding": f"{grid_m} x {grid_n} grid of row x column blocks of c: {m} rows x {n_loc} columns "
                                   f"per GPU, no collective, c left sharded",
                       "plan": f"{'2x' if plan.cta_pair else ''}128x{plan.block_n} split{plan.split_k} "
                               f"stages{plan.stages} grid{plan.grid}",
                       "l2": f"{nsets} rotating buffer sets of {set_bytes >> 20} MiB (> 2x L2) between launches",
                       "spot_check_pass": ok},
            "pct_fp8_peak_nominal": round(100 * value / (NOMINAL_FP8_TFLOPS * world), 2),
            "roofline": {"bound": "tensor", "achieved": round(per_gpu_tflops, 2), "peak": round(fp8_peak, 1),
                         "unit": "TFLOP/s", "frac": round(per_gpu_tflops / fp8_peak, 4),
                         "peak_source": f"2 x bf16_tflops of {peaks['source']} (fp8 tcgen05 rate is twice bf16)",
                         "traffic": HEADLINE_DRAM_BYTES if (world == 1 and not args.shape) else None,
                         "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                         "algorithmic_bytes": algorithmic_bytes(m, n_loc, k)},
            "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 3), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if mn_ms is not None:
            line["mn_major_operands"] = {"ms_per_step": round(mn_ms, 5),
                                         "value": round(flops / (mn_ms * 1e-3) / 1e12, 2), "unit": UNIT}
        if grouped is not None:
            line["grouped"] = grouped
        if gather_ms is not None:
            line["all_gather_c"] = {"ms": round(gather_ms, 4), "bytes_per_rank": 2 * m * n_loc,
                                    "note": "NCCL all_gather_into_tensor of the bf16 blocks into [ranks, rows, columns]; "
                                            "outside the timed GEMM"}
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        if per_shape:
            line["per_shape"] = per_shape
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # 2000 steps of ~0.3 ms: long enough for the power cap to settle and for the clock sampler
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-shape sweep (N=1 only)")
    ap.add_argument("--shape", default="", help="M,N,K of another workload (for small profiler captures)")
    ap.add_argument("--grid", default="", help="ROWSxCOLS grid of the ranks (default: the cost model's choice)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
