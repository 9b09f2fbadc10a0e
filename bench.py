#!/usr/bin/env python
"""Benchmark of the LSH hot path on the SIFT-shaped RPLSH workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = fit(X) then query(Q): X is 1,000,000 x 128 fp32 with components
clip(round(Gamma(0.5, 40)), 0, 255) (SIFT-shaped synthetic; the SIFT1M files are not
available offline), Q is 10,000 rows of the same law, RPLSH with 32 tables x 16 hashes,
seed 0, query batch 10,000.  `value` is rows indexed-and-queried per second over all GPUs
with inputs resident in HBM; `e2e` is the same step through the public Python API with
pinned HOST arrays in and the candidates CSR read back to the host.

At N > 1 (torchrun, one rank per GPU) each rank holds its own 1M-row shard (weak scaling),
the queries are the same on every rank, and the per-shard candidates are exchanged over NCCL
(one all-to-all) so that rank j holds the merged CSR, with global row ids, of the j-th slice
of the queries.

`--impl reference` times upstream cuLSH's own CUDA build (oracle/_ref, compiled from the
upstream sources by oracle/Makefile) on the same workload when that module loads, else the
NumPy restatement of the path on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS, N_QUERIES, N_FEATURES = 1_000_000, 10_000, 128
N_TABLES, N_HASHES, SEED = 32, 16, 0
WORKLOAD = "RPLSH 1Mx128 fp32 SIFT-shaped synthetic, 32 tables x 16 hashes, 10k queries, batch 10k"  # at the default --rows/--queries


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(torch, device, rank):
    """Seeded synthetic data generated on the device (NumPy's gamma sampler needs ~15 s for X)."""
    g = torch.Generator(device=device)

    def draw(rows, seed):
        g.manual_seed(seed)
        conc = torch.full((rows, N_FEATURES), 0.5, device=device)
        x = torch._standard_gamma(conc, generator=g) * 40.0
        return torch.clamp(torch.round(x), 0, 255).to(torch.float32).contiguous()

    return draw(N_ROWS, 100 + rank), draw(N_QUERIES, 99)


def measure_tf32_peak(torch, device):
    """Dense TF32 matmul throughput (8192^3, best of 5), the denominator of the projection's
    roofline; MEASURED_PEAKS.json holds only the bf16 figure."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(8192, 8192, device=device)
        b = torch.randn(8192, 8192, device=device)
        best = None
        for i in range(7):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if i >= 2:
                best = ms if best is None else min(best, ms)
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def cpu_baseline(sample_rows=200_000, sample_queries=2_000):
    """NumPy restatement of the path (oracle/) on a bounded sample of the workload."""
    from oracle import oracle
    rng = np.random.default_rng(100)
    X = np.clip(np.round(rng.gamma(0.5, 40.0, (sample_rows, N_FEATURES))), 0, 255).astype(np.float32)
    Q = np.clip(np.round(rng.gamma(0.5, 40.0, (sample_queries, N_FEATURES))), 0, 255).astype(np.float32)
    P = np.random.default_rng(0).standard_normal((N_TABLES * N_HASHES, N_FEATURES)).astype(np.float32)
    t0 = time.perf_counter()
    bits = (~np.signbit(X @ P.T)).astype(np.uint8)
    tables = oracle.fast_fit_packed(oracle.pack_bits_msb_first(bits, N_TABLES, N_HASHES))
    t1 = time.perf_counter()
    qbits = (~np.signbit(Q @ P.T)).astype(np.uint8)
    oracle.fast_query_packed(tables, oracle.pack_bits_msb_first(qbits, N_TABLES, N_HASHES))
    t2 = time.perf_counter()
    return {"value": sample_rows / (t2 - t0), "unit": "rows/s", "cores": os.cpu_count(), "kind": "port",
            "fit_rows_per_s": sample_rows / (t1 - t0), "query_qps": sample_queries / (t2 - t1),
            "sample": f"{sample_rows} rows + {sample_queries} queries of the same law, same 32x16 RPLSH "
                      f"(NumPy matmul/argsort/searchsorted/unique, BLAS threads = all cores)"}


def dist_setup(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    else:
        torch.cuda.set_device(local)
    return world, rank, local


def max_over_ranks(torch, value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(torch, world):
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    world, rank, local = dist_setup(args)
    device = torch.device(f"cuda:{local}")
    import culsh_b200
    from culsh_b200 import _culsh_core, sharded

    Xd, Qd = make_inputs(torch, device, rank)
    Xh = torch.empty(Xd.shape, dtype=torch.float32, pin_memory=True)
    Qh = torch.empty(Qd.shape, dtype=torch.float32, pin_memory=True)
    Xh.copy_(Xd)
    Qh.copy_(Qd)
    torch.cuda.synchronize()
    Xh_np, Qh_np = Xh.numpy(), Qh.numpy()

    lsh = culsh_b200.RPLSH(N_TABLES, N_HASHES, seed=SEED)
    core = _culsh_core.RPLSHCore(N_TABLES, N_HASHES, SEED)
    core.set_profiling(True)

    stage = {"fit": [], "query": []}

    def step(X, Q, host_out):
        model = lsh.fit(X)
        s_fit = core.last_stats()
        cand = model.query(Q, batch_size=N_QUERIES)
        s_q = core.last_stats()
        if world > 1:  # each rank receives the merged lists of its slice of the queries
            cand, _ = sharded.exchange_by_query(cand, row_base=rank * N_ROWS,
                                                    row_bases=[r * N_ROWS for r in range(world)])
        d2h = 0
        if host_out and cand is not None:
            off = cand.get_offsets()
            cnt = cand.get_counts()
            idx = cand.get_indices()
            d2h = off.nbytes + cnt.nbytes + idx.nbytes
        return s_fit, s_q, d2h

    for _ in range(args.warmup):
        step(Xd, Qd, False)
    sampler = ClockSampler(local)
    barrier(torch, world)
    sampler.start()
    t0 = time.perf_counter()
    launches = 0
    for _ in range(args.steps):
        s_fit, s_q, _ = step(Xd, Qd, False)
        stage["fit"].append(s_fit)
        stage["query"].append(s_q)
        launches += s_fit["launches"] + s_q["launches"]
    barrier(torch, world)
    t_dev = max_over_ranks(torch, time.perf_counter() - t0, world, device)
    clocks = sampler.stop()

    # end to end: pinned host arrays in, CSR read back
    d2h = 0
    t_e2e = float("nan")
    if not args.skip_e2e:
        for _ in range(min(args.warmup, 2)):
            step(Xh_np, Qh_np, True)
        barrier(torch, world)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            _, _, b = step(Xh_np, Qh_np, True)
            d2h = max(d2h, b)
        barrier(torch, world)
        t_e2e = max_over_ranks(torch, time.perf_counter() - t0, world, device)

    if rank != 0:
        return
    peaks = load_peaks()
    ms_step = t_dev / args.steps * 1e3
    total_rows = N_ROWS * world
    fit_ms = statistics.mean(s["total_ms"] for s in stage["fit"])
    hash_ms = statistics.mean(s["hash_ms"] for s in stage["fit"])
    scatter_ms = statistics.mean(s["scatter_ms"] for s in stage["fit"])
    q_ms = statistics.mean(s["total_ms"] for s in stage["query"])
    gather_ms = statistics.mean(s["gather_ms"] for s in stage["query"])
    sf, sq = stage["fit"][-1], stage["query"][-1]
    passes = max(1, sf["sort_passes"])
    items = sf["n_items"]
    kb = 4 * sf["key_words"]
    tf32 = measure_tf32_peak(torch, device) if not args.skip_cpu else 690.0
    flops = 2.0 * N_ROWS * N_FEATURES * N_TABLES * N_HASHES
    proj = {"bound": "tensor", "achieved": flops / (hash_ms * 1e-3) / 1e12,
            "peak": tf32 / 3.0, "unit": "TFLOP/s",
            "kernel": "project_tc_kernel" if sf["hash_path"] == 1 else "project_simt_kernel",
            "note": "fp32-equivalent flop 2*n*d*H over the CUDA-event time of the projection launch; "
                    "peak = TF32 dense matmul measured in this run (8192^3) / 3 (3xTF32)",
            "tf32_tflops_measured": tf32, "traffic": None}
    proj["frac"] = proj["achieved"] / proj["peak"]
    sort_bytes = items * (kb + 4) * 2.0
    sort = {"bound": "hbm", "achieved": sort_bytes / (scatter_ms * 1e-3) / 1e9,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "kernel": "radix_scatter_kernel",
            "note": f"(key {kb} B + row id 4 B) read + written per item, one launch (the scatter of the "
                    f"last of {passes} passes) timed with CUDA events; peak {peaks['source']}", "traffic": None}
    sort["frac"] = sort["achieved"] / sort["peak"]
    gat_bytes = 4.0 * (sq["raw_candidates"] + 3 * sq["unique_candidates"])
    gather = {"bound": "hbm", "achieved": gat_bytes / (gather_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
              "unit": "GB/s", "kernel": "dedupe_bitmap_kernel+compact",
              "note": "4*raw read + 4*uniq written to scratch + 4*uniq read + 4*uniq written"}
    gather["frac"] = gather["achieved"] / gather["peak"]
    dominant = proj if hash_ms >= scatter_ms else sort
    line = {
        "metric": "RPLSH 1Mx128 32x16: fit + 10k-query rows/s",
        "value": total_rows / (t_dev / args.steps), "unit": "rows/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": N_ROWS, "queries": N_QUERIES,
                   "l2": "inputs (512 MB per step) larger than L2, no flush", "seed": SEED,
                   "parallelism": f"row-sharded x{world}" if world > 1 else "single GPU"},
        "fit_rows_per_s": N_ROWS * world / (fit_ms * 1e-3), "query_qps": N_QUERIES / (q_ms * 1e-3),
        "stage_ms": {"fit_total": fit_ms, "hash": hash_ms, "sort": statistics.mean(s["sort_ms"] for s in stage["fit"]),
                     "sort_scatter": scatter_ms, "build": statistics.mean(s["build_ms"] for s in stage["fit"]),
                     "query_total": q_ms, "query_hash": statistics.mean(s["hash_ms"] for s in stage["query"]),
                     "lookup": statistics.mean(s["lookup_ms"] for s in stage["query"]), "gather": gather_ms},
        "shape": {"buckets": sf["n_buckets"], "raw_candidates": sq["raw_candidates"],
                  "unique_candidates": sq["unique_candidates"]},
        "roofline": dominant, "roofline_all": {"projection": proj, "sort": sort, "gather": gather},
        "e2e": {"value": total_rows / (t_e2e / args.steps), "unit": "rows/s",
                "ms_per_step": t_e2e / args.steps * 1e3,
                "h2d_bytes_per_step": int(Xh_np.nbytes + Qh_np.nbytes), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": launches, "clocks": clocks,
    }
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------
def load_reference_module():
    path = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(path):
        return None
    sys.path.insert(0, path)
    try:
        import _culsh_core as ref
        return ref
    except Exception:
        return None


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ref = load_reference_module() if not args.reference_cpu else None
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    base = {"metric": "RPLSH 1Mx128 32x16: fit + 10k-query rows/s", "unit": "rows/s", "impl": "reference",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": N_ROWS, "queries": N_QUERIES, "seed": SEED}}
    if ref is None or not have_gpu:
        cb = cpu_baseline()
        base.update({"value": cb["value"], "ms_per_step": None, "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "rows/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    # upstream's CUDA build, driven through its own pybind11 API with torch tensors
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device(f"cuda:{local}")
    Xd, Qd = make_inputs(torch, device, 0)
    Xh = torch.empty(Xd.shape, dtype=torch.float32, pin_memory=True).copy_(Xd)
    Qh = torch.empty(Qd.shape, dtype=torch.float32, pin_memory=True).copy_(Qd)
    torch.cuda.synchronize()
    core = ref.RPLSHCore(N_TABLES, N_HASHES, SEED)

    def step(host):
        if host:
            X = Xh.to(device, non_blocking=True)
            Q = Qh.to(device, non_blocking=True)
            torch.cuda.synchronize()
        else:
            X, Q = Xd, Qd
        t0 = time.perf_counter()
        ix = core.fit_float(X, N_ROWS, N_FEATURES)
        t1 = time.perf_counter()
        cand = core.query_float(Q, N_QUERIES, ix, N_QUERIES)
        t2 = time.perf_counter()
        d2h = 0
        if host:
            a, b, c = cand.get_offsets(), cand.get_counts(), cand.get_indices()
            d2h = a.nbytes + b.nbytes + c.nbytes
        return t1 - t0, t2 - t1, d2h

    for _ in range(args.warmup):
        step(False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    fits, queries = [], []
    for _ in range(args.steps):
        f, q, _ = step(False)
        fits.append(f)
        queries.append(q)
    torch.cuda.synchronize()
    t_dev = time.perf_counter() - t0
    step(True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    d2h = 0
    for _ in range(args.steps):
        _, _, d2h = step(True)
    torch.cuda.synchronize()
    t_e2e = time.perf_counter() - t0
    base.update({
        "value": N_ROWS / (t_dev / args.steps), "ms_per_step": t_dev / args.steps * 1e3,
        "fit_rows_per_s": N_ROWS / statistics.mean(fits), "query_qps": N_QUERIES / statistics.mean(queries),
        "stage_ms": {"fit_total": statistics.mean(fits) * 1e3, "query_total": statistics.mean(queries) * 1e3},
        "cpu_baseline": {"value": N_ROWS / (t_dev / args.steps), "unit": "rows/s", "cores": 0, "kind": "reference",
                         "sample": "full workload; upstream cuLSH CUDA build (its cuBLAS/CUB kernels compiled for "
                                   "sm_100) on one B200 - upstream has no CPU implementation of this path"},
        "e2e": {"value": N_ROWS / (t_e2e / args.steps), "unit": "rows/s", "ms_per_step": t_e2e / args.steps * 1e3,
                "h2d_bytes_per_step": int(Xh.numel() * 4 + Qh.numel() * 4), "d2h_bytes_per_step": int(d2h)},
        "reference_device": "B200 (upstream CUDA build)",
    })
    if world > 1:
        base["config"]["note"] = "upstream is single-GPU: rank 0 runs one 1M-row shard"
    print(json.dumps(base))


def main():
    global N_ROWS, N_QUERIES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=N_ROWS, help="rows per GPU (default: the 1M-row workload)")
    ap.add_argument("--queries", type=int, default=N_QUERIES)
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: no host-input leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling runs: no CPU baseline leg")
    ap.add_argument("--reference-cpu", action="store_true",
                    help="reference arm: time the NumPy restatement on the host cores instead of "
                         "upstream's CUDA build")
    args = ap.parse_args()
    N_ROWS, N_QUERIES = args.rows, args.queries
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
