#!/usr/bin/env python
"""Benchmark of the LSH hot path (hash -> bucket index -> lookup -> gather/dedupe -> CSR).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

Default workload "c2" (the one the headline metric is quoted on): one step = fit(X) then
query(Q); X is 1,000,000 x 128 fp32 with components clip(round(Gamma(0.5, 40)), 0, 255)
(SIFT-shaped synthetic; the SIFT1M files are not available offline), Q is 10,000 rows of the
same law, RPLSH with 32 tables x 16 hashes, seed 0, query batch 10,000.  `value` is rows
indexed-and-queried per second over all GPUs with inputs resident in HBM; `e2e` is the same
step with pinned HOST arrays in and the candidates CSR read back to the host.

Other workloads (same JSON line, for the remaining benchmark configurations):
  c1  PStableLSH 10,000 x 128 N(0,1), 100 queries, 16 x 8, window "auto" (= 11), seed 42
  c3  MinHashLSH 2,000,000 rows x 2^20 columns, row nnz ~ U[20,200], Zipf(1.1) column ids,
      10,000 queries (half fresh, half perturbed copies), 32 x 4, seed 1
  c4  PStableLSH, one 12,500,000 x 96 shard per GPU of the 100M-row mixture of 4,096 Gaussians
      (sigma 0.15), 10,000 queries, 16 x 8, window 4, seed 2
  c5  RPLSH fit_query self-join, 10,000,000 x 256 unit-sphere rows, 48 x 24, seed 3 (1 GPU)

At N > 1 (torchrun, one rank per GPU) each rank holds its own shard (weak scaling), the
queries are the same on every rank, and rank j ends up with the merged CSR, with global row
ids, of the j-th slice of the queries: every rank publishes its per-shard CSR in peer-mapped
device memory and each rank's merge kernel reads the lists it needs straight from its peers
over NVLink (NCCL carries only two one-word all-reduces per step as barriers).

`--impl reference` times upstream cuLSH's own CUDA build (oracle/_ref, compiled from the
upstream sources by oracle/Makefile) on the same workload when that module loads, else the
NumPy restatement of the path on the host cores.

Every fit in the timed regions generates its hash parameters again (the per-handle parameter
cache is switched off), as upstream does; `cached_params` gives the same step with the cache
on, `first_call_ms` the very first step of the process (cold scratch, cold allocator).

Outside the timed regions both arms add `parity` (number of candidates and a checksum of the
CSR of one step), and this arm, when upstream's build loads, counts the signature elements on
which the two builds disagree and whether each lies inside the 1e-5 rounding band.  With the
default workload the line also carries `extra`: a few steps of c4 (one 12.5M-row shard per
GPU) and of the c5 self-join (10M rows over all GPUs).
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

WORKLOADS = {
    "c1": dict(family="pslsh", n=10_000, nq=100, d=128, L=16, k=8, w=11, seed=42, mode="fit+query",
               name="PStableLSH 10kx128 N(0,1), 16 tables x 8 hashes, window auto(=11), 100 queries"),
    "c2": dict(family="rplsh", n=1_000_000, nq=10_000, d=128, L=32, k=16, seed=0, mode="fit+query",
               name="RPLSH 1Mx128 fp32 SIFT-shaped synthetic, 32 tables x 16 hashes, 10k queries, batch 10k"),
    "c3": dict(family="minhash", n=2_000_000, nq=10_000, d=1 << 20, L=32, k=4, seed=1, mode="fit+query",
               name="MinHashLSH 2M rows x 2^20 cols, nnz U[20,200], Zipf(1.1) ids, 32 tables x 4 hashes, 10k queries"),
    "c4": dict(family="pslsh", n=12_500_000, nq=10_000, d=96, L=16, k=8, w=4, seed=2, mode="fit+query",
               name="PStableLSH 12.5Mx96 shard per GPU (100M-row mixture of 4096 Gaussians), 16x8, w=4, 10k queries"),
    "c5": dict(family="rplsh", n=10_000_000, nq=0, d=256, L=48, k=24, seed=3, mode="fit_query",
               name="RPLSH fit_query self-join 10Mx256 unit sphere, 48 tables x 24 hashes"),
}
METRICS = {
    "c1": "PStableLSH 10kx128 16x8: fit + 100-query rows/s",
    "c2": "RPLSH 1Mx128 32x16: fit + 10k-query rows/s",
    "c3": "MinHashLSH 2Mx2^20 32x4: fit + 10k-query rows/s",
    "c4": "PStableLSH 12.5Mx96 shard 16x8: fit + 10k-query rows/s",
    "c5": "RPLSH 10Mx256 48x24: fit_query rows/s",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        # nvidia-smi numbers GPUs physically, CUDA numbers the visible ones: address by UUID
        self.gpu = str(gpu_index)
        try:
            import torch
            self.gpu = "GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid)
        except Exception:
            pass
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu)],
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


# ------------------------------------------------------------------------------------------
# synthetic inputs (seeded, generated on the device)
# ------------------------------------------------------------------------------------------
def _csr_from_pairs(torch, rows, cols, n_rows):
    """Sorted, duplicate-free CSR (int32 indices / indptr) from (row, col) pairs."""
    key = torch.unique(rows.to(torch.int64) << 32 | cols.to(torch.int64))
    r = (key >> 32)
    indices = (key & 0xFFFFFFFF).to(torch.int32)
    indptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=key.device)
    indptr[1:] = torch.cumsum(torch.bincount(r, minlength=n_rows), 0)
    return indices.contiguous(), indptr.to(torch.int32).contiguous()


def _zipf_columns(torch, count, n_cols, g, device, s=1.1):
    """Column ids with P(id = i) ~ (i+1)^-s, by inverting the continuous CDF."""
    u = torch.rand(count, device=device, generator=g, dtype=torch.float64)
    a = 1.0 - s
    x = (1.0 - u * (1.0 - float(n_cols) ** a)) ** (1.0 / a)
    return torch.clamp(x.to(torch.int64) - 1, 0, n_cols - 1)


def make_inputs(torch, device, rank, wl, spec):
    """Returns (X, Q): dense fp32 tensors, or (indices, indptr) tuples for MinHash."""
    g = torch.Generator(device=device)
    n, nq, d = spec["n"], spec["nq"], spec["d"]
    if wl == "c1":
        X = torch.from_numpy(np.random.RandomState(42).randn(n, d).astype(np.float32)).to(device)
        Q = torch.from_numpy(np.random.RandomState(7).randn(nq, d).astype(np.float32)).to(device)
        return X, Q
    if wl == "c2":
        def draw(rows, seed):
            g.manual_seed(seed)
            conc = torch.full((rows, d), 0.5, device=device)
            x = torch._standard_gamma(conc, generator=g) * 40.0
            return torch.clamp(torch.round(x), 0, 255).to(torch.float32).contiguous()
        return draw(n, 100 + rank), draw(nq, 99)
    if wl == "c3":
        def rows_csr(n_rows, seed):
            g.manual_seed(seed)
            nnz = torch.randint(20, 201, (n_rows,), device=device, generator=g)
            rows = torch.repeat_interleave(torch.arange(n_rows, device=device), nnz)
            cols = _zipf_columns(torch, int(rows.numel()), d, g, device)
            return rows, cols
        rows, cols = rows_csr(n, 300 + rank)
        X = _csr_from_pairs(torch, rows, cols, n)
        # queries: half fresh rows, half copies of random X rows with ~10% of the columns
        # dropped and ~10% new Zipf columns added
        half = nq // 2
        fr, fc = rows_csr(half, 299)
        g.manual_seed(298)
        src = torch.randint(0, n, (nq - half,), device=device, generator=g)
        xi, xp = X[0].to(torch.int64), X[1].to(torch.int64)
        lens = xp[src + 1] - xp[src]
        qrow = torch.repeat_interleave(torch.arange(nq - half, device=device), lens)
        start = torch.repeat_interleave(xp[src], lens)
        within = torch.arange(int(lens.sum()), device=device) - torch.repeat_interleave(torch.cumsum(lens, 0) - lens, lens)
        ccol = xi[start + within]
        keep = torch.rand(ccol.numel(), device=device, generator=g) >= 0.1
        add_n = torch.clamp((lens.to(torch.float32) * 0.1).round().to(torch.int64), min=1)
        arow = torch.repeat_interleave(torch.arange(nq - half, device=device), add_n)
        acol = _zipf_columns(torch, int(arow.numel()), d, g, device)
        qr = torch.cat([fr, qrow[keep] + half, arow + half])
        qc = torch.cat([fc, ccol[keep], acol])
        return X, _csr_from_pairs(torch, qr, qc, nq)
    if wl == "c4":
        g.manual_seed(2)
        centres = torch.randn(4096, d, device=device, generator=g)
        g.manual_seed(400 + rank)
        X = centres[torch.randint(0, 4096, (n,), device=device, generator=g)]
        X = (X + 0.15 * torch.randn(n, d, device=device, generator=g)).contiguous()
        g.manual_seed(399)
        Q = centres[torch.randint(0, 4096, (nq,), device=device, generator=g)]
        Q = (Q + 0.15 * torch.randn(nq, d, device=device, generator=g)).contiguous()
        return X, Q
    if wl == "c5":
        g.manual_seed(3)
        X = torch.randn(n, d, device=device, generator=g)
        X = (X / X.norm(dim=1, keepdim=True)).contiguous()
        return X, None
    raise ValueError(wl)


def to_pinned_host(torch, t):
    if t is None:
        return None
    if isinstance(t, tuple):
        return tuple(to_pinned_host(torch, x) for x in t)
    h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    h.copy_(t)
    return h.numpy()


def nbytes_of(x):
    if x is None:
        return 0
    if isinstance(x, tuple):
        return sum(nbytes_of(y) for y in x)
    return int(x.nbytes) if hasattr(x, "nbytes") else int(x.numel() * x.element_size())


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


CPU_SAMPLES = {  # bounded samples of each workload for the CPU leg: (rows, queries)
    "c1": (10_000, 100), "c2": (200_000, 2_000), "c3": (20_000, 500), "c4": (200_000, 2_000),
    "c5": (100_000, 0),
}


def cpu_baseline(wl="c2"):
    """NumPy restatement of the path (oracle/) on a bounded sample of workload `wl`: same value
    law (the sample is drawn by make_inputs on the CPU), same tables x hashes, hash parameters
    from NumPy's generator."""
    import torch
    from oracle import oracle
    spec = dict(WORKLOADS[wl])
    rows, queries = CPU_SAMPLES[wl]
    spec["n"], spec["nq"] = min(rows, spec["n"]), min(queries, spec["nq"])
    n, nq, L, k, d = spec["n"], spec["nq"], spec["L"], spec["k"], spec["d"]
    X, Q = make_inputs(torch, torch.device("cpu"), 0, wl, spec)
    as_np = lambda t: None if t is None else (tuple(x.numpy() for x in t) if isinstance(t, tuple) else t.numpy())  # noqa: E731
    X, Q = as_np(X), as_np(Q)
    H = L * k
    rng = np.random.default_rng(spec["seed"])
    if spec["family"] == "minhash":
        A, B = oracle.minhash_normalize(rng.integers(0, 1 << 32, H, dtype=np.uint64),
                                        rng.integers(0, 1 << 32, H, dtype=np.uint64))
        hash_fn = lambda M: oracle.minhash_signatures(M[0], M[1], A, B)  # noqa: E731
    elif spec["family"] == "rplsh":
        P = rng.standard_normal((H, d)).astype(np.float32)
        hash_fn = lambda M: (~np.signbit(M @ P.T)).astype(np.uint8)  # noqa: E731
    else:
        P = (rng.standard_normal((H, d)) / spec["w"]).astype(np.float32)
        bias = rng.uniform(0.0, 1.0, H).astype(np.float32)
        hash_fn = lambda M: np.floor(M @ P.T + bias[None, :]).astype(np.int32)  # noqa: E731
    t0 = time.perf_counter()
    sig_x = hash_fn(X)
    if spec["mode"] == "fit_query":
        kx, kq = oracle.signature_keys(sig_x, sig_x[:0], L, k)
        tables = oracle.fast_fit_packed(kx)
        t1 = time.perf_counter()
        oracle.fast_query_packed(tables, kx)
        nq_run = n
    else:
        sig_q = hash_fn(Q)
        kx, kq = oracle.signature_keys(sig_x, sig_q, L, k)
        tables = oracle.fast_fit_packed(kx)
        t1 = time.perf_counter()
        oracle.fast_query_packed(tables, kq)
        nq_run = nq
    t2 = time.perf_counter()
    return {"value": n / (t2 - t0), "unit": "rows/s", "cores": os.cpu_count(), "kind": "port",
            "fit_rows_per_s": n / (t1 - t0), "query_qps": nq_run / max(t2 - t1, 1e-9),
            "sample": f"{n} rows + {nq_run} queries of the {wl} law, same {L}x{k} {spec['family']} "
                      f"(NumPy matmul / argsort / searchsorted / unique, BLAS threads = all cores)"}


# ------------------------------------------------------------------------------------------
# result checks (outside the timed regions)
# ------------------------------------------------------------------------------------------
CHECKSUM_MOD = (1 << 61) - 1


def csr_checksum(torch, indices, offsets, device):
    """sum over (query q, candidate id) of id * (q + 1), mod 2^61 - 1, on the device.
    `indices` / `offsets` are torch tensors or NumPy arrays (int32 / 64-bit)."""
    if not torch.is_tensor(offsets):
        offsets = torch.from_numpy(np.ascontiguousarray(offsets).view(np.int64))
    offsets = offsets.to(device=device, dtype=torch.int64)
    total = int(offsets[-1].item())
    acc, step = 0, 1 << 26
    for lo in range(0, total, step):
        hi = min(total, lo + step)
        chunk = indices[lo:hi]
        if not torch.is_tensor(chunk):
            chunk = torch.from_numpy(np.ascontiguousarray(chunk))
        ids = chunk.to(device=device, dtype=torch.int64)
        pos = torch.arange(lo, hi, device=device, dtype=torch.int64)
        q = torch.searchsorted(offsets, pos, right=True)  # = query index + 1
        acc = (acc + int(((ids * q) % CHECKSUM_MOD).sum().item())) % CHECKSUM_MOD
    return acc


def row_signatures(torch, device, ix, n, L):
    """uint8 [L, n, s]: raw signature bytes of every (table, row), recovered from an index's
    four arrays (either implementation's getters)."""
    s = int(ix.sig_nbytes)
    bco = torch.from_numpy(ix.get_bucket_candidate_offsets()).to(device).long()
    bs = torch.from_numpy(ix.get_bucket_signatures()).to(device).view(-1, s)
    cand = torch.from_numpy(ix.get_candidate_indices()).to(device).long()
    B = bco.numel() - 1
    bucket_of_item = torch.repeat_interleave(torch.arange(B, device=device), bco[1:] - bco[:-1])
    out = torch.empty((L * n, s), dtype=torch.uint8, device=device)
    table = torch.arange(n * L, device=device) // n
    out[table * n + cand] = bs[bucket_of_item]
    return out.view(L, n, s)


def signature_mismatch(torch, family, sig_a, sig_b, X, P, bias, k, rel=1e-5):
    """Compare two [L, n, s] signature arrays element by element (k elements per signature) and
    classify every differing element by a float64 recomputation of its projection: inside the
    band when |x.p| <= rel * sum|x_i p_i| (RPLSH) or dist(x.p + b, Z) <= rel * max(1, sum|x_i
    p_i| + |b|) (p-stable).  Returns counts and the rows that hold a differing element."""
    L, n, s = sig_a.shape
    eb = s // k
    differ = (sig_a.view(L, n, k, eb) != sig_b.view(L, n, k, eb)).any(dim=3)
    where = differ.nonzero()
    m = int(where.shape[0])
    in_band = 0
    for lo in range(0, m, 1 << 16):
        t, row, j = where[lo:lo + (1 << 16)].unbind(1)
        h = t * k + j
        x, p = X[row].double(), P[h].double()
        v, scale = (x * p).sum(1), (x.abs() * p.abs()).sum(1)
        if family == "rplsh":
            ok = v.abs() <= rel * scale
        else:
            b = bias[h].double()
            v = v + b
            ok = (v - torch.round(v)).abs() <= rel * torch.clamp(scale + b.abs(), min=1.0)
        in_band += int(ok.sum().item())
    rows = torch.unique(where[:, 1]) if m else where.new_zeros(0)
    return {"elements": int(L * n * k), "mismatch": m, "in_band": in_band, "out_of_band": m - in_band,
            "rows": rows}


def dist_setup():
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
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
# one step of a workload on either implementation's core classes (same class surface)
# ------------------------------------------------------------------------------------------
def make_core(mod, spec):
    if spec["family"] == "rplsh":
        return mod.RPLSHCore(spec["L"], spec["k"], spec["seed"])
    if spec["family"] == "pslsh":
        return mod.PSLSHCore(spec["L"], spec["k"], spec["w"], spec["seed"])
    return mod.MinHashCore(spec["L"], spec["k"], spec["seed"])


def core_fit(core, spec, X):
    if spec["family"] == "minhash":
        return core.fit(X[0], X[1], spec["n"], spec["d"])
    return core.fit_float(X, spec["n"], spec["d"])


def core_query(core, spec, Q, index, batch):
    if spec["family"] == "minhash":
        return core.query(Q[0], Q[1], spec["nq"], index)
    return core.query_float(Q, spec["nq"], index, batch)


def read_back(cand):
    a, b, c = cand.get_offsets(), cand.get_counts(), cand.get_indices()
    return a.nbytes + b.nbytes + c.nbytes


def config_of(wl, spec):
    """The same dict in both arms."""
    return {"workload": spec["name"], "id": wl, "rows_per_gpu": spec["n"], "queries": spec["nq"],
            "seed": spec["seed"]}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels,
# from ncu captures of launches of exactly this size (summaries and commands under profiles/);
# a workload or size without a capture reports null.
NCU_TRAFFIC = {
    ("c2", 1_000_000): {
        "gather": 273_526_528 + 677_084_416,   # profiles/dedupe_chained_rank_kernel_c2_1M.md
        "sort": 264_078_336 + 203_595_776,     # profiles/radix_scatter_kernel_c2_1M.md (second pass)
        "hash": 512_630_784 + 113_564_928,     # profiles/project_tc_kernel_c2_1M.md
    },
}


def check_exchange(torch, world, rank, n, local_cand, merged, span):
    """After an exchange every rank checks its merged slice: ids ascending inside a query, ids of
    shard r inside r's row range, per-query count equal to the sum of the per-shard counts,
    and for one query per rank the merged list equal to the shards' lists laid end to end."""
    import torch.distributed as dist
    from culsh_b200 import sharded
    lo, hi = span
    problems = []
    idx, off = sharded._csr_tensors(merged)
    l_idx, l_off = sharded._csr_tensors(local_cand)
    counts = (l_off[1:] - l_off[:-1]).contiguous()
    total = counts.clone()
    dist.all_reduce(total)
    mine = off[1:] - off[:-1]
    if mine.numel() != hi - lo or not bool((mine == total[lo:hi]).all()):
        problems.append("per-query counts differ from the sum over shards")
    if idx.numel():
        if int(idx.min()) < 0 or int(idx.max()) >= n * world:
            problems.append("id outside the global row range")
        d = idx[1:] > idx[:-1]
        starts = off[1:-1]
        starts = starts[(starts > 0) & (starts < idx.numel())]
        d[starts - 1] = True
        if not bool(d.all()):
            problems.append("ids not strictly ascending inside a query")
    for j in range(world):  # rank j's first query, gathered from every shard
        qj = sharded.shard_bounds(local_cand.n_queries, world, j)[0]
        piece = (l_idx[int(l_off[qj]):int(l_off[qj + 1])].long() + rank * n).cpu()
        parts = [None] * world
        dist.all_gather_object(parts, piece)
        if j == rank and hi > lo:
            want = torch.cat(parts)
            got = idx[int(off[0]):int(off[1])].long().cpu()
            if want.numel() != got.numel() or not bool((want == got).all()):
                problems.append(f"query {qj}: merged list differs from the shards' lists")
    flag = torch.tensor([len(problems)], device=idx.device if idx.numel() else off.device)
    dist.all_reduce(flag)
    return "ok" if int(flag.item()) == 0 else ("FAILED: " + "; ".join(problems) if problems else "FAILED on another rank")


def run_workload(torch, args, wl, spec, world, rank, local, exchange, steps, warmup, e2e=True, checks=True):
    """Times `steps` steps of one workload on this rank (collectively at world > 1) and returns
    the measurements; rank 0 turns them into the JSON line."""
    from culsh_b200 import _culsh_core, sharded
    import culsh_b200
    device = torch.device(f"cuda:{local}")
    sharded_join = spec["mode"] == "fit_query" and world > 1
    if sharded_join:  # strong scaling: the rows of the one data set are cut over the ranks
        lo, hi = sharded.shard_bounds(spec["n"], world, rank)
        full = dict(spec)
        Xd, Qd = make_inputs(torch, device, 0, wl, full)
        Xd = Xd[lo:hi].contiguous()
        n = hi - lo
    else:
        Xd, Qd = make_inputs(torch, device, rank, wl, spec)
        n = spec["n"]
    nq = spec["nq"]
    spec_local = dict(spec, n=n)
    core = make_core(_culsh_core, spec_local)
    core.set_profiling(True)
    batch = nq if wl == "c2" else None
    stage = {"fit": [], "query": []}
    keep = {}

    def step(X, Q, host_out):
        if sharded_join:
            est = culsh_b200.RPLSH(spec["L"], spec["k"], seed=spec["seed"])
            cand, _ = sharded.fit_query_sharded(est, X, exchange)
            s_fit = core.last_stats()
            s_q = dict(s_fit, total_ms=0.0, hash_ms=0.0, lookup_ms=0.0, launches=0)
        elif spec["mode"] == "fit_query":
            cand = core.fit_query_float(X, n, spec["d"])
            s_fit = core.last_stats()
            s_q = dict(s_fit, total_ms=0.0, hash_ms=0.0, lookup_ms=0.0, launches=0)
        else:
            index = core_fit(core, spec_local, X)
            s_fit = core.last_stats()
            cand = core_query(core, spec_local, Q, index, batch)
            s_q = core.last_stats()
            if world > 1:  # each rank pulls the lists of its slice of the queries from its peers
                keep["local"] = cand
                cand, keep["span"] = exchange.exchange(cand, [r * n for r in range(world)])
                s_q = dict(s_q, **{"x_" + key: val for key, val in exchange.last_ms.items()})
        keep["cand"] = cand
        return s_fit, s_q, (read_back(cand) if host_out else 0)

    out = {"n": n, "nq": nq, "device": device, "in_bytes": nbytes_of(Xd), "nnz": int(Xd[0].numel()) if isinstance(Xd, tuple) else 0}
    barrier(torch, world)
    t0 = time.perf_counter()
    step(Xd, Qd, False)
    barrier(torch, world)
    out["first_call_ms"] = max_over_ranks(torch, time.perf_counter() - t0, world, device) * 1e3

    def timed(n_warm, n_steps, X, Q, host_out, record):
        for _ in range(n_warm):
            step(X, Q, host_out)
        barrier(torch, world)
        t0 = time.perf_counter()
        launches, moved = 0, 0
        for _ in range(n_steps):
            s_fit, s_q, b = step(X, Q, host_out)
            moved = max(moved, b)
            if record:
                stage["fit"].append(s_fit)
                stage["query"].append(s_q)
                launches += s_fit["launches"] + s_q["launches"]
        barrier(torch, world)
        return max_over_ranks(torch, time.perf_counter() - t0, world, device), launches, moved

    # same step with the per-handle parameter cache on (a repeated fit with one seed)
    out["t_cached"], _, _ = timed(warmup, max(3, steps // 5), Xd, Qd, False, False)
    core.set_param_cache(False)   # from here on every fit generates its parameters, as upstream does
    sampler = ClockSampler(local)
    for _ in range(warmup):
        step(Xd, Qd, False)
    barrier(torch, world)
    sampler.start()
    out["t_dev"], out["launches"], _ = timed(0, steps, Xd, Qd, False, True)
    out["clocks"] = sampler.stop()
    out["stage"] = stage

    out["exchange_check"] = None
    if world > 1 and checks and not sharded_join:
        out["exchange_check"] = check_exchange(torch, world, rank, n, keep["local"], keep["cand"], keep["span"])

    out["parity"] = None
    if checks and world == 1:
        cand = keep["cand"]
        idx, off = sharded._csr_tensors(cand)
        out["parity"] = {"unique_candidates": int(cand.n_total_candidates),
                         "csr_checksum": csr_checksum(torch, idx, off, device)}
        out["parity"].update(parity_against_reference(torch, wl, spec_local, core, Xd, device))
    keep.clear()

    out["t_e2e"], out["h2d"], out["d2h"] = float("nan"), 0, 0
    if e2e:
        Xh, Qh = to_pinned_host(torch, Xd), to_pinned_host(torch, Qd)
        out["h2d"] = nbytes_of(Xh) + nbytes_of(Qh)
        out["t_e2e"], _, out["d2h"] = timed(2, steps, Xh, Qh, True, False)
    core.set_param_cache(True)
    return out


def parity_against_reference(torch, wl, spec, core, Xd, device):
    """When upstream's CUDA build (oracle/_ref) loads: fit the same rows with it and compare the
    stored signatures of the two indexes element by element (dense families), or the four
    index arrays (MinHash)."""
    ref = load_reference_module()
    n, L, k = spec["n"], spec["L"], spec["k"]
    sig_bytes = k * (1 if spec["family"] == "rplsh" else 4)
    if ref is None:
        return {"reference": "upstream build not loadable"}
    if float(n) * L * sig_bytes > 8e9:
        return {"reference": "skipped: signature arrays above 8 GB (covered at reduced size by tests/)"}
    torch.cuda.synchronize()
    ours = core_fit(core, spec, Xd)
    theirs = core_fit(make_core(ref, spec), spec, Xd)
    if spec["family"] == "minhash":
        same = all(np.array_equal(getattr(ours, g)(), getattr(theirs, g)())
                   for g in ("get_table_bucket_offsets", "get_bucket_candidate_offsets",
                             "get_bucket_signatures", "get_candidate_indices", "get_hash_a", "get_hash_b"))
        return {"reference": "upstream CUDA build, same rows", "index_arrays_equal": bool(same)}
    P_ours, P_ref = ours.get_projection_matrix(), theirs.get_projection_matrix()
    params_equal = bool(np.array_equal(P_ours, P_ref))
    bias = None
    if spec["family"] == "pslsh":
        params_equal = params_equal and bool(np.array_equal(ours.get_bias(), theirs.get_bias()))
        bias = torch.from_numpy(theirs.get_bias()).to(device)
    P = torch.from_numpy(P_ref).to(device).view(L * k, spec["d"])
    mm = signature_mismatch(torch, spec["family"], row_signatures(torch, device, theirs, n, L),
                            row_signatures(torch, device, ours, n, L), Xd, P, bias, k)
    return {"reference": "upstream CUDA build, same rows", "hash_parameters_equal": params_equal,
            "sig_elements": mm["elements"], "sig_mismatch_in_band": mm["in_band"],
            "sig_mismatch_out_of_band": mm["out_of_band"], "rows_with_mismatch": int(mm["rows"].numel())}


def line_of(torch, args, wl, spec, world, m, peaks, tf32):
    """The JSON line of one measured workload."""
    steps, stage = m["steps"], m["stage"]
    n, nq = m["n"], m["nq"]
    mean = lambda key, which: statistics.mean(s[key] for s in stage[which])  # noqa: E731
    sharded_join = spec["mode"] == "fit_query" and world > 1
    total_rows = spec["n"] if sharded_join else n * world
    fit_ms, hash_ms, scatter_ms = mean("total_ms", "fit"), mean("hash_ms", "fit"), mean("scatter_ms", "fit")
    q_ms, gather_ms = mean("total_ms", "query"), mean("gather_ms", "query")
    sf, sq = stage["fit"][-1], stage["query"][-1]
    passes = max(1, sf["sort_passes"])
    items, kb = sf["n_items"], 4 * sf["key_words"]
    roof = {}
    if spec["family"] == "minhash":
        nnz = m["nnz"]
        evals = float(nnz) * spec["L"] * spec["k"]
        hbytes = 4.0 * nnz + 4.0 * (n + 1) + 4.0 * n * spec["L"] * sf["key_words"]
        roof["hash"] = {"bound": "hbm", "achieved": hbytes / (hash_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "kernel": "minhash_kernel", "traffic": None,
                        "note": "integer-issue bound by nature: 4*nnz + 4*(n+1) + 4*n*L*NW bytes over the event "
                                "time; hash evaluations/s in hash_evals_per_s",
                        "hash_evals_per_s": evals / (hash_ms * 1e-3)}
    elif hash_ms > 0:
        flops = 2.0 * n * spec["d"] * spec["L"] * spec["k"]
        lo_frac = statistics.mean(s.get("hash_lo_fraction", 1.0) for s in stage["fit"])
        roof["hash"] = {"bound": "tensor", "achieved": flops / (hash_ms * 1e-3) / 1e12, "peak": tf32 / 3.0,
                        "unit": "TFLOP/s", "traffic": None,
                        "frac_fp32_equiv": flops / (hash_ms * 1e-3) / 1e12 / (tf32 / 3.0),
                        "frac_tensor_issue": flops * (2.0 + lo_frac) / (hash_ms * 1e-3) / 1e12 / tf32,
                        "mma_per_k_block": 2.0 + lo_frac,
                        "kernel": "project_tc_kernel" if sf["hash_path"] == 1 else "project_simt_kernel",
                        "note": "fp32-equivalent flop 2*n*d*H over the CUDA-event time of the projection "
                                "launch; peak = TF32 dense matmul measured in this run (8192^3) / 3 (3xTF32)",
                        "tf32_tflops_measured": tf32}
    if scatter_ms > 0:
        roof["sort"] = {"bound": "hbm", "achieved": items * (kb + 4) * 2.0 / (scatter_ms * 1e-3) / 1e9,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "kernel": "radix_scatter_kernel", "traffic": None,
                        "note": f"(key {kb} B + row id 4 B) read + written per item, one launch (the scatter of the "
                                f"last of {passes} passes) timed with CUDA events; peak {peaks['source']}"}
    dedupe_ms = mean("dedupe_ms", "query")
    if dedupe_ms > 0:
        roof["gather"] = {"bound": "hbm", "peak": peaks["hbm_gbs"], "unit": "GB/s", "traffic": None,
                          "achieved": 4.0 * (sq["raw_candidates"] + sq["unique_candidates"]) / (dedupe_ms * 1e-3) / 1e9,
                          "kernel": "dedupe kernel of the gather (chained rank / bitmap / warp path)",
                          "note": "4 B per raw candidate id read + 4 B per unique id written, over the CUDA-event "
                                  f"time of the dedupe launch alone; peak {peaks['source']}"}
    for key, r in roof.items():
        r["frac"] = r["achieved"] / r["peak"]
        traffic = NCU_TRAFFIC.get((wl, n), {}).get(key)
        r["traffic"] = traffic
        r["traffic_note"] = ("ncu DRAM bytes of one launch of this size (profiles/)" if traffic is not None
                             else "no ncu capture of a launch of this size")
    shares = {"hash": hash_ms if "hash" in roof else 0.0, "sort": scatter_ms * passes if "sort" in roof else 0.0,
              "gather": dedupe_ms if "gather" in roof else 0.0}
    dominant = roof[max(shares, key=shares.get)] if roof else None
    t_dev = m["t_dev"]
    in_bytes = m["in_bytes"]
    line = {
        "metric": METRICS[wl],
        "value": total_rows / (t_dev / steps), "unit": "rows/s",
        "n_gpus": world, "steps": steps, "warmup": m["warmup"], "ms_per_step": t_dev / steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if sharded_join else "weak", "vs_baseline": None,
        "dtype": "u32" if spec["family"] == "minhash" else "f32", "data": "synthetic",
        "config": config_of(wl, spec),
        "l2": (f"inputs ({in_bytes >> 20} MB per step) larger than L2, no flush" if in_bytes > (130 << 20)
               else f"inputs ({in_bytes >> 10} KB) fit L2: small configuration, no flush"),
        "parallelism": (f"row-sharded x{world}, peer-memory candidate exchange fused with the merge"
                        if world > 1 else "single GPU"),
        "hash_parameters": "generated by every fit inside the timed region (parameter cache off)",
        "cached_params": {"ms_per_step": m["t_cached"] / max(3, steps // 5) * 1e3,
                          "note": "same step with the per-handle parameter cache on"},
        "first_call_ms": m["first_call_ms"],
        "fit_rows_per_s": total_rows / ((fit_ms + mean("params_ms", "fit")) * 1e-3),
        "hash_rows_per_s": (total_rows / (hash_ms * 1e-3)) if hash_ms > 0 else None,
        "query_qps": (nq / (q_ms * 1e-3)) if q_ms > 0 else None,
        "stage_ms": {"params": mean("params_ms", "fit"), "fit_total": fit_ms, "hash": hash_ms,
                     "sort": mean("sort_ms", "fit"),
                     "sort_scatter_last_pass": scatter_ms, "build": mean("build_ms", "fit"),
                     "query_total": q_ms, "query_hash": mean("hash_ms", "query"),
                     "lookup": mean("lookup_ms", "query"), "gather": gather_ms, "gather_dedupe_kernel": dedupe_ms},
        "shape": {"buckets": sf["n_buckets"], "raw_candidates": sq["raw_candidates"],
                  "unique_candidates": sq["unique_candidates"], "key_words": sf["key_words"],
                  "elem_bytes": sf["elem_bytes"], "sort_passes": passes},
        "roofline": dominant, "roofline_all": roof,
        "e2e": {"value": total_rows / (m["t_e2e"] / steps), "unit": "rows/s",
                "ms_per_step": m["t_e2e"] / steps * 1e3,
                "h2d_bytes_per_step": int(m["h2d"]), "d2h_bytes_per_step": int(m["d2h"])},
        "gpu_launches": m["launches"], "clocks": m["clocks"],
    }
    if world > 1 and "x_push" in sq:
        line["exchange_ms"] = {key[2:]: mean(key, "query") for key in sq if key.startswith("x_")}
        line["exchange_ms"]["note"] = ("rank 0's host wall time per step of the exchange: all-gather of the per-query "
                                       "counts, positions, the push kernel (peer stores), closing barrier")
    if m["parity"] is not None:
        line["parity"] = m["parity"]
    if m["exchange_check"] is not None:
        line["exchange_check"] = m["exchange_check"]
    return line


def run_ours(args, wl, spec):
    import torch
    world, rank, local = dist_setup()
    device = torch.device(f"cuda:{local}")
    from culsh_b200 import sharded
    exchange = sharded.PeerExchange(device=local) if world > 1 else None
    m = run_workload(torch, args, wl, spec, world, rank, local, exchange, args.steps, args.warmup,
                     e2e=not args.skip_e2e, checks=not args.skip_checks)
    m["steps"], m["warmup"] = args.steps, args.warmup
    extra, extra_errors = {}, {}
    if wl == "c2" and args.rows is None and not args.no_extra:
        torch.cuda.empty_cache()
        for ew in ("c4", "c5"):
            try:
                em = run_workload(torch, args, ew, dict(WORKLOADS[ew]), world, rank, local, exchange, 5, 3,
                                  e2e=False, checks=False)
            except Exception as ex:  # the headline line must still be printed
                extra_errors[ew] = f"{type(ex).__name__}: {ex}"[:300]
                break
            em["steps"], em["warmup"] = 5, 3
            extra[ew] = em
            torch.cuda.empty_cache()
    if exchange is not None:
        exchange.close()
    if rank != 0:
        return
    peaks = load_peaks()
    tf32 = measure_tf32_peak(torch, device)
    line = line_of(torch, args, wl, spec, world, m, peaks, tf32)
    if extra:
        line["extra"] = {}
        for ew, em in extra.items():
            el = line_of(torch, args, ew, dict(WORKLOADS[ew]), world, em, peaks, tf32)
            line["extra"][ew] = {key: el[key] for key in ("metric", "value", "unit", "ms_per_step", "steps", "scaling",
                                                       "config", "stage_ms", "shape", "first_call_ms")}
    for ew, msg in extra_errors.items():
        line.setdefault("extra", {})[ew] = {"error": msg}
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_baseline(wl)
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


def run_reference(args, wl, spec):
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
    n, nq = spec["n"], spec["nq"]
    base = {"metric": METRICS[wl], "unit": "rows/s", "impl": "reference",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u32" if spec["family"] == "minhash" else "f32",
            "data": "synthetic", "config": config_of(wl, spec)}
    if ref is None or not have_gpu:
        cb = cpu_baseline(wl)
        base.update({"value": cb["value"], "ms_per_step": None, "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "rows/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    # upstream's CUDA build, driven through its own pybind11 API with torch tensors
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device(f"cuda:{local}")
    Xd, Qd = make_inputs(torch, device, 0, wl, spec)
    torch.cuda.synchronize()
    core = make_core(ref, spec)
    batch = nq if wl == "c2" else (100_000 if wl == "c5" else None)

    def to_dev(h):
        if h is None:
            return None
        if isinstance(h, tuple):
            return tuple(to_dev(x) for x in h)
        return torch.from_numpy(h).to(device, non_blocking=True)

    keep = {}

    def step(X, Q, host):
        if host:
            X, Q = to_dev(X), to_dev(Q)
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        if spec["mode"] == "fit_query":
            # upstream's Python layer turns fit_query(batch_size=b) into fit + batched query
            # (python/culsh/rp_lsh.py:145-147); the unbatched call needs ~46 GB of projection scratch
            ix = core.fit_float(X, n, spec["d"])
            t1 = time.perf_counter()
            cand = core.query_float(X, n, ix, batch)
        else:
            ix = core_fit(core, spec, X)
            t1 = time.perf_counter()
            cand = core_query(core, spec, Q, ix, batch)
        t2 = time.perf_counter()
        keep["cand"] = cand
        return t1 - t0, t2 - t1, (read_back(cand) if host else 0)

    for _ in range(args.warmup):
        step(Xd, Qd, False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    fits, queries = [], []
    for _ in range(args.steps):
        f, q, _ = step(Xd, Qd, False)
        fits.append(f)
        queries.append(q)
    torch.cuda.synchronize()
    t_dev = time.perf_counter() - t0
    cand = keep.pop("cand")
    parity = {"unique_candidates": int(cand.n_total_candidates),
              "csr_checksum": csr_checksum(torch, cand.get_indices(), cand.get_offsets(), device)}
    del cand
    e2e = {"value": None, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not args.skip_e2e:
        Xh, Qh = to_pinned_host(torch, Xd), to_pinned_host(torch, Qd)
        step(Xh, Qh, True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        d2h = 0
        for _ in range(args.steps):
            _, _, d2h = step(Xh, Qh, True)
        torch.cuda.synchronize()
        t_e2e = time.perf_counter() - t0
        e2e = {"value": n / (t_e2e / args.steps), "unit": "rows/s", "ms_per_step": t_e2e / args.steps * 1e3,
               "h2d_bytes_per_step": int(nbytes_of(Xh) + nbytes_of(Qh)), "d2h_bytes_per_step": int(d2h)}
    base.update({
        "value": n / (t_dev / args.steps), "ms_per_step": t_dev / args.steps * 1e3,
        "fit_rows_per_s": n / statistics.mean(fits),
        "query_qps": (nq or n) / statistics.mean(queries),
        "stage_ms": {"fit_total": statistics.mean(fits) * 1e3, "query_total": statistics.mean(queries) * 1e3},
        "cpu_baseline": {"value": n / (t_dev / args.steps), "unit": "rows/s", "cores": 0, "kind": "reference",
                         "sample": "full workload; upstream cuLSH CUDA build (its cuBLAS/CUB kernels compiled for "
                                   "sm_100) on one B200 - upstream has no CPU implementation of this path"},
        "e2e": e2e, "reference_device": "B200 (upstream CUDA build)", "parity": parity,
    })
    if world > 1:
        base["note"] = "upstream is single-GPU: rank 0 runs one shard"
    print(json.dumps(base))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c2")
    ap.add_argument("--rows", type=int, default=None, help="rows per GPU (default: the workload's)")
    ap.add_argument("--queries", type=int, default=None)
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: no host-input leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling runs: no CPU baseline leg")
    ap.add_argument("--skip-checks", action="store_true", help="profiling runs: no parity / exchange checks")
    ap.add_argument("--no-extra", action="store_true",
                    help="default workload only: leave out the short c4 / c5 runs reported under `extra`")
    ap.add_argument("--reference-cpu", action="store_true",
                    help="reference arm: time the NumPy restatement on the host cores instead of "
                         "upstream's CUDA build")
    args = ap.parse_args()
    spec = dict(WORKLOADS[args.workload])
    if args.rows:
        spec["n"] = args.rows
    if args.queries is not None and spec["nq"]:
        spec["nq"] = args.queries
    if args.impl == "reference":
        run_reference(args, args.workload, spec)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args, args.workload, spec)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
