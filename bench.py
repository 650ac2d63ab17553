"""Headline benchmark: IVF-SQ8 search QPS on a synthetic stand-in for Deep-10M.

Workload (the configuration the headline metric is quoted on): base 10,000,000 x 96 fp32 drawn from a Gaussian
mixture of 16,384 centres (uniform[-1,1], sigma 0.15, seed 2), SQ8 codes, nlist 16,384, nprobe 64,
10,000 queries from the same mixture (seed 3), k = 10, L2.  The dataset named by the reference's
documentation is not available offline; this seeded synthetic set has its shape.

A step is one search of the whole 10,000-query batch through the C ABI (vb200_ivf_search):
routing, pair grouping, list scan with fused top-k, merge.  `value` times it with queries and
results resident in HBM; `e2e` times the same call with pinned host buffers, so the host<->device
copies are inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

The default line also carries, outside its timed region:
  pruning_off      the same steps with the scan's exact list pruning switched off (every probed list is scanned)
  sweep            nprobe 32 and 128 of the same configuration, ids checked against the CPU scan on a sample
  second_base      the same index shape over a mixture that does not mirror nlist (overlapping components)
  extra_workloads  short runs of the other configurations (k-means training, bf16 BruteForce, IVF-RaBitQ with
                   rerank), each with its own roofline, CPU baseline and a parity check against the oracle

Each of the other configurations can also be the line itself:

    python bench.py --workload kmeans       # k-means training, 1,000,000 x 128 against 4,096 centroids
    python bench.py --workload bruteforce   # exact bf16 inner-product kNN, one GPU's 6,250,000 x 768 shard
    python bench.py --workload rabitq       # IVF-RaBitQ 1,000,000 x 960, nlist 4,096, nprobe 64, k 100, rerank 4k
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
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

N_BASE = 10_000_000
DIM = 96
NLIST = 16_384
NPROBE = 64
N_QUERY = 10_000
K = 10
N_CENTRES = 16_384
SIGMA = 0.15
TRAIN_ROWS = 64 * NLIST          # the reference's default train_sample_count: max(65536, 64 * nlist)
KMEANS_ITERS = 25                # hard-coded in IVFNearestPartition::Train
FALLBACK_HBM_GBS = 6650.0
FP32_FMA_PEAK_T = 148 * 128 * 1.965e9 / 1e12   # fp32 FMA/s of one B200 in units of 1e12: SMs x lanes x max SM clock
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture of the scan kernel on the
# 2,000,000-row case) per byte of codes the kernel reported as read in that capture: lists that several
# tiles scan are L2 hits after the first, so the ratio is below one.  `traffic` is this ratio times the
# code bytes the timed run itself reports, per rank.
SCAN_DRAM_PER_CODE_BYTE = 0.79   # 116.5 MB of DRAM traffic for 148.3 MB of codes fetched
WORKLOAD_NAME = "IVF-SQ8 search, 10M x 96, nlist 16384, nprobe 64, 10000 queries, k 10"
METRIC_NAME = "QPS at nprobe=64, IVF-SQ8 10Mx96, k=10"


def env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


def scaled(n: int) -> int:
    """VB200_BENCH_SCALE shrinks the workload for dry runs; the default 1.0 is the real config."""
    s = float(os.environ.get("VB200_BENCH_SCALE", "1.0"))
    return max(1, int(n * s))


def host_threads() -> int:
    """Cores this process may run on.  Passed to the CPU arm explicitly: under torchrun the
    environment carries OMP_NUM_THREADS=1, which must not make the CPU baseline single-core."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def oracle_module():
    from oracle import pyoracle as O

    O.set_threads(host_threads())
    return O


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    out = {"hbm_gbs": FALLBACK_HBM_GBS, "hbm_kind": "fallback", "tflops": 1590.0, "tflops_kind": "fallback"}
    if p.exists():
        try:
            j = json.loads(p.read_text())
            out.update(hbm_gbs=float(j["hbm_gbs"]), hbm_kind="measured", tflops=float(j["bf16_tflops"]),
                       tflops_kind="measured (burst)")
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.thread = None
        self.t_begin = None

    def start(self) -> None:
        """Starts nvidia-smi in its sampling loop and waits for its first line (its start-up takes driver
        locks for tens of milliseconds, which must not fall into a timed region)."""
        if env_int("VB200_BENCH_NO_CLOCKS", 0):   # to measure what the sampling itself costs
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        deadline = time.time() + 3.0
        while not self.lines and time.time() < deadline:
            time.sleep(0.01)
        self.t_begin = time.time()

    def begin(self) -> None:
        """Marks the start of the timed region (start() ran before the warm-up)."""
        self.t_begin = time.time()

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self) -> dict:
        """Ends the sampling; the samples taken since start() returned (the timed region) are summarised,
        or, if the region was shorter than one sampling period, the ones on either side of it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t_end = time.time()
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [text for t, text in self.lines if self.t_begin is not None and self.t_begin <= t <= t_end]
        around = [text for t, text in self.lines
                  if self.t_begin is not None and self.t_begin - 0.15 <= t <= t_end + 0.15]
        lines = inside or around or [text for _, text in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "samples_inside_timed_region": len(inside)}


class Ctx:
    """Rank, device and the timing rule shared by every workload: K steps between a barrier +
    synchronize on both sides, device time from CUDA events on the launching (default) stream, max
    over ranks."""

    def __init__(self):
        import torch

        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.device)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist_mod

            self.dist = dist_mod
            self.dist.init_process_group("nccl", device_id=self.device)
        self.peaks = measured_peaks()
        self._comm = None

    @property
    def comm(self):
        """The library's own communicator (vb200_comm_init); torch.distributed only carries its id."""
        if self._comm is None and self.world > 1:
            from vsag_b200 import parallel

            self._comm = parallel.Comm(self.dist, self.rank, self.world, self.device)
        return self._comm

    def timed(self, fn, steps: int) -> float:
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def close(self) -> None:
        if self._comm is not None:
            self._comm.close()
        if self.world > 1:
            self.dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# IVF-SQ8 workload
# ------------------------------------------------------------------------------------------------
def make_data(device, n_base: int, n_query: int, n_centres: int = N_CENTRES, sigma: float = SIGMA, seed: int = 2):
    """Seeded Gaussian-mixture base rows and queries, generated on the device in slices."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    n_centres = max(16, scaled(n_centres))   # a scaled-down dry run keeps rows per mixture component
    centres = torch.rand((n_centres, DIM), generator=g, device=device) * 2.0 - 1.0
    base = torch.empty((n_base, DIM), dtype=torch.float32, device=device)
    step = 1_000_000
    for b in range(0, n_base, step):
        e = min(n_base, b + step)
        which = torch.randint(0, n_centres, (e - b,), generator=g, device=device)
        base[b:e] = centres[which] + sigma * torch.randn((e - b, DIM), generator=g, device=device)
    gq = torch.Generator(device=device)
    gq.manual_seed(seed + 1)
    which = torch.randint(0, n_centres, (n_query,), generator=gq, device=device)
    queries = centres[which] + sigma * torch.randn((n_query, DIM), generator=gq, device=device)
    return base, queries.contiguous()


def build_index(engine, base, nlist: int, rank: int, world: int, dist):
    """Trains on rank 0 (centroid sums use float atomics, so ranks would otherwise disagree in the
    last bit), shares the model, and lets every rank add the rows of the lists it owns."""
    import torch

    ix = engine.IvfHandle(DIM, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    if world > 1:
        ix.set_shard(rank, world)
    train_rows = min(base.shape[0], scaled(TRAIN_ROWS))
    centroids = torch.empty((nlist, DIM), dtype=torch.float32, device=base.device)
    model = torch.empty((2, DIM), dtype=torch.float32, device=base.device)
    if rank == 0:
        trainer = engine.IvfHandle(DIM, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
        # a strided sample stands in for the reference's reservoir sample of the same size
        stride = max(1, base.shape[0] // train_rows)
        sample = base[::stride][:train_rows].contiguous()
        # k-means++ seeding as KMeansCluster::Run does by default, then the Lloyd iterations
        seeds = engine.kmeans_init(sample, nlist, seed=47)
        trainer.train(sample, iters=env_int("VB200_BENCH_KMEANS_ITERS", KMEANS_ITERS), init=seeds)
        del seeds
        centroids.copy_(torch.from_numpy(trainer.get_centroids()))
        lower, diff = trainer.get_sq8_model()
        model[0].copy_(torch.from_numpy(lower))
        model[1].copy_(torch.from_numpy(diff))
        trainer.close()
        del sample
    if world > 1:
        dist.broadcast(centroids, src=0)
        dist.broadcast(model, src=0)
    ix.set_centroids(centroids)
    ix.set_sq8_model(model[0].contiguous(), model[1].contiguous())
    ids = torch.arange(base.shape[0], dtype=torch.int64, device=base.device)
    ix.add(base, ids)
    return ix


def recall_at_k(engine, base, queries, got_ids, sample: int, bf=None) -> float:
    """recall@k of the first `sample` queries against exact fp32 search on the same base."""
    import torch

    own = bf is None
    if own:
        bf = engine.BfHandle(DIM, engine.METRIC_L2, engine.QUANT_FP32)
        ids = torch.arange(base.shape[0], dtype=torch.int64, device=base.device)
        bf.add(base, ids)
    exact, _ = bf.search(queries[:sample].contiguous(), K)
    if own:
        bf.close()
    exact = exact.cpu().numpy()
    got = got_ids[:sample].cpu().numpy() if hasattr(got_ids, "cpu") else got_ids[:sample]
    hits = sum(len(set(a.tolist()) & set(b.tolist())) for a, b in zip(got, exact))
    return hits / float(sample * K)


# ---- CPU arm: the reference's scan loop on the host cores --------------------------------------
def cpu_scan_setup(ix, queries_host: np.ndarray, nprobe: int):
    """Host copies of the inverted file plus the probe lists, for the CPU scan."""
    sizes, codes, inner = ix.get_lists()
    off = np.zeros(sizes.size + 1, np.int64)
    np.cumsum(sizes, out=off[1:])
    lower, diff = ix.get_sq8_model()
    probes, _ = ix.route(queries_host, nprobe)
    return dict(codes=codes, off=off, inner=inner, lower=lower, diff=diff, probes=probes, sizes=sizes)


def cpu_scan_run(host: dict, queries_host: np.ndarray, count: int, probes=None):
    """Times the reference's per-query bucket scan (32-code blocks + bounded heap) over `count`
    queries, one query per worker thread on every core.  The distance kernel is the reference's own
    compiled SQ8ComputeL2Sqr when oracle/_ref is present ("reference"), else the oracle's scalar
    restatement ("port").  Routing is not timed: the probe lists come from the engine, which
    favours the CPU arm (the reference routes through a graph search)."""
    import ctypes as C

    O = oracle_module()
    R = O.ref()
    fn = C.cast(R.ref_SQ8ComputeL2Sqr, C.c_void_p) if R is not None else None
    kind = "reference" if R is not None else "port"
    q = np.ascontiguousarray(queries_host[:count])
    probes = np.ascontiguousarray((host["probes"] if probes is None else probes)[:count])
    threads = host_threads()
    t0 = time.perf_counter()
    ids, dists = O.ivf_sq8_search(host["codes"], host["off"], host["inner"], host["lower"], host["diff"], q,
                                  probes, K, metric=0, fn=fn, nthreads=threads)
    dt = time.perf_counter() - t0
    return count / dt, kind, threads, dt, ids, dists


def run_reference_arm(args) -> None:
    """`--impl reference`: the reference's CPU implementation of the scan on this box's cores."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from vsag_b200 import engine

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    n_base, n_query, nlist = scaled(N_BASE), scaled(N_QUERY), max(16, scaled(NLIST))
    base, queries = make_data(device, n_base, n_query)
    # The index (codes, lists) is an input of the measurement; it is built with the engine because
    # the reference library cannot be built offline.  Only the CPU scan below is timed.
    ix = build_index(engine, base, nlist, 0, 1, None)
    qh = queries.cpu().numpy()
    host = cpu_scan_setup(ix, qh, min(NPROBE, nlist))
    sample = min(n_query, env_int("VB200_CPU_SAMPLE", 2000))
    for _ in range(max(1, args.warmup)):
        cpu_scan_run(host, qh, min(sample, 200))
    times, qps, kind, cores = [], 0.0, "port", 1
    for _ in range(args.steps):
        qps, kind, cores, dt, _, _ = cpu_scan_run(host, qh, sample)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = sample / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC_NAME, "value": value,
        "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME,
                   "n_base": n_base, "dim": DIM, "nlist": nlist, "nprobe": min(NPROBE, nlist), "n_query": n_query, "k": K},
        "cpu_baseline": {"value": value, "unit": "queries/s", "cores": cores, "kind": kind,
                         "sample": f"{sample} of {n_query} queries per step, scan + top-k only "
                                   "(probe lists and the inverted file come from the engine), one query per thread"},
        "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def scan_probe(ix, step_fn, repeats: int):
    """Kernel-only figures of the scan from a few extra (untimed-for-value) steps: device time of the
    scan launches from the events the library records around them, the logical scan volume and the
    code bytes actually read."""
    ms, logical, read = [], [], []
    for _ in range(repeats):
        step_fn()
        ms.append(ix.last_scan_ms())
        logical.append(ix.last_scan_bytes())
        read.append(ix.last_scanned_bytes())
    return float(np.mean(ms)), float(np.mean(logical)), float(np.mean(read))


def scan_roofline(peaks: dict, kernel_ms: float, logical: float, read: float, unique_bytes: float | None,
                  pruned: bool = True) -> dict:
    """Roofline of the scan kernel on the bytes it fetched, with the logical figure beside it.

    read     pairs scanned x list length x code size: what the kernel's loads requested (a list scanned
             by several query tiles counts once per tile; most of those re-reads are L2 hits)
    logical  the reference's scan volume: every (query, probed list) pair, pruned or not
    On the tensor-core kernel a (query, code byte) is three int8 multiply-adds; `read` is that count / 3."""
    peak = peaks["hbm_gbs"]
    sec = kernel_ms / 1e3
    achieved = read / sec / 1e9
    out = {"bound": "hbm",
           "kernel": ("ivf_sq8_first_kernel (first phase) + ivf_sq8_scan_tc_kernel (second phase)" if pruned
                      else "ivf_sq8_scan_tc_kernel"),
           "achieved": achieved, "peak": peak, "unit": "GB/s",
           "frac": achieved / peak, "peak_source": peaks["hbm_kind"], "kernel_ms": kernel_ms,
           # the captured ratio belongs to the pruned step; no capture exists of the unpruned one
           "traffic": SCAN_DRAM_PER_CODE_BYTE * read if pruned else None,
           "traffic_source": f"{SCAN_DRAM_PER_CODE_BYTE} DRAM bytes per code byte read (ncu capture of the 2M-row "
                             "case, both scan launches of a step) x code_bytes_read of this run and rank",
           "code_bytes_read": read, "algorithmic_bytes": logical, "algorithmic_gbs": logical / sec / 1e9,
           "algorithmic_frac": logical / sec / 1e9 / peak,
           "note": "achieved = code bytes the kernel read / its device time; algorithmic_* counts every probed "
                   "list of every query as the reference's scan reads them, pruned or not"}
    if unique_bytes is not None:
        out["unique_list_bytes"] = unique_bytes
    return out


INT8_TENSOR_PEAK_TOPS = 4500.0   # nominal dense int8 rate of one B200 (no measured figure exists for kind::i8)


def fma_roofline(kernel_ms: float, macs: float) -> dict:
    """The scan's arithmetic against the tensor pipe: every (query, code byte) scanned is three int8
    multiply-adds (the three terms of the query weight) on `tcgen05.mma.kind::i8`."""
    t = 6.0 * macs / (kernel_ms / 1e3) / 1e12
    return {"bound": "tensor (int8)", "achieved": t, "peak": INT8_TENSOR_PEAK_TOPS, "unit": "TOP/s",
            "frac": t / INT8_TENSOR_PEAK_TOPS, "peak_source": "nominal dense int8",
            "note": "2 x 3 int8 terms per (query, code byte) scanned; work items are padded to 32 queries, so the "
                    "pipe executes more than this"}


def run_ivf_sq8(args, ctx: Ctx) -> dict:
    import torch

    from vsag_b200 import engine

    world, rank, device, dist = ctx.world, ctx.rank, ctx.device, ctx.dist
    n_base, n_query, nlist = scaled(N_BASE), scaled(N_QUERY), max(16, scaled(NLIST))
    nprobe = min(NPROBE, nlist)
    base, queries = make_data(device, n_base, n_query)
    ix = build_index(engine, base, nlist, rank, world, dist)
    if not env_int("VB200_BENCH_PRUNING", 1):
        ix.set_list_pruning(False)     # profiling aid: the timed region itself runs unpruned

    out_ids = torch.empty((n_query, K), dtype=torch.int64, device=device)
    out_d = torch.empty((n_query, K), dtype=torch.float32, device=device)
    sharded = None
    if world > 1:
        from vsag_b200 import parallel

        sharded = parallel.ShardedIvfSearch(ix, n_query, K, world, device, dist, rank, comm=ctx.comm)

    def step_device(np_=nprobe):
        if world == 1:
            ix.search(queries, K, np_, out=(out_ids, out_d))
        else:
            # one C-ABI call per rank: every rank routes its slice of the batch, the probe lists are
            # all-gathered, every rank scans the probed lists it owns, and the per-shard top-k are
            # all-gathered over NVLink and merged locally
            sharded.search(queries, np_, 2.0, out_ids, out_d)

    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()              # before the warm-up: its start-up must not fall into the timed region
    for _ in range(args.warmup):
        step_device()
    torch.cuda.synchronize()
    sampler.begin()
    launches0 = engine.kernel_launches()
    torch.cuda.nvtx.range_push("timed_steps")   # lets a profiler pick out the timed region
    total_ms = ctx.timed(step_device, args.steps)
    torch.cuda.nvtx.range_pop()
    launches = engine.kernel_launches() - launches0
    clocks = sampler.stop() if rank == 0 else None
    kernel_ms, logical, read = scan_probe(ix, step_device, min(5, args.steps))
    ms_per_step = total_ms / args.steps
    value = n_query / (ms_per_step / 1e3)

    # end to end: pinned host queries in, host results out, through the same C-ABI call
    q_host = torch.empty((n_query, DIM), dtype=torch.float32, pin_memory=True)
    q_host.copy_(queries)
    ids_host = torch.empty((n_query, K), dtype=torch.int64, pin_memory=True)
    d_host = torch.empty((n_query, K), dtype=torch.float32, pin_memory=True)

    def step_e2e():
        if world == 1:
            ix.search(q_host, K, nprobe, out=(ids_host, d_host))
        else:
            sharded.search(q_host, nprobe, 2.0, ids_host, d_host)   # host buffers through the same C-ABI call

    for _ in range(2):
        step_e2e()
    e2e_ms = ctx.timed(step_e2e, args.steps) / args.steps
    e2e_value = n_query / (e2e_ms / 1e3)

    per_rank = torch.tensor([kernel_ms, logical, read], dtype=torch.float64, device=device)
    if world > 1:
        gathered = [torch.empty_like(per_rank) for _ in range(world)]
        dist.all_gather(gathered, per_rank)
        per_rank_rows = [g.cpu().tolist() for g in gathered]
    else:
        per_rank_rows = [per_rank.cpu().tolist()]

    if rank != 0:
        return {}
    roof = scan_roofline(ctx.peaks, kernel_ms, logical, read, None)
    roof["all_ranks_algorithmic_bytes"] = float(sum(r[1] for r in per_rank_rows))
    if world > 1:
        roof["per_rank"] = [{"kernel_ms": r[0], "code_bytes_read": r[2],
                             "traffic": SCAN_DRAM_PER_CODE_BYTE * r[2]} for r in per_rank_rows]
    line = {
        "metric": METRIC_NAME, "value": value, "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME,
                   "n_base": n_base, "dim": DIM, "nlist": nlist, "nprobe": nprobe, "n_query": n_query,
                   "k": K, "parallelism": f"lists sharded over {world} GPU(s)",
                   "l2_policy": "codes (960 MB) exceed the 126 MB L2; no flush between steps"},
        "e2e": {"value": e2e_value, "unit": "queries/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": n_query * DIM * 4, "d2h_bytes_per_step": n_query * K * 12},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roof,
        "roofline_tensor": fma_roofline(kernel_ms, read),
    }
    if world > 1 or env_int("VB200_BENCH_SKIP_EXTRAS", 0):
        return line

    # ---- everything below is outside the timed regions of the headline ----
    sample = min(n_query, env_int("VB200_CPU_SAMPLE", 2000))
    rsample = min(n_query, env_int("VB200_RECALL_SAMPLE", 1000))
    qh = q_host.numpy()
    bf = engine.BfHandle(DIM, engine.METRIC_L2, engine.QUANT_FP32)
    bf.add(base, torch.arange(base.shape[0], dtype=torch.int64, device=device))
    line["config"]["recall_at_10"] = recall_at_k(engine, base, queries, out_ids, rsample, bf)
    host = cpu_scan_setup(ix, qh, nprobe)
    cpu_scan_run(host, qh, min(sample, 100))
    qps, kind, cores, dt, cpu_ids, _ = cpu_scan_run(host, qh, sample)
    line["cpu_baseline"] = {"value": qps, "unit": "queries/s", "cores": cores, "kind": kind,
                            "sample": f"{sample} of {n_query} queries, scan + top-k only (probe lists and the "
                                      f"inverted file come from the engine), one query per thread, {dt:.2f} s",
                            "ids_agree_with_gpu": float(np.mean(cpu_ids == ids_host.numpy()[:sample]))}
    sizes = host["sizes"]

    def unique_bytes(probes: np.ndarray) -> float:
        lists = np.unique(probes[probes >= 0])
        return float(sizes[lists].sum()) * DIM

    # the same steps with the exact list pruning off: every probed list of every query is scanned,
    # which is the reference's schedule of work and the figure that judges the kernel, not the data
    ix.set_list_pruning(False)
    for _ in range(2):
        step_device()
    off_steps = max(3, min(args.steps, 10))
    off_ms = ctx.timed(step_device, off_steps) / off_steps
    k_ms, lg, rd = scan_probe(ix, step_device, 3)
    off_ids = out_ids.cpu().numpy()
    ix.set_list_pruning(True)
    uniq = unique_bytes(host["probes"])
    off_roof = scan_roofline(ctx.peaks, k_ms, lg, rd, uniq, pruned=False)
    line["pruning_off"] = {
        "ms_per_step": off_ms, "value": n_query / (off_ms / 1e3), "kernel_ms": k_ms,
        "frac": uniq / (k_ms / 1e3) / 1e9 / ctx.peaks["hbm_gbs"],
        "frac_note": "probed lists' codes counted once each (the bytes that must cross HBM) / kernel time / HBM peak",
        "frac_pairs": off_roof["frac"], "frac_tensor_int8": fma_roofline(k_ms, rd)["frac"],
        "code_bytes_read": rd, "unique_list_bytes": uniq,
        "ids_agree_with_cpu": float(np.mean(cpu_ids == off_ids[:sample])),
        "ids_agree_with_pruned": float(np.mean(off_ids == ids_host.numpy())),
    }

    # nprobe 32 and 128 of the same configuration
    sweep = []
    ssample = min(sample, 500)
    for np_ in (32, 128):
        np_ = min(np_, nlist)
        for _ in range(2):
            step_device(np_)
        s_steps = max(3, min(args.steps, 10))
        s_ms = ctx.timed(lambda: step_device(np_), s_steps) / s_steps
        k_ms, lg, rd = scan_probe(ix, lambda: step_device(np_), 3)
        got = out_ids.cpu().numpy()
        probes, _ = ix.route(qh[:ssample], np_)
        _, _, _, _, want_ids, _ = cpu_scan_run(host, qh, ssample, probes=probes)
        entry = {"nprobe": np_, "ms_per_step": s_ms, "value": n_query / (s_ms / 1e3), "kernel_ms": k_ms,
                 "recall_at_10": recall_at_k(engine, base, queries, out_ids, rsample, bf),
                 "ids_agree_with_cpu": float(np.mean(want_ids == got[:ssample])), "ids_sample": ssample,
                 "roofline": scan_roofline(ctx.peaks, k_ms, lg, rd, None)}
        sweep.append(entry)
    line["config"]["sweep"] = sweep
    bf.close()
    del bf, host, cpu_ids

    # a second base that does not mirror the index: 1,024 overlapping components (sigma 0.4) under
    # the same 16,384 lists, so a query's neighbours spread over many lists and little can be pruned
    ix.close()
    del base, queries, ix
    torch.cuda.empty_cache()
    line["second_base"] = second_base_run(args, ctx, engine, n_base, n_query, nlist, nprobe)
    return line


def second_base_run(args, ctx: Ctx, engine, n_base: int, n_query: int, nlist: int, nprobe: int) -> dict:
    import torch

    device = ctx.device
    base, queries = make_data(device, n_base, n_query, n_centres=1024, sigma=0.4, seed=12)
    ix = build_index(engine, base, nlist, 0, 1, None)
    out_ids = torch.empty((n_query, K), dtype=torch.int64, device=device)
    out_d = torch.empty((n_query, K), dtype=torch.float32, device=device)

    def step():
        ix.search(queries, K, nprobe, out=(out_ids, out_d))

    for _ in range(3):
        step()
    steps = max(3, min(args.steps, 10))
    ms = ctx.timed(step, steps) / steps
    k_ms, lg, rd = scan_probe(ix, step, 3)
    got = out_ids.cpu().numpy()
    qh = queries.cpu().numpy()
    host = cpu_scan_setup(ix, qh, nprobe)
    ssample = min(n_query, 500)
    _, kind, cores, dt, want_ids, _ = cpu_scan_run(host, qh, ssample)
    uniq = float(host["sizes"][np.unique(host["probes"])].sum()) * DIM
    out = {"data": "10M x 96 from 1,024 components, sigma 0.4 (seed 12): components overlap and do not match nlist",
           "ms_per_step": ms, "value": n_query / (ms / 1e3), "kernel_ms": k_ms,
           "recall_at_10": recall_at_k(engine, base, queries, out_ids, min(n_query, 500)),
           "ids_agree_with_cpu": float(np.mean(want_ids == got[:ssample])), "ids_sample": ssample,
           "cpu_qps": ssample / dt, "cpu_cores": cores, "cpu_kind": kind,
           "roofline": scan_roofline(ctx.peaks, k_ms, lg, rd, uniq),
           "frac_tensor_int8": fma_roofline(k_ms, rd)["frac"],
           "pruned_share_of_pairs": 1.0 - rd / lg if lg > 0 else None}
    ix.close()
    return out


# ------------------------------------------------------------------------------------------------
# dense workloads (tensor-core kernels) and IVF-RaBitQ
# ------------------------------------------------------------------------------------------------
def run_kmeans(args, ctx: Ctx, steps: int, warmup: int) -> dict:
    """k-means training, 1,000,000 x 128 rows against 4,096 centroids initialised from the first rows.  A step
    is one Lloyd iteration (assignment + centroid update).  Under torchrun the ranks are replicas."""
    import torch

    from vsag_b200 import engine

    world, rank, device = ctx.world, ctx.rank, ctx.device
    n, dim, k = scaled(1_000_000), 128, max(64, scaled(4096))
    g = torch.Generator(device=device)
    g.manual_seed(1 + rank)
    centres = torch.rand((k, dim), generator=g, device=device) * 2.0 - 1.0
    x = centres[torch.randint(0, k, (n,), generator=g, device=device)]
    x = (x + 0.1 * torch.randn((n, dim), generator=g, device=device)).contiguous()
    seeds = x[:k].clone()
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    engine.kmeans_train(x, seeds, warmup)                      # warm-up iterations
    launches0 = engine.kernel_launches()
    sampler.begin()
    torch.cuda.nvtx.range_push("timed_steps")
    ms = ctx.timed(lambda: engine.kmeans_train(x, seeds, steps), 1) / steps
    torch.cuda.nvtx.range_pop()
    clocks = sampler.stop() if rank == 0 else None
    launches = engine.kernel_launches() - launches0
    x_host = torch.empty((n, dim), dtype=torch.float32, pin_memory=True)
    x_host.copy_(x)
    seeds_host = seeds.cpu().numpy()
    e2e_ms = ctx.timed(lambda: engine.kmeans_train(x_host, seeds_host, steps), 1) / steps
    flops = 2.0 * n * k * dim
    peak, peak_kind = ctx.peaks["tflops"], ctx.peaks["tflops_kind"]
    line = {
        "metric": "k-means Lloyd iterations, 1M x 128 rows against 4,096 centroids", "value": world * n / (ms / 1e3),
        "unit": "rows assigned/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16x3 (split fp32), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "k-means training: one step = one Lloyd iteration (assignment + centroid update)",
                   "rows": n, "dim": dim, "centroids": k, "init": "first rows",
                   "l2_policy": "points (512 MB) exceed the 126 MB L2; no flush between iterations",
                   "parallelism": f"{world} independent replica(s)"},
        "e2e": {"value": world * n / (e2e_ms / 1e3), "unit": "rows assigned/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": n * dim * 4 // steps, "d2h_bytes_per_step": (k * dim * 4 + n * 4) // steps},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "tc_candidates_kernel<0> (assignment)", "achieved": flops / (ms / 1e3) / 1e12,
                     "peak": peak, "unit": "TFLOP/s", "frac": flops / (ms / 1e3) / 1e12 / peak, "peak_source": peak_kind,
                     "traffic": None,
                     "note": "achieved = 2*rows*centroids*dim per iteration over the whole iteration's time; the kernel "
                             "issues three bf16 MMAs per product (hi*hi, hi*lo, lo*hi)"},
    }
    if rank == 0 and not env_int("VB200_BENCH_SKIP_EXTRAS", 0):
        # parity, iteration by iteration: the labels of a row sample against the oracle's assignment to
        # the same centroids (KMeansCluster::find_nearest_one_with_blas restated), then the engine's update
        O = oracle_module()
        sample = min(n, env_int("VB200_KMEANS_CPU_SAMPLE", 10000))
        xs = x[:sample].cpu().numpy()
        c = seeds_host.copy()
        iters = min(steps, 10)
        agree, cpu_s = [], 0.0
        for it in range(iters):
            labels = engine.kmeans_assign(x, c)
            t0 = time.perf_counter()
            want, _ = O.kmeans_assign(xs, c)
            cpu_s += time.perf_counter() - t0
            agree.append(float(np.mean(labels[:sample].cpu().numpy() == want)))
            c, _ = engine.kmeans_update(x, labels, k, it)
        line["parity"] = {"labels_agree_with_oracle_per_iteration": agree, "rows_sampled": sample, "iterations": iters}
        line["cpu_baseline"] = {"value": sample * iters / cpu_s, "unit": "rows assigned/s", "cores": host_threads(),
                                "kind": "port", "sample": f"assignment of {sample} of {n} rows, {iters} iterations, {cpu_s:.2f} s"}
    return line


def run_bruteforce(args, ctx: Ctx, steps: int, warmup: int) -> dict:
    """bf16 inner-product BruteForce search: every rank holds a 6,250,000 x 768 row range of one base (eight ranks
    hold the whole 50,000,000-row configuration), 10,000 queries, k 100; partial top-k merged after an all-gather."""
    import torch

    from vsag_b200 import engine, parallel

    world, rank, device, dist = ctx.world, ctx.rank, ctx.device, ctx.dist
    n, dim, nq, k = scaled(6_250_000), 768, max(128, scaled(10_000)), 100
    ix = engine.BfHandle(dim, engine.METRIC_IP, engine.QUANT_BF16)
    g = torch.Generator(device=device)
    g.manual_seed(6 + rank)
    first_rows = None
    for b in range(0, n, 500_000):
        c = min(500_000, n - b)
        rows = torch.randn((c, dim), generator=g, device=device)
        rows = (rows / rows.norm(dim=1, keepdim=True)).contiguous()
        if b == 0:
            first_rows = rows[: min(c, 200_000)].clone()
        ix.add(rows, torch.arange(rank * n + b, rank * n + b + c, dtype=torch.int64, device=device))
    del rows
    gq = torch.Generator(device=device)
    gq.manual_seed(7)
    q = torch.randn((nq, dim), generator=gq, device=device)
    q = (q / q.norm(dim=1, keepdim=True)).contiguous()
    out_ids = torch.empty((nq, k), dtype=torch.int64, device=device)
    out_d = torch.empty((nq, k), dtype=torch.float32, device=device)
    comm = ctx.comm

    def step(queries=q, ids=out_ids, dists=out_d):
        if world == 1:
            ix.search(queries, k, out=(ids, dists))
        else:
            # one C-ABI call: this rank's rows, an all-gather of the packed per-rank top-k, the merge
            ix.search_sharded(comm, queries, k, out=(ids, dists))

    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(warmup):
        step()
    launches0 = engine.kernel_launches()
    sampler.begin()
    torch.cuda.nvtx.range_push("timed_steps")
    ms = ctx.timed(step, steps) / steps
    torch.cuda.nvtx.range_pop()
    clocks = sampler.stop() if rank == 0 else None
    launches = engine.kernel_launches() - launches0
    q_host = torch.empty((nq, dim), dtype=torch.float32, pin_memory=True)
    q_host.copy_(q)
    ids_host = torch.empty((nq, k), dtype=torch.int64, pin_memory=True)
    d_host = torch.empty((nq, k), dtype=torch.float32, pin_memory=True)

    def step_e2e():
        step(q_host, ids_host, d_host)   # host buffers straight through the C-ABI call, at every N

    step_e2e()
    e2e_ms = ctx.timed(step_e2e, steps) / steps
    flops = 2.0 * n * dim * nq
    peak, peak_kind = ctx.peaks["tflops"], ctx.peaks["tflops_kind"]
    line = {
        "metric": "BruteForce bf16 inner-product kNN, k=100, 10,000 queries", "value": nq / (ms / 1e3),
        "unit": "queries/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "exact kNN over bf16 rows: one step = one search of the whole query batch",
                   "rows_per_gpu": n, "rows": n * world, "dim": dim, "n_query": nq, "k": k,
                   "l2_policy": "the base (9.6 GB per GPU) exceeds the 126 MB L2; no flush between steps",
                   "parallelism": f"rows sharded over {world} GPU(s), per-shard top-k merged after an all-gather"},
        "e2e": {"value": nq / (e2e_ms / 1e3), "unit": "queries/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": nq * dim * 4, "d2h_bytes_per_step": nq * k * 12},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "tc_candidates_kernel<1>", "achieved": flops / (ms / 1e3) / 1e12,
                     "peak": peak, "unit": "TFLOP/s", "frac": flops / (ms / 1e3) / 1e12 / peak, "peak_source": peak_kind,
                     "traffic": None, "note": "achieved = 2*rows*dim*queries per GPU over the whole step's time"},
    }
    if rank == 0 and not env_int("VB200_BENCH_SKIP_EXTRAS", 0):
        O = oracle_module()
        parity = {}
        # (1) the engine's result over this rank's full shard against a plain fp32 matmul of the same
        # bf16-rounded operands (torch, independent of the engine's kernels), on a query sample
        if world == 1:
            chk = min(nq, 32)
            got = out_ids[:chk].cpu().numpy()

            def round_bf16(t):   # generic::FloatToBF16: add half an ulp of bf16, truncate
                return (((t.contiguous().view(torch.int32) + 0x8000) >> 16) << 16).view(torch.float32)

            q16 = round_bf16(q[:chk])
            best_s = torch.full((chk, k), -float("inf"), device=device)
            best_i = torch.zeros((chk, k), dtype=torch.int64, device=device)
            g2 = torch.Generator(device=device)
            g2.manual_seed(6 + rank)     # the generator and slicing the shard was built with
            for b in range(0, n, 500_000):
                c = min(500_000, n - b)
                rows = torch.randn((c, dim), generator=g2, device=device)
                rows = round_bf16(rows / rows.norm(dim=1, keepdim=True))
                s_all = torch.cat([best_s, q16 @ rows.T], dim=1)
                i_all = torch.cat([best_i, torch.arange(b, b + c, device=device).expand(chk, -1)], dim=1)
                best_s, pos = torch.topk(s_all, k, dim=1)
                best_i = torch.gather(i_all, 1, pos)
            want = best_i.cpu().numpy()
            parity["full_shard_recall_vs_torch_fp32"] = float(np.mean(
                [len(set(a.tolist()) & set(b.tolist())) / k for a, b in zip(got, want)]))
            parity["full_shard_queries_checked"] = chk
            del rows, best_s, best_i
        # (2) against the oracle (HalfPrecisionQuantizer restated) over the first rows of the shard: the
        # whole query batch is searched so the tensor-core path runs, a sample is compared
        sub_rows, sub_q = int(first_rows.shape[0]), min(nq, env_int("VB200_CPU_SAMPLE", 64))
        small = engine.BfHandle(dim, engine.METRIC_IP, engine.QUANT_BF16)
        small.add(first_rows, torch.arange(sub_rows, dtype=torch.int64, device=device))
        s_ids, s_d = small.search(q, k)
        base16 = O.float_to_bf16(first_rows.cpu().numpy())
        t0 = time.perf_counter()
        w_ids, w_d = O.bf_search_bf16(base16, q[:sub_q].cpu().numpy(), k, metric=1, nthreads=host_threads())
        dt = time.perf_counter() - t0
        small.close()
        parity["ids_agree_with_oracle"] = float(np.mean(s_ids[:sub_q].cpu().numpy() == w_ids))
        parity["max_rel_dist_err_vs_oracle"] = float(np.max(np.abs(s_d[:sub_q].cpu().numpy() - w_d) /
                                                            np.maximum(np.abs(w_d), 1e-6)))
        parity["oracle_sample"] = f"{sub_q} queries x first {sub_rows} rows"
        line["parity"] = parity
        line["cpu_baseline"] = {"value": sub_q / dt * sub_rows / n, "unit": "queries/s", "cores": host_threads(),
                                "kind": "port",
                                "sample": f"{sub_q} queries against {sub_rows} of {n} rows in {dt:.2f} s, scaled by rows"}
    ix.close()
    return line


def run_rabitq(args, ctx: Ctx, steps: int, warmup: int) -> dict:
    """IVF with 1-bit RaBitQ codes and fp32 rerank: 1,000,000 x 960 (4,096 components in [0,1], sigma 0.05, clipped,
    seed 4), nlist 4,096, nprobe 64, 1,000 queries (seed 5), k 100, rerank of 4k candidates.  One GPU."""
    import torch

    from vsag_b200 import engine

    device = ctx.device
    n, dim, nlist, nprobe, nq, k, factor = scaled(1_000_000), 960, max(16, scaled(4096)), 64, max(64, scaled(1000)), 100, 4.0
    nprobe = min(nprobe, nlist)
    g = torch.Generator(device=device)
    g.manual_seed(4)
    centres = torch.rand((nlist, dim), generator=g, device=device)
    base = torch.empty((n, dim), dtype=torch.float32, device=device)
    for b in range(0, n, 250_000):
        e = min(n, b + 250_000)
        which = torch.randint(0, nlist, (e - b,), generator=g, device=device)
        base[b:e] = (centres[which] + 0.05 * torch.randn((e - b, dim), generator=g, device=device)).clamp_(0.0, 1.0)
    gq = torch.Generator(device=device)
    gq.manual_seed(5)
    which = torch.randint(0, nlist, (nq,), generator=gq, device=device)
    q = (centres[which] + 0.05 * torch.randn((nq, dim), generator=gq, device=device)).clamp_(0.0, 1.0).contiguous()
    O = oracle_module()
    rot = O.random_rotation(dim, seed=4)
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_RABITQ, use_reorder=True)
    ix.set_rabitq_rotation(rot)
    train_rows = min(n, max(65536, 64 * nlist))
    stride = max(1, n // train_rows)
    sample = base[::stride][:train_rows].contiguous()
    seeds = engine.kmeans_init(sample, nlist, seed=47)
    ix.train(sample, iters=env_int("VB200_BENCH_KMEANS_ITERS", KMEANS_ITERS), init=seeds)
    del sample, seeds
    ix.add(base, torch.arange(n, dtype=torch.int64, device=device))
    out_ids = torch.empty((nq, k), dtype=torch.int64, device=device)
    out_d = torch.empty((nq, k), dtype=torch.float32, device=device)

    def step(queries=q, ids=out_ids, dists=out_d):
        ix.search(queries, k, nprobe, factor=factor, out=(ids, dists))

    sampler = ClockSampler(ctx.local_rank)
    sampler.start()
    for _ in range(warmup):
        step()
    launches0 = engine.kernel_launches()
    sampler.begin()
    torch.cuda.nvtx.range_push("timed_steps")
    ms = ctx.timed(step, steps) / steps
    torch.cuda.nvtx.range_pop()
    clocks = sampler.stop()
    launches = engine.kernel_launches() - launches0
    k_ms, lg, rd = scan_probe(ix, step, 3)
    q_host = torch.empty((nq, dim), dtype=torch.float32, pin_memory=True)
    q_host.copy_(q)
    ids_host = torch.empty((nq, k), dtype=torch.int64, pin_memory=True)
    d_host = torch.empty((nq, k), dtype=torch.float32, pin_memory=True)
    step(q_host, ids_host, d_host)
    e2e_ms = ctx.timed(lambda: step(q_host, ids_host, d_host), steps) / steps
    peak = ctx.peaks["hbm_gbs"]
    rerank_bytes = float(nq) * factor * k * dim * 4
    line = {
        "metric": "QPS at nprobe=64, IVF-RaBitQ 1Mx960, k=100, rerank 4k", "value": nq / (ms / 1e3), "unit": "queries/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "1-bit codes, f32 query and rerank", "data": "synthetic",
        "config": {"workload": "IVF-RaBitQ search, 1M x 960, nlist 4096, nprobe 64, 1000 queries, k 100, rerank 400",
                   "n_base": n, "dim": dim, "nlist": nlist, "nprobe": nprobe, "n_query": nq, "k": k, "factor": factor,
                   "l2_policy": "codes (128 MB) fit the 126 MB L2 only just; the fp32 rows (3.84 GB) do not; no flush"},
        "e2e": {"value": nq / (e2e_ms / 1e3), "unit": "queries/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": nq * dim * 4, "d2h_bytes_per_step": nq * k * 12},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "ivf_rabitq_scan_kernel", "achieved": lg / (k_ms / 1e3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": lg / (k_ms / 1e3) / 1e9 / peak, "peak_source": ctx.peaks["hbm_kind"],
                     "kernel_ms": k_ms, "traffic": None, "algorithmic_bytes": lg,
                     "step_bytes": lg + rerank_bytes, "step_frac": (lg + rerank_bytes) / (ms / 1e3) / 1e9 / peak,
                     "note": "achieved = probed list lengths x 128 B per query tile / scan kernel time (a list probed by "
                             "several tiles is an L2 hit after the first); step_* adds the rerank's 400 fp32 rows per query "
                             "over the whole step"},
    }
    if not env_int("VB200_BENCH_SKIP_EXTRAS", 0):
        # parity on a query sample at full size: the oracle's scan over the engine's own lists with the
        # same probe lists, then its fp32 rerank over the candidates' rows
        chk = min(nq, env_int("VB200_RABITQ_CPU_SAMPLE", 100))
        qh = q[:chk].cpu().numpy()
        sizes, codes, inner = ix.get_lists()
        off = np.zeros(sizes.size + 1, np.int64)
        np.cumsum(sizes, out=off[1:])
        centroid = ix.get_rabitq_centroid()
        probes, _ = ix.route(qh, nprobe)
        t0 = time.perf_counter()
        qcodes = O.rabitq_process_query(qh, rot, centroid)
        cand, _ = O.ivf_rabitq_search(codes, off, inner, dim, qcodes, probes, int(factor * k), nthreads=host_threads())
        uniq, inv = np.unique(cand[cand >= 0], return_inverse=True)
        rows = base[torch.from_numpy(uniq).to(device)].cpu().numpy()
        remap = cand.copy()
        remap[cand >= 0] = inv
        w_local, w_d = O.rerank_fp32(rows, qh, remap, k)
        dt = time.perf_counter() - t0
        w_ids = np.where(w_local >= 0, uniq[np.clip(w_local, 0, None)], -1)
        got_ids, got_d = out_ids[:chk].cpu().numpy(), out_d[:chk].cpu().numpy()
        fin = np.isfinite(w_d)
        line["parity"] = {"ids_agree_with_oracle": float(np.mean(got_ids == w_ids)),
                          "max_rel_dist_err_vs_oracle": float(np.max(np.abs(got_d[fin] - w_d[fin]) /
                                                                     np.maximum(np.abs(w_d[fin]), 1e-6))),
                          "queries_checked": chk}
        bf = engine.BfHandle(dim, engine.METRIC_L2, engine.QUANT_FP32)
        bf.add(base, torch.arange(n, dtype=torch.int64, device=device))
        exact, _ = bf.search(q[:chk].contiguous(), k)
        bf.close()
        exact = exact.cpu().numpy()
        line["config"]["recall_at_100"] = float(np.mean(
            [len(set(a.tolist()) & set(b.tolist())) / k for a, b in zip(got_ids, exact)]))
        line["cpu_baseline"] = {"value": chk / dt, "unit": "queries/s", "cores": host_threads(), "kind": "port",
                                "sample": f"{chk} of {nq} queries: query transform, scan of the probed lists, fp32 rerank "
                                          f"(probe lists and the inverted file come from the engine), {dt:.2f} s"}
    ix.close()
    return line


def brief(line: dict) -> dict:
    """The fields of a workload's own line that the headline carries under extra_workloads."""
    keep = ("metric", "value", "unit", "ms_per_step", "steps", "dtype", "config", "e2e", "gpu_launches", "roofline",
            "parity", "cpu_baseline", "n_gpus")
    return {k: line[k] for k in keep if k in line}


def engine_release() -> None:
    """The training entry point keeps its workspace between calls; the other workloads want the memory."""
    from vsag_b200 import engine

    engine.release_workspaces()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--workload", default="ivf_sq8", choices=["ivf_sq8", "kmeans", "bruteforce", "rabitq"])
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "engine":
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
        return

    # Libraries write to stdout as they please (NCCL prints its version line when a communicator is
    # created, through C stdio); this program's stdout carries the JSON line only, so everything before
    # it goes to stderr.
    import ctypes

    libc = ctypes.CDLL(None)
    sys.stdout.flush()
    libc.fflush(None)
    saved_stdout = os.dup(1)
    os.dup2(2, 1)

    def restore_stdout():
        sys.stdout.flush()
        libc.fflush(None)
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)

    ctx = Ctx()
    if args.workload == "kmeans":
        line = run_kmeans(args, ctx, args.steps, args.warmup)
    elif args.workload == "bruteforce":
        line = run_bruteforce(args, ctx, args.steps, args.warmup)
    elif args.workload == "rabitq":
        line = run_rabitq(args, ctx, args.steps, args.warmup) if ctx.rank == 0 else {}
    else:
        line = run_ivf_sq8(args, ctx)
        if not env_int("VB200_BENCH_SKIP_EXTRAS", 0) and not env_int("VB200_BENCH_SKIP_WORKLOADS", 0):
            import torch

            torch.cuda.empty_cache()
            extras = {}
            if ctx.world == 1:
                extras["kmeans"] = brief(run_kmeans(args, ctx, 10, 3))
                engine_release()
                torch.cuda.empty_cache()
                extras["rabitq"] = brief(run_rabitq(args, ctx, 5, 3))
                torch.cuda.empty_cache()
            # at N GPUs every rank holds one 6.25M-row shard: eight ranks are the whole 50M x 768 configuration
            bf_line = run_bruteforce(args, ctx, 3, 3)
            if ctx.rank == 0:
                extras["bruteforce_bf16"] = brief(bf_line)
                line["extra_workloads"] = extras
    ctx.close()
    restore_stdout()
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
