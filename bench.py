"""Benchmark of the FP32 CSR SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = the SpMM C = A * B on the power-law graph at K = 32, 64 and 128 (three products).
Workload at N = 1: R-MAT scale 20, edge factor 16, symmetric, values U(0,1), B in U(-1,1)
(seeded synthetic stand-in for the public GNN graphs the reference measures on).  At N > 1
every added GPU brings one more such row block: A is the vertical stack of N independent
R-MAT blocks (M = N * 2^20 rows, 2^20 columns), cut into N nnz-balanced row shards by the
library's partitioner; B is replicated, C stays row-sharded, there is no data-path
collective (weak scaling).

Prints one JSON line (rank 0).  `value` is kernel-only throughput with operands resident in
HBM; `e2e` goes through the host-buffer C-ABI entry point with the copies inside the timed
region; `roofline` is for the K = 128 product kernel; `cpu_baseline` is the CPU oracle on the
host cores.  `--impl reference` times the CPU restatement of the reference's CSR row loop
(the reference has no CPU SpMM and its CUDA kernels are what this library replaces).
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
sys.path.insert(0, os.path.join(ROOT, "tests"))

KS = (32, 64, 128)
SCALE = 20
EDGE_FACTOR = 16
GRAPH_SEED = 2
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the K = 128 product kernel on
# the N = 1 workload, from the ncu capture summarised in profiles/spmm_warp_kernel_rmat20.md
# (1314.4 MB read + 522.1 MB written; the same full-size workload, about 1 GB on the device).
NCU_TRAFFIC_BYTES_K128 = 1836496216


def load_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, indices):
        """indices: the GPUs of all ranks, this rank's own first."""
        self.indices = list(indices)
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ",".join(str(i) for i in self.indices), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smmax, reasons, per_gpu = [], [], set(), {}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                idx, mhz, mx = int(f[0]), float(f[1]), float(f[2])
            except ValueError:
                continue
            per_gpu.setdefault(idx, []).append(mhz)
            smmax.append(mx)
            if idx == self.indices[0]:
                sm.append(mhz)
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        out = {"sm_mhz": statistics.median(sm) if sm else None,
               "sm_max_mhz": max(smmax) if smmax else None,
               "samples": len(sm), "reasons": sorted(reasons)}
        if len(per_gpu) > 1:
            out["per_gpu_sm_mhz"] = {str(i): statistics.median(v) for i, v in sorted(per_gpu.items())}
        return out


def build_workload(pkg, n_gpus, rank):
    """Returns this rank's shard of the stacked R-MAT matrix plus global figures."""
    blocks = [pkg.gen_rmat(SCALE, EDGE_FACTOR, seed=GRAPH_SEED + 1000 * g) for g in range(n_gpus)]
    N = blocks[0]["N"]
    row_ptr = np.zeros(sum(b["M"] for b in blocks) + 1, dtype=np.int64)
    off, base = 0, 0
    for b in blocks:
        row_ptr[off + 1: off + b["M"] + 1] = b["row_ptr"][1:].astype(np.int64) + base
        off += b["M"]
        base += b["nnz"]
    assert base < 2 ** 31
    row_ptr = row_ptr.astype(np.int32)
    col_idx = np.concatenate([b["col_idx"] for b in blocks]) if n_gpus > 1 else blocks[0]["col_idx"]
    vals = np.concatenate([b["vals"] for b in blocks]) if n_gpus > 1 else blocks[0]["vals"]
    bounds = pkg.shard_bounds(row_ptr, n_gpus)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    l_rp, l_ci, l_v = pkg.shard_csr(row_ptr, col_idx, vals, lo, hi)
    info = {"M": len(row_ptr) - 1, "N": N, "nnz": int(base), "rows_local": hi - lo,
            "nnz_local": int(len(l_ci)), "max_degree": int(np.diff(row_ptr).max()),
            "empty_rows": int((np.diff(row_ptr) == 0).sum())}
    n_ref = int(len(np.unique(l_ci)))
    return np.ascontiguousarray(l_rp), np.ascontiguousarray(l_ci), np.ascontiguousarray(l_v), info, n_ref


def run_reference_arm(args, pkg):
    """CPU restatement of the reference's CSR row loop, all host threads, full N = 1 workload."""
    import oracle_lib
    g = pkg.gen_rmat(SCALE, EDGE_FACTOR, seed=GRAPH_SEED)
    Bs = {K: pkg.host_fill_uniform(g["N"] * K, GRAPH_SEED, 100 + K, -1.0, 1.0).reshape(g["N"], K) for K in KS}
    Cs = {K: np.empty((g["M"], K), dtype=np.float32) for K in KS}
    threads = oracle_lib.num_threads()

    def step():
        for K in KS:
            oracle_lib.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], Bs[K], out=Cs[K])

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * g["nnz"] * sum(KS)
    val = flops / dt / 1e9
    line = {
        "impl": "reference", "metric": "SpMM GFLOPS (2*nnz*K/s), K=32+64+128", "value": val, "unit": "GFLOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "rmat scale %d ef %d symmetric, K=32/64/128, CPU CSR row loop" % (SCALE, EDGE_FACTOR),
                   "M": g["M"], "N": g["N"], "nnz": g["nnz"]},
        "cpu_baseline": {"value": val, "unit": "GFLOPS", "cores": threads, "kind": "port",
                         "sample": "full N=1 workload (all three K), every step"},
        "e2e": {"value": val, "unit": "GFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only-k", type=int, default=0, help="profiling aid: run a single K")
    ap.add_argument("--no-compare", action="store_true",
                    help="skip the off-path cuSPARSE column (torch.sparse CSR product, N = 1 only)")
    ap.add_argument("--b-sharded", action="store_true",
                    help="B is produced row-sharded (a GNN layer's output): every step all-gathers it "
                         "with NCCL into each GPU's own HBM before the local product")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    # torchrun exports OMP_NUM_THREADS=1 to every rank; the host-side generator and the CPU
    # baseline are OpenMP code, so give them the cores back before the libraries load
    # (all of them for the reference arm, which only rank 0 runs; an equal share otherwise).
    cores = os.cpu_count() or 1
    threads = os.environ.get("HPSPMM_BENCH_THREADS")
    if threads is None and (world > 1 or "OMP_NUM_THREADS" not in os.environ):
        threads = str(cores if args.impl == "reference" else max(1, cores // max(world, 1)))
    if threads is not None:
        os.environ["OMP_NUM_THREADS"] = threads

    import __graft_entry__ as entry
    pkg = entry.load_package()

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args, pkg)
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    n_gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if n_gpus > 1:
        dist.init_process_group("nccl", device_id=dev)

    ks = KS if not args.only_k else (args.only_k,)
    warmup = max(args.warmup, 3)

    omp = os.environ.get("OMP_NUM_THREADS")
    rp, ci, v, info, n_ref = build_workload(pkg, n_gpus, rank)
    M_l, N, nnz_l = len(rp) - 1, info["N"], len(ci)

    ctx = pkg.Context(local_rank)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream

    t_rp = torch.from_numpy(rp).to(dev)
    t_ci = torch.from_numpy(ci).to(dev)
    t_v = torch.from_numpy(v).to(dev)
    Bs, Cs = {}, {}
    for K in ks:
        Bs[K] = torch.empty((N, K), dtype=torch.float32, device=dev)
        # B replicated: every rank fills the same seeded stream on its own device
        ctx.fill_uniform(Bs[K].data_ptr(), N * K, GRAPH_SEED, 100 + K, -1.0, 1.0, sptr)
        Cs[K] = torch.empty((M_l, K), dtype=torch.float32, device=dev)
    # one plan per product width: the nominal chunk size is chosen from K, and a GNN layer
    # reuses its plan across epochs
    plans = {K: ctx.plan_create(M_l, nnz_l, t_rp.data_ptr(), K, None, sptr, N=N,
                                col_idx=t_ci.data_ptr()) for K in ks}
    plan_info = {str(K): ctx.plan_info(plans[K]) for K in ks}

    # --b-sharded: each rank owns N / world rows of B; the gathered copy is what the kernel reads
    b_sharded = args.b_sharded and n_gpus > 1 and N % n_gpus == 0
    if b_sharded:
        rows_b = N // n_gpus
        B_own = {K: Bs[K][rank * rows_b:(rank + 1) * rows_b].clone() for K in ks}

    def step(events=None, collective=True):
        for i, K in enumerate(ks):
            if events is not None:
                events[i][0].record(stream)
            if b_sharded and collective:
                dist.all_gather_into_tensor(Bs[K], B_own[K])
            ctx.spmm_csr(M_l, N, K, nnz_l, t_rp.data_ptr(), t_ci.data_ptr(), t_v.data_ptr(),
                         Bs[K].data_ptr(), Cs[K].data_ptr(), plan=plans[K], stream=sptr)
            if events is not None:
                events[i][1].record(stream)

    def barrier():
        if n_gpus > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()

    per_k_events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in ks] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    phys = [int(x) for x in visible.split(",")] if visible else list(range(max(n_gpus, local_rank + 1)))
    mine = phys[local_rank] if local_rank < len(phys) else local_rank
    sampler = ClockSampler([mine] + [p for p in phys[:n_gpus] if p != mine])
    launches_before = ctx.launch_count()
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0.record(stream)
    for s in range(args.steps):
        step(per_k_events[s])
    e1.record(stream)
    barrier()
    launches = ctx.launch_count() - launches_before
    total_ms = e0.elapsed_time(e1)
    # keep every GPU busy a little longer so the clock sampler (rank 0 watches all of them) sees the
    # loaded state; each rank loops on its own, so no collective here
    t_end = time.time() + 0.5
    while time.time() < t_end:
        step(collective=False)
    torch.cuda.synchronize()
    if n_gpus > 1:
        dist.barrier()   # every GPU stays loaded until the sampler is stopped
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    nnz_all = torch.tensor([float(nnz_l)], dtype=torch.float64, device=dev)
    per_rank_ms = [total_ms / args.steps]
    if n_gpus > 1:
        mine = t.clone()
        every = [torch.zeros_like(mine) for _ in range(n_gpus)]
        dist.all_gather(every, mine)
        per_rank_ms = [float(x.item()) / args.steps for x in every]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz_all, op=dist.ReduceOp.SUM)
    max_ms = float(t.item())
    ms_per_step = max_ms / args.steps
    nnz_total = float(nnz_all.item())
    value = 2.0 * nnz_total * sum(ks) / (ms_per_step * 1e-3) / 1e9

    per_k_ms = {}
    for i, K in enumerate(ks):
        per_k_ms[K] = statistics.mean(per_k_events[s][i][0].elapsed_time(per_k_events[s][i][1])
                                      for s in range(args.steps))

    # ---- end to end through the host-buffer entry point --------------------------------
    e2e = None
    if not args.no_e2e:
        pin = lambda a: torch.from_numpy(a).pin_memory()
        h_rp, h_ci, h_v = pin(rp), pin(ci), pin(v)
        h_B = {K: Bs[K].cpu().pin_memory() for K in ks}
        h_C = {K: torch.empty((M_l, K), dtype=torch.float32).pin_memory() for K in ks}

        def e2e_step():
            for K in ks:
                ctx.spmm_csr_host(M_l, N, K, nnz_l, h_rp.data_ptr(), h_ci.data_ptr(), h_v.data_ptr(),
                                  h_B[K].data_ptr(), h_C[K].data_ptr())

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / args.e2e_steps
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if n_gpus > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        h2d = sum((M_l + 1) * 4 + nnz_l * 8 + N * K * 4 for K in ks)
        d2h = sum(M_l * K * 4 for K in ks)
        e2e = {"value": 2.0 * nnz_total * sum(ks) / dt / 1e9, "unit": "GFLOPS",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": dt * 1e3, "steps": args.e2e_steps}
        # the host entry point works in 32-column slabs, so rows split across chunks are summed in
        # another order than on the resident path: equal within the parity tolerance, not bit for bit
        Kc = max(ks)
        torch.testing.assert_close(h_C[Kc], Cs[Kc].cpu(), rtol=1e-4, atol=1e-3)

    # ---- roofline of the dominant kernel (largest K) -----------------------------------
    peak, peak_kind = load_peak()
    Kd = max(ks)
    alg_bytes = pkg.spmm_algorithmic_bytes(M_l, n_ref, Kd, nnz_l)
    achieved = alg_bytes / (per_k_ms[Kd] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "spmm_warp_kernel K=%d (carries of split rows settled inside it)" % Kd,
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_K128 if (n_gpus == 1 and Kd == 128) else None,
                "algorithmic_bytes": alg_bytes, "ms": per_k_ms[Kd],
                "per_k": {str(K): {"ms": per_k_ms[K],
                                   "gflops": 2.0 * nnz_l * K / (per_k_ms[K] * 1e-3) / 1e9,
                                   "frac": pkg.spmm_algorithmic_bytes(M_l, n_ref, K, nnz_l)
                                   / (per_k_ms[K] * 1e-3) / 1e9 / peak} for K in ks}}

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------
    cpu = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        import oracle_lib
        outs = {K: np.empty((M_l, K), dtype=np.float32) for K in ks}
        hB = {K: Bs[K].cpu().numpy() for K in ks}

        def cpu_pass():
            for K in ks:
                oracle_lib.spmm_f32(rp, ci, v, hB[K], out=outs[K])

        cpu_pass()
        t0 = time.perf_counter()
        reps = 2
        for _ in range(reps):
            cpu_pass()
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": 2.0 * nnz_l * sum(ks) / dt / 1e9, "unit": "GFLOPS", "cores": oracle_lib.num_threads(),
               "kind": "port", "sample": "full workload, all K, 1 warm-up + 2 timed passes",
               "ms_per_pass": dt * 1e3}

    # ---- off-path comparison column: cuSPARSE CSR SpMM through torch.sparse (library code, N = 1 only),
    # the baseline the reference's own driver prints beside its kernels (test/test_all.cpp:61-87)
    compare = None
    if rank == 0 and n_gpus == 1 and not args.no_compare:
        compare = {"cusparse_csr_ms": {}, "note": "torch.sparse CSR @ dense (cuSPARSE SpMM), same operands, "
                   "3 warm-up + 10 timed launches, CUDA events"}
        try:
            import warnings
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")   # torch announces that sparse CSR support is in beta
                A_t = torch.sparse_csr_tensor(t_rp.to(torch.int64), t_ci.to(torch.int64), t_v, size=(M_l, N))
            for K in ks:
                for _ in range(3):
                    out = A_t @ Bs[K]
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(10):
                    out = A_t @ Bs[K]
                b.record()
                torch.cuda.synchronize()
                compare["cusparse_csr_ms"][str(K)] = a.elapsed_time(b) / 10
                torch.testing.assert_close(out, Cs[K], rtol=1e-3, atol=1e-3)
                del out
            del A_t
        except Exception as exc:   # a library column must never fail the bench
            compare["error"] = "%s: %s" % (type(exc).__name__, str(exc)[:200])
        rec = os.path.join(ROOT, "tests", "golden", "reference_timings.json")
        if os.path.exists(rec):
            with open(rec) as fh:
                compare["reference_kernels_recorded"] = json.load(fh)

    if rank == 0:
        line = {
            "metric": "SpMM GFLOPS (2*nnz*K/s), K=32+64+128", "value": value, "unit": "GFLOPS",
            "n_gpus": n_gpus, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "rmat scale %d ef %d symmetric x%d row blocks, K=%s, B replicated, C row-sharded"
                                   % (SCALE, EDGE_FACTOR, n_gpus, "/".join(map(str, ks))),
                       "M": info["M"], "N": N, "nnz": info["nnz"], "max_degree": info["max_degree"],
                       "empty_rows": info["empty_rows"], "n_ref_rank0": n_ref,
                       "plan": plan_info, "l2": "operands larger than L2 (no flush)",
                       "b": "all-gathered per step (NCCL)" if b_sharded else "replicated",
                       "parallelism": "row-shard x%d" % n_gpus,
                       "per_rank_ms_per_step": [round(x, 4) for x in per_rank_ms]},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "comparisons": compare,
            "clocks": clocks,
        }
        print(json.dumps(line))
    for K in ks:
        ctx.plan_destroy(plans[K])
    if n_gpus > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
