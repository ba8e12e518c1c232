"""Benchmark of the FP32 CSR SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = the SpMM C = A * B on the power-law graph at K = 32, 64 and 128 (three products).
Workload: R-MAT scale 20, edge factor 16, symmetric, values U(0,1), B in U(-1,1) (a seeded synthetic
stand-in for the public GNN graphs the reference measures on).

N = 1: operands resident in HBM, one cached plan per width.
N > 1: the SAME graph, strong-scaled: A is cut into N nnz-balanced row blocks, rank r owns rows
[bounds[r], bounds[r+1]) of A, of C and of B (a vertex's features live where its row lives), so
every product starts with an exchange: each rank receives, over NCCL into its own HBM, the rows of
B its shard references (hpspmm_sharded_*).  The exchange is INSIDE the timed step.  The three
exchanges of a step are begun first and the products follow in turn, so an exchange overlaps the
previous product.  Printed beside `value`: the same step with the exchanges skipped (kernel only),
with one blocking call per product, and with a plain all-gather of B instead of the needed rows.

Prints one JSON line (rank 0).  `value` is whole-job throughput, device-timed, max over ranks;
`e2e` goes through the host-buffer entry points with the copies inside the timed region;
`roofline` is for the K = 128 product kernel; `cpu_baseline` is the CPU restatement of the
reference's row loop on the host cores.  `--impl reference` times the reference's own kernels
(LBSpMM, its flagship, compiled unmodified into oracle/_ref/libref_spmm.so) on one GPU through
the reference's own entry point, which uploads, runs 200 launches and reports their mean; when that
library is absent it times the CPU restatement instead and says so.
"""
import argparse
import ctypes
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
NVLINK_GBS = 770.0    # measured peer copy per direction per GPU on this pool (900 nominal)
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "spmm_warp_kernel_rmat20_k128.traffic.json")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_spmm.so")
METRIC = "SpMM GFLOPS (2*nnz*K/s), K=32+64+128"


def load_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(signature):
    """DRAM bytes per launch of the K = 128 kernel from the tracked ncu capture, or None when the
    capture was taken of another kernel instantiation than the one that runs now."""
    try:
        rec = json.load(open(TRAFFIC_FILE))
    except Exception:
        return None, "no capture on file"
    if rec.get("kernel") != signature:
        return None, "capture on file is of %s, the run used %s" % (rec.get("kernel"), signature)
    return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"]), rec.get("source", "")


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


def graph_info(g):
    deg = np.diff(g["row_ptr"])
    return {"M": g["M"], "N": g["N"], "nnz": g["nnz"], "max_degree": int(deg.max()),
            "empty_rows": int((deg == 0).sum())}


def workload_name(n_gpus):
    base = "rmat scale %d ef %d symmetric, K=%s" % (SCALE, EDGE_FACTOR, "/".join(map(str, KS)))
    if n_gpus == 1:
        return base + ", operands resident, C = A*B"
    return base + (", strong-scaled over %d row blocks balanced by entries + a weight per row; B row-sharded like A, "
                   "the rows each shard references exchanged inside the step; C row-sharded" % n_gpus)


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------

def cpu_port_sample(pkg, g, Bs, passes=1):
    """CPU restatement of the reference's CSR row loop on all host threads, full workload."""
    import oracle_lib
    outs = {K: np.empty((g["M"], K), dtype=np.float32) for K in KS}

    def one():
        for K in KS:
            oracle_lib.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], Bs[K], out=outs[K])

    one()
    t0 = time.perf_counter()
    for _ in range(passes):
        one()
    dt = (time.perf_counter() - t0) / passes
    return {"value": 2.0 * g["nnz"] * sum(KS) / dt / 1e9, "unit": "GFLOPS", "cores": oracle_lib.num_threads(),
            "kind": "port", "sample": "full workload (all three K), 1 warm-up + %d timed pass(es)" % passes,
            "ms_per_pass": dt * 1e3}


def load_ref_lib():
    if not os.path.exists(REF_LIB):
        return None, "oracle/_ref/libref_spmm.so not built on this box"
    try:
        lib = ctypes.CDLL(REF_LIB)
    except OSError as exc:
        return None, "libref_spmm.so does not load: %s" % str(exc)[:120]
    I, P, F = ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)
    for fn in (lib.ref_gespmm, lib.ref_lbspmm):
        fn.argtypes = [I, I, I, I, P, P, P, P, P, F]
        fn.restype = I
    lib.ref_launches_per_call.restype = I
    D = ctypes.POINTER(ctypes.c_double)
    lib.ref_lbspmm_phases.argtypes = [I, I, I, I, P, P, P, P, P, F, D, D]
    lib.ref_lbspmm_phases.restype = I
    return lib, ""


def padded_coo(g):
    """The reference's COO view: one row id per entry, (0, 0, 0.0) padding to a multiple of 32
    (spmm/mm/spmm_common.cpp:210-226)."""
    pad = (-g["nnz"]) % 32
    rows = np.repeat(np.arange(g["M"], dtype=np.int32), np.diff(g["row_ptr"]))
    z = np.zeros(pad, np.int32)
    return (np.concatenate([rows, z]), np.concatenate([g["col_idx"], z]),
            np.concatenate([g["vals"], np.zeros(pad, np.float32)]))


def silence_stdout():
    """The reference's entry points print their time to stdout; keep the JSON line the only output."""
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)
    os.close(devnull)
    return saved


def restore_stdout(saved):
    sys.stdout.flush()
    os.dup2(saved, 1)
    os.close(saved)


def time_reference_kernels(lib, g, Bs, coo, which=("lbspmm",)):
    """Runs the reference's own entry points on host operands.  Returns per K the mean launch time
    the reference's timer reports and the wall time of the whole call (upload, 200 launches, download)."""
    M, N = g["M"], g["N"]
    r, c, v = coo
    out = {}
    launches = lib.ref_launches_per_call()
    saved = silence_stdout()
    try:
        for K in KS:
            C = np.empty((M, K), np.float32)
            ms = ctypes.c_float()
            rec = {}
            if "lbspmm" in which:
                up, down = ctypes.c_double(), ctypes.c_double()
                rc = lib.ref_lbspmm_phases(M, N, K, len(r), r.ctypes.data, c.ctypes.data, v.ctypes.data,
                                           Bs[K].ctypes.data, C.ctypes.data, ctypes.byref(ms), ctypes.byref(up),
                                           ctypes.byref(down))
                if rc != 0:
                    raise RuntimeError("the reference's LBSpMM failed at K=%d" % K)
                rec["lbspmm_ms"] = ms.value
                rec["lbspmm_upload_ms"] = up.value * 1e3
                rec["lbspmm_download_ms"] = down.value * 1e3
            if "gespmm" in which:
                t0 = time.perf_counter()
                rc = lib.ref_gespmm(M, N, K, g["nnz"], g["row_ptr"].ctypes.data, g["col_idx"].ctypes.data,
                                    g["vals"].ctypes.data, Bs[K].ctypes.data, C.ctypes.data, ctypes.byref(ms))
                rec["gespmm_wall_s"] = time.perf_counter() - t0
                rec["gespmm_ms"] = ms.value if rc == 0 else None
            out[K] = rec
    finally:
        restore_stdout(saved)
    return out, launches


def run_reference_arm(args, pkg, n_gpus):
    g = pkg.gen_rmat(SCALE, EDGE_FACTOR, seed=GRAPH_SEED)
    Bs = {K: pkg.host_fill_uniform(g["N"] * K, GRAPH_SEED, 100 + K, -1.0, 1.0).reshape(g["N"], K) for K in KS}
    info = graph_info(g)
    flops = 2.0 * g["nnz"] * sum(KS)
    lib, why = load_ref_lib()
    gpu_ok = False
    if lib is not None:
        try:
            import torch
            gpu_ok = torch.cuda.is_available()
            if not gpu_ok:
                why = "no CUDA device for the reference's kernels"
        except Exception as exc:
            why = "torch unavailable: %s" % exc
    cpu = cpu_port_sample(pkg, g, Bs, passes=1)
    line = {"impl": "reference", "metric": METRIC, "unit": "GFLOPS", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong" if n_gpus > 1 else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "cpu_baseline": cpu}
    cfg = {"workload": workload_name(n_gpus)}
    cfg.update(info)
    if lib is not None and gpu_ok:
        coo = padded_coo(g)
        steps = max(1, args.steps)
        warm = max(1, min(args.warmup, 2))
        for _ in range(warm):
            time_reference_kernels(lib, g, Bs, coo)
        kernel_ms, e2e_ms = [], []
        launches = 200
        for _ in range(steps):
            rec, launches = time_reference_kernels(lib, g, Bs, coo)
            kernel_ms.append(sum(rec[K]["lbspmm_ms"] for K in KS))
            # one product end to end = the reference's upload + one launch of its loop + its download
            e2e_ms.append(sum(rec[K]["lbspmm_upload_ms"] + rec[K]["lbspmm_ms"] + rec[K]["lbspmm_download_ms"]
                              for K in KS))
        k_ms, e_ms = statistics.mean(kernel_ms), statistics.mean(e2e_ms)
        r, c, v = coo
        h2d = sum(len(r) * 12 + g["N"] * K * 4 for K in KS)
        d2h = sum(g["M"] * K * 4 for K in KS)
        cfg["reference_entry"] = ("LBSpMM (HP-SpMM, spmm/mm/spmm_kernel.cu:733-768) on one GPU: per product "
                                  "Matrix::to(kCUDA) uploads from pageable memory, %d launches timed by its own "
                                  "GpuTimer, C read back; kernels compiled unmodified for sm_100a" % launches)
        cfg["per_k_ms"] = {str(K): rec[K]["lbspmm_ms"] for K in KS}
        cfg["per_k_upload_ms"] = {str(K): rec[K]["lbspmm_upload_ms"] for K in KS}
        cfg["per_k_download_ms"] = {str(K): rec[K]["lbspmm_download_ms"] for K in KS}
        line.update({"value": flops / (k_ms * 1e-3) / 1e9, "ms_per_step": k_ms, "kind": "reference",
                     "e2e": {"value": flops / (e_ms * 1e-3) / 1e9, "unit": "GFLOPS", "h2d_bytes_per_step": int(h2d),
                             "d2h_bytes_per_step": int(d2h), "ms_per_step": e_ms,
                             "how": "the reference's own upload (Matrix::to(kCUDA), pageable host memory) + the mean "
                                    "of its %d timed launches + its own download (Matrix::to(kCPU)), per product" % launches},
                     "gpu_launches": int(launches * len(KS) * steps), "config": cfg})
    else:
        # the reference's kernels cannot run here: time the CPU restatement of its row loop instead
        steps = max(1, min(args.steps, 10))
        cpu = cpu_port_sample(pkg, g, Bs, passes=steps)
        cfg["reference_kernels"] = "unavailable: " + why
        cfg["reference_entry"] = "CPU restatement of the CSR row loop of spmm/mm/spmm_kernel.cu:324-346, all host threads"
        line.update({"value": cpu["value"], "ms_per_step": cpu["ms_per_pass"], "kind": "port", "cpu_baseline": cpu,
                     "e2e": {"value": cpu["value"], "unit": "GFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                     "gpu_launches": 0, "config": cfg})
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# this library, one GPU
# ------------------------------------------------------------------------------------------------

def make_sampler(n_gpus, local_rank):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    phys = [int(x) for x in visible.split(",")] if visible else list(range(max(n_gpus, local_rank + 1)))
    mine = phys[local_rank] if local_rank < len(phys) else local_rank
    return ClockSampler([mine] + [p for p in phys[:n_gpus] if p != mine])


def run_single(args, pkg):
    import torch
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ks = KS if not args.only_k else (args.only_k,)
    warmup = max(args.warmup, 3)
    g = pkg.gen_rmat(SCALE, EDGE_FACTOR, seed=GRAPH_SEED)
    info = graph_info(g)
    rp, ci, v = g["row_ptr"], g["col_idx"], g["vals"]
    M, N, nnz = g["M"], g["N"], g["nnz"]
    n_ref = int(len(np.unique(ci)))

    ctx = pkg.Context(0)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    t_rp, t_ci, t_v = (torch.from_numpy(a).to(dev) for a in (rp, ci, v))
    Bs, Cs = {}, {}
    for K in ks:
        Bs[K] = torch.empty((N, K), dtype=torch.float32, device=dev)
        ctx.fill_uniform(Bs[K].data_ptr(), N * K, GRAPH_SEED, 100 + K, -1.0, 1.0, sptr)
        Cs[K] = torch.empty((M, K), dtype=torch.float32, device=dev)
    # one plan per product width: the nominal chunk size is chosen from K, and a GNN layer
    # reuses its plan across epochs
    plans = {K: ctx.plan_create(M, nnz, t_rp.data_ptr(), K, None, sptr, N=N, col_idx=t_ci.data_ptr()) for K in ks}
    plan_info = {str(K): ctx.plan_info(plans[K]) for K in ks}

    def step(events=None):
        for i, K in enumerate(ks):
            if events is not None:
                events[i][0].record(stream)
            ctx.spmm_csr(M, N, K, nnz, t_rp.data_ptr(), t_ci.data_ptr(), t_v.data_ptr(),
                         Bs[K].data_ptr(), Cs[K].data_ptr(), plan=plans[K], stream=sptr)
            if events is not None:
                events[i][1].record(stream)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    per_k_events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in ks] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = make_sampler(1, 0)
    launches_before = ctx.launch_count()
    sampler.start()
    time.sleep(0.3)
    torch.cuda.synchronize()
    e0.record(stream)
    for s in range(args.steps):
        step(per_k_events[s])
    e1.record(stream)
    torch.cuda.synchronize()
    launches = ctx.launch_count() - launches_before
    ms_per_step = e0.elapsed_time(e1) / args.steps
    t_end = time.time() + 0.5     # keep the GPU loaded a little longer so the sampler sees it under load
    while time.time() < t_end:
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    value = 2.0 * nnz * sum(ks) / (ms_per_step * 1e-3) / 1e9
    per_k_ms = {K: statistics.mean(per_k_events[s][i][0].elapsed_time(per_k_events[s][i][1])
                                   for s in range(args.steps)) for i, K in enumerate(ks)}

    # ---- end to end: host buffers in, host buffers out, A uploaded once per step ----------------
    e2e = None
    if not args.no_e2e:
        pin = lambda a: torch.from_numpy(a).pin_memory()
        h_rp, h_ci, h_v = pin(rp), pin(ci), pin(v)
        h_B = {K: Bs[K].cpu().pin_memory() for K in ks}
        h_C = {K: torch.empty((M, K), dtype=torch.float32).pin_memory() for K in ks}

        def e2e_step():
            ctx.spmm_csr_host_multi(M, N, nnz, h_rp.data_ptr(), h_ci.data_ptr(), h_v.data_ptr(), list(ks),
                                    [h_B[K].data_ptr() for K in ks], [h_C[K].data_ptr() for K in ks])

        e2e_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / args.e2e_steps
        h2d = (M + 1) * 4 + nnz * 8 + sum(N * K * 4 for K in ks)
        d2h = sum(M * K * 4 for K in ks)
        e2e = {"value": 2.0 * nnz * sum(ks) / dt / 1e9, "unit": "GFLOPS", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": dt * 1e3, "steps": args.e2e_steps,
               "h2d_gbs": h2d / dt / 1e9, "d2h_gbs": d2h / dt / 1e9,
               "entry": "hpspmm_spmm_csr_f32_host_multi: A once, then the column slabs of the three products through "
                        "one upload / product / download pipeline, pinned host buffers"}
        # slabs are narrower products, so rows split across chunks are summed in another order than on the
        # resident path: equal within the parity tolerance, not bit for bit
        for K in ks:
            torch.testing.assert_close(h_C[K], Cs[K].cpu(), rtol=1e-4, atol=1e-3)

    # ---- roofline of the dominant kernel (largest K) --------------------------------------------
    peak, peak_kind = load_peak()
    Kd = max(ks)
    alg = {K: pkg.spmm_algorithmic_bytes(M, n_ref, K, nnz) for K in ks}
    achieved = alg[Kd] / (per_k_ms[Kd] * 1e-3) / 1e9
    signature = ctx.kernel_signature(plans[Kd], Kd)
    traffic, traffic_note = ncu_traffic(signature) if Kd == 128 else (None, "captured at K = 128 only")
    roofline = {"bound": "hbm", "kernel": signature + " (carries of split rows settled inside it)",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_note,
                "algorithmic_bytes": alg[Kd], "ms": per_k_ms[Kd]}

    # ---- CPU baseline -----------------------------------------------------------------------------
    cpu = None
    hB = None
    if not args.no_cpu_baseline or not args.no_compare:
        hB = {K: Bs[K].cpu().numpy() for K in ks}
    if not args.no_cpu_baseline and ks == KS:
        cpu = cpu_port_sample(pkg, g, hB, passes=2)

    # ---- off-path comparison columns, the baselines the reference's own driver prints beside its kernels
    # (test/test_all.cpp:61-107): cuSPARSE CSR SpMM (through torch.sparse) and the reference's kernels, live
    compare = None
    if not args.no_compare:
        compare = {"cusparse_csr_ms": {}, "note": "torch.sparse CSR @ dense (cuSPARSE SpMM), same operands, "
                   "3 warm-up + 10 timed launches, CUDA events"}
        try:
            import warnings
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")   # torch announces that sparse CSR support is in beta
                A_t = torch.sparse_csr_tensor(t_rp.to(torch.int64), t_ci.to(torch.int64), t_v, size=(M, N))
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
        if 128 in ks:
            # this library's own alternative at K = 128: the rows of B fetched by TMA gather4 (HPSPMM_ALGO_TMA)
            try:
                tma_opts = pkg.Opts(algo=pkg.ALGO_TMA)
                keep = Cs[128].clone()
                run_tma = lambda: ctx.spmm_csr(M, N, 128, nnz, t_rp.data_ptr(), t_ci.data_ptr(), t_v.data_ptr(),
                                               Bs[128].data_ptr(), Cs[128].data_ptr(), plan=plans[128],
                                               opts=tma_opts, stream=sptr)
                for _ in range(3):
                    run_tma()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(10):
                    run_tma()
                b.record(stream)
                torch.cuda.synchronize()
                compare["own_tma_kernel_k128"] = {"ms": a.elapsed_time(b) / 10, "default_kernel_ms": per_k_ms[128],
                                                  "bit_equal_to_default": bool(torch.equal(keep, Cs[128])),
                                                  "bounded_waits_that_ran_out": ctx.tma_fallbacks()}
                del keep
            except Exception as exc:
                compare["own_tma_kernel_k128"] = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:200])}
        lib, why = load_ref_lib()
        if lib is not None and ks == KS:
            try:
                rec, launches_ref = time_reference_kernels(lib, g, hB, padded_coo(g), which=("lbspmm", "gespmm"))
                live = {"launches_per_figure": launches_ref, "note": "the reference's LBSpMM / GESpMM entry points "
                        "(unmodified sources, sm_100a) on the same graph and GPU, after the timed region"}
                for K in ks:
                    live[str(K)] = {"lbspmm_ms": rec[K]["lbspmm_ms"], "gespmm_ms": rec[K]["gespmm_ms"],
                                    "ours_ms": per_k_ms[K],
                                    "lbspmm_over_ours": rec[K]["lbspmm_ms"] / per_k_ms[K] if rec[K]["lbspmm_ms"] else None}
                compare["reference_kernels_live"] = live
            except Exception as exc:
                compare["reference_kernels_live"] = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:200])}
        else:
            compare["reference_kernels_live"] = {"unavailable": why or "single-K run"}
            rec_path = os.path.join(ROOT, "tests", "golden", "reference_timings.json")
            if os.path.exists(rec_path):
                with open(rec_path) as fh:
                    compare["reference_kernels_recorded_earlier"] = json.load(fh)

    cfg = {"workload": workload_name(1), "n_ref": n_ref, "plan": plan_info,
           "l2": "operands larger than L2 (no flush)", "b": "resident", "parallelism": "one GPU"}
    cfg.update(info)
    line = {"metric": METRIC, "value": value, "unit": "GFLOPS", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": cfg, "roofline": roofline, "cpu_baseline": cpu,
            "e2e": e2e, "gpu_launches": int(launches), "comparisons": compare, "clocks": clocks}
    for K in ks:   # flat, so that they survive a parser that keeps top-level keys only
        line["ms_k%d" % K] = per_k_ms[K]
        line["gflops_k%d" % K] = 2.0 * nnz * K / (per_k_ms[K] * 1e-3) / 1e9
        line["frac_k%d" % K] = alg[K] / (per_k_ms[K] * 1e-3) / 1e9 / peak
    print(json.dumps(line))
    for K in ks:
        ctx.plan_destroy(plans[K])
    return 0


# ------------------------------------------------------------------------------------------------
# this library, N GPUs: strong-scaled, rows of B exchanged inside the step
# ------------------------------------------------------------------------------------------------

def run_sharded(args, pkg, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    ks = KS
    warmup = max(args.warmup, 3)

    g = pkg.gen_rmat(SCALE, EDGE_FACTOR, seed=GRAPH_SEED)     # every rank builds the same seeded graph
    info = graph_info(g)
    N, nnz_total = g["N"], g["nnz"]
    bounds = (pkg.shard_bounds_weighted(g["row_ptr"], world, args.row_weight) if args.row_weight > 0
              else pkg.shard_bounds(g["row_ptr"], world))
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    rp, ci, v = (np.ascontiguousarray(a) for a in (rp, ci, v))
    M_l, nnz_l = hi - lo, len(ci)
    n_ref_l = int(len(np.unique(ci)))

    ctx = pkg.Context(local_rank)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    # the communicator id travels through the process group the launcher set up
    idt = torch.zeros(pkg.COMM_ID_BYTES, dtype=torch.uint8, device=dev)
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    comm_id = bytes(idt.cpu().numpy().tobytes())
    sp = pkg.ShardedSpmm(ctx, world, rank, comm_id, M_l, N, rp, ci, bounds, max(ks),
                         exchange=pkg.EXCHANGE_NEEDED_ROWS, stream=sptr)
    sp_info = sp.info()
    t_v = torch.from_numpy(v).to(dev)
    B_own, Cs = {}, {}
    for K in ks:
        # this rank's rows of the same seeded B the one-GPU run uses
        full = pkg.host_fill_uniform(N * K, GRAPH_SEED, 100 + K, -1.0, 1.0).reshape(N, K)
        B_own[K] = torch.from_numpy(np.ascontiguousarray(full[lo:hi])).to(dev)
        del full
        Cs[K] = torch.empty((M_l, K), dtype=torch.float32, device=dev)

    order = sorted(ks, reverse=not args.narrow_first)
    slot_of = {K: i for i, K in enumerate(ks)}

    def step_overlapped():
        # widest first: the exchanges are longer than the products, so the product left with nothing to hide
        # behind should be the smallest one
        for K in order:
            sp.begin(slot_of[K], K, B_own[K].data_ptr(), sptr)
        for K in order:
            sp.product(slot_of[K], K, t_v.data_ptr(), Cs[K].data_ptr(), stream=sptr)

    def step_kernels(events=None):
        for slot, K in enumerate(ks):
            if events is not None:
                events[slot][0].record(stream)
            sp.product(slot, K, t_v.data_ptr(), Cs[K].data_ptr(), stream=sptr)
            if events is not None:
                events[slot][1].record(stream)

    def step_blocking(which):
        for K in ks:
            which.spmm(K, t_v.data_ptr(), B_own[K].data_ptr(), Cs[K].data_ptr(), stream=sptr)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        barrier()
        return a.elapsed_time(b) / steps

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        vals = [float(e.item()) for e in every]
        return max(vals), vals

    for _ in range(warmup):
        step_overlapped()
    barrier()
    sampler = make_sampler(world, local_rank)
    launches_before = ctx.launch_count()
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_mine = timed(step_overlapped, args.steps)
    launches = ctx.launch_count() - launches_before
    ms_per_step, per_rank_ms = max_over_ranks(ms_mine)
    value = 2.0 * nnz_total * sum(ks) / (ms_per_step * 1e-3) / 1e9

    # the same step without the exchanges (the rows of the last exchange are still in place)
    for _ in range(3):
        step_kernels()
    per_k_events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in ks]
                    for _ in range(args.steps)]
    it = iter(per_k_events)
    kernel_ms, per_rank_kernel = max_over_ranks(timed(lambda: step_kernels(next(it)), args.steps))
    per_k_ms = {K: statistics.mean(ev[i][0].elapsed_time(ev[i][1]) for ev in per_k_events) for i, K in enumerate(ks)}
    # one blocking call per product: exchange, then product, nothing overlapped
    for _ in range(2):
        step_blocking(sp)
    blocking_ms, _ = max_over_ranks(timed(lambda: step_blocking(sp), max(3, args.steps // 2)))
    clocks = None
    # keep every GPU busy a little longer so the clock sampler (rank 0 watches all of them) sees the loaded state
    t_end = time.time() + 0.5
    while time.time() < t_end:
        step_kernels()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        clocks = sampler.stop()

    # for comparison, each with its own plan and buffers: the same needed rows packed and sent by NCCL
    # send / receive instead of pushed, and a plain all-gather of B
    allgather_ms = nccl_rows_ms = None
    if not args.no_compare:
        for mode in (pkg.EXCHANGE_NEEDED_ROWS_NCCL, pkg.EXCHANGE_ALL_ROWS):
            other = pkg.ShardedSpmm(ctx, world, rank, pkg_comm_id(pkg, dist, dev, rank), M_l, N, rp, ci, bounds,
                                    max(ks), exchange=mode, stream=sptr)

            def step_other():
                for slot, K in enumerate(ks):
                    other.begin(slot, K, B_own[K].data_ptr(), sptr)
                for slot, K in enumerate(ks):
                    other.product(slot, K, t_v.data_ptr(), Cs[K].data_ptr(), stream=sptr)

            for _ in range(2):
                step_other()
            ms, _ = max_over_ranks(timed(step_other, max(3, args.steps // 2)))
            if mode == pkg.EXCHANGE_ALL_ROWS:
                allgather_ms = ms
            else:
                nccl_rows_ms = ms
            other.close()

    # ---- end to end: values and this rank's rows of B from pinned host memory, C back to it, every step;
    # the sparsity structure stays in the shard plan (it is what a training loop keeps across steps)
    e2e = None
    if not args.no_e2e:
        h_v = torch.from_numpy(v).pin_memory()
        h_B = {K: B_own[K].cpu().pin_memory() for K in ks}
        h_C = {K: torch.empty((M_l, K), dtype=torch.float32).pin_memory() for K in ks}
        d_v2 = torch.empty_like(t_v)
        d_B2 = {K: torch.empty_like(B_own[K]) for K in ks}
        lib = ctx.lib

        def e2e_step():
            lib.hpspmm_memcpy_h2d(ctx.handle, d_v2.data_ptr(), h_v.data_ptr(), nnz_l * 4, sptr)
            for slot, K in enumerate(ks):
                lib.hpspmm_memcpy_h2d(ctx.handle, d_B2[K].data_ptr(), h_B[K].data_ptr(), h_B[K].numel() * 4, sptr)
                sp.begin(slot, K, d_B2[K].data_ptr(), sptr)
            for slot, K in enumerate(ks):
                sp.product(slot, K, d_v2.data_ptr(), Cs[K].data_ptr(), stream=sptr)
                lib.hpspmm_memcpy_d2h(ctx.handle, h_C[K].data_ptr(), Cs[K].data_ptr(), M_l * K * 4, sptr)
            ctx.stream_sync(sptr)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        mine = (time.perf_counter() - t0) / args.e2e_steps
        barrier()
        dt, per_rank_e2e = max_over_ranks(mine)
        h2d = nnz_l * 4 + sum(M_l * K * 4 for K in ks)     # B_own has M_l rows (square graph)
        d2h = sum(M_l * K * 4 for K in ks)
        tot = torch.tensor([float(h2d), float(d2h)], dtype=torch.float64, device=dev)
        dist.all_reduce(tot)
        e2e = {"value": 2.0 * nnz_total * sum(ks) / dt / 1e9, "unit": "GFLOPS",
               "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()),
               "ms_per_step": dt * 1e3, "steps": args.e2e_steps,
               "per_rank_ms_per_step": [round(x * 1e3, 3) for x in per_rank_e2e],
               "rank0_h2d_gbs": h2d / mine / 1e9, "rank0_d2h_gbs": d2h / mine / 1e9,
               "entry": "per rank: values and own rows of B up (pinned), hpspmm_sharded_exchange_begin / "
                        "hpspmm_sharded_product, C block down; sparsity structure resident in the shard plan"}

    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "M_l": M_l, "nnz_l": nnz_l, "n_ref_l": n_ref_l,
                                      "rows_received": sp_info["rows_received"], "rows_sent": sp_info["rows_sent"]})
    if rank == 0:
        peak, peak_kind = load_peak()
        Kd = max(ks)
        alg = {K: pkg.spmm_algorithmic_bytes(M_l, n_ref_l, K, nnz_l) for K in ks}
        achieved = alg[Kd] / (per_k_ms[Kd] * 1e-3) / 1e9
        recv_rows = max(x["rows_received"] for x in gathered)
        recv_bytes = recv_rows * 4 * sum(ks)
        roofline = {"bound": "hbm", "kernel": "rank 0's local product, K=%d" % Kd, "achieved": achieved, "peak": peak,
                    "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                    "algorithmic_bytes": alg[Kd], "ms": per_k_ms[Kd]}
        cfg = {"workload": workload_name(world), "parallelism": "row-shard x%d" % world,
               "row_weight": args.row_weight, "row_bounds": [int(x) for x in bounds],
               "b": "row-sharded; per product each rank receives the rows its shard references, pushed by their owners "
                    "into its own HBM (peer stores over NVLink, a 4-byte NCCL all-reduce as the completion signal); "
                    "three exchanges begun first, products in turn",
               "l2": "operands larger than L2 at N <= 2; smaller shards are not flushed (steady-state training loop)",
               "per_rank_ms_per_step": [round(x, 4) for x in per_rank_ms],
               "kernel_only_ms_per_step": kernel_ms,
               "kernel_only_gflops": 2.0 * nnz_total * sum(ks) / (kernel_ms * 1e-3) / 1e9,
               "per_rank_kernel_only_ms": [round(x, 4) for x in per_rank_kernel],
               "blocking_calls_ms_per_step": blocking_ms,
               "allgather_ms_per_step": allgather_ms,
               "needed_rows_by_nccl_sendrecv_ms_per_step": nccl_rows_ms,
               "exchange": {"rows_received_max_rank": recv_rows, "bytes_received_per_step_max_rank": recv_bytes,
                            "nvlink_floor_ms": recv_bytes / (NVLINK_GBS * 1e9) * 1e3,
                            "allgather_rows_per_rank": N - min(x["M_l"] for x in gathered),
                            "hidden_ms": max(0.0, blocking_ms - ms_per_step),
                            "exposed_ms": max(0.0, ms_per_step - kernel_ms)},
               "shards": gathered}
        cfg.update(info)
        line = {"metric": METRIC, "value": value, "unit": "GFLOPS", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg, "roofline": roofline,
                "cpu_baseline": None, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
                "kernel_only_ms_per_step": kernel_ms, "blocking_calls_ms_per_step": blocking_ms,
                "allgather_ms_per_step": allgather_ms, "needed_rows_by_nccl_sendrecv_ms_per_step": nccl_rows_ms}
        for K in ks:
            line["ms_k%d_rank0_kernel" % K] = per_k_ms[K]
        print(json.dumps(line))
    sp.close()
    ctx.close()
    dist.destroy_process_group()
    return 0


def run_cfg3_replicated(args, pkg, rank, local_rank, world):
    """BASELINE config 3: the uniform sparse graph (Erdos-Renyi, 2.45 M rows, mean degree 50), K = 64, strong-scaled
    over nnz-balanced row blocks with B REPLICATED on every GPU: no exchange, C row-sharded.  A secondary workload
    (`--workload cfg3`); the default bench line stays on config 2."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    K = 64
    g = pkg.gen_erdos_renyi(2_450_000, 2_450_000, 50.0, seed=3)
    N, nnz_total = g["N"], g["nnz"]
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = (np.ascontiguousarray(a) for a in pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi))
    M_l, nnz_l = hi - lo, len(ci)
    ctx = pkg.Context(local_rank)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    t_rp, t_ci, t_v = (torch.from_numpy(a).to(dev) for a in (rp, ci, v))
    B = torch.empty((N, K), dtype=torch.float32, device=dev)
    ctx.fill_uniform(B.data_ptr(), N * K, 3, 64, -1.0, 1.0, sptr)     # every rank fills the same seeded stream
    C = torch.empty((M_l, K), dtype=torch.float32, device=dev)
    plan = ctx.plan_create(M_l, nnz_l, t_rp.data_ptr(), K, None, sptr, N=N, col_idx=t_ci.data_ptr())

    def step():
        ctx.spmm_csr(M_l, N, K, nnz_l, t_rp.data_ptr(), t_ci.data_ptr(), t_v.data_ptr(), B.data_ptr(), C.data_ptr(),
                     plan=plan, stream=sptr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record(stream)
    for _ in range(args.steps):
        step()
    b.record(stream)
    barrier()
    ms = a.elapsed_time(b) / args.steps
    per_rank = [ms]
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank = [float(x.item()) for x in every]
    ms_max = max(per_rank)
    if rank == 0:
        peak, peak_kind = load_peak()
        n_ref = int(len(np.unique(ci)))
        alg = pkg.spmm_algorithmic_bytes(M_l, n_ref, K, nnz_l)
        gather_bytes = 4.0 * (M_l + 1) + 8.0 * nnz_l + 4.0 * K * nnz_l + 4.0 * K * M_l
        print(json.dumps({
            "metric": "SpMM GFLOPS (2*nnz*K/s), K=64", "value": 2.0 * nnz_total * K / (ms_max * 1e-3) / 1e9,
            "unit": "GFLOPS", "n_gpus": world, "steps": args.steps, "ms_per_step": ms_max, "scaling": "strong",
            "dtype": "f32", "data": "synthetic", "higher_is_better": True,
            "config": {"workload": "erdos-renyi 2.45M rows mean degree 50 (config 3), K=64, B replicated, "
                                   "nnz-balanced row blocks x%d, no exchange" % world,
                       "M": g["M"], "N": N, "nnz": nnz_total, "per_rank_ms": [round(x, 4) for x in per_rank]},
            "roofline": {"bound": "hbm", "kernel": ctx.kernel_signature(plan, K), "achieved": alg / (per_rank[0] * 1e-3) / 1e9,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": alg / (per_rank[0] * 1e-3) / 1e9 / peak, "algorithmic_bytes": alg,
                         "zero_reuse_gather_gbs": gather_bytes / (per_rank[0] * 1e-3) / 1e9}}))
    ctx.plan_destroy(plan)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def pkg_comm_id(pkg, dist, dev, rank):
    import torch
    idt = torch.zeros(pkg.COMM_ID_BYTES, dtype=torch.uint8, device=dev)
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    return bytes(idt.cpu().numpy().tobytes())


def run_ceilings(pkg):
    """Load-path ceilings of the GPU with the gather shape of the product kernels (hpspmm_probe_gather_gbs):
    one JSON line with GB/s per row size and access pattern."""
    ctx = pkg.Context(0)
    n = 16 * 1024 * 1024
    out = []
    for rb in (128, 256, 512):
        for name, rows, pattern, hot_rows, hot_share in (
                ("stream over a 64 MB table", (64 << 20) // rb, 0, 0, 0.0),
                ("random rows, 32 MB table (L2-resident)", (32 << 20) // rb, 1, 0, 0.0),
                ("random rows, 64 MB table (L2-resident)", (64 << 20) // rb, 1, 0, 0.0),
                ("random rows, 1048576-row table", 1 << 20, 1, 0, 0.0),
                ("random rows, 546186-row table (the referenced part of B on the bench graph)", 546186, 1, 0, 0.0),
                ("same table, 25 % of the gathers on its 1770 hottest rows", 546186, 2, 1770, 0.25),
                ("same table, 55 % of the gathers on its 14000 hottest rows", 546186, 2, 14000, 0.55),
                ("random rows, 4194304-row table (DRAM)", 1 << 22, 1, 0, 0.0)):
            gbs, ms = ctx.probe_gather(rb, rows, n, pattern, hot_rows, hot_share, 10)
            out.append({"row_bytes": rb, "pattern": name, "table_mb": rows * rb / 1e6, "ms": ms, "gbs": gbs,
                        "bytes_per_clk_per_sm_at_1.9ghz": gbs * 1e9 / (148 * 1.9e9)})
    tma = []
    for rb in (128, 256, 512):
        for name, rows in (("random rows, 64 MB table (L2-resident)", (64 << 20) // rb),
                           ("random rows, 546186-row table", 546186)):
            for ctas in (1, 2, 3):
                gbs, ms, _, done = ctx.probe_tma_gather(rb, rows, n, ctas, 10)
                tma.append({"row_bytes": rb, "pattern": name, "ctas_per_sm": ctas, "table_mb": rows * rb / 1e6, "ms": ms,
                            "gbs": gbs, "gathers": done, "bytes_per_clk_per_sm_at_1.9ghz": gbs * 1e9 / (148 * 1.9e9)})
    ctx.close()
    print(json.dumps({"ceilings": out, "tma_gather4": tma, "gathers_per_launch": n}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only-k", type=int, default=0, help="profiling aid (one GPU): run a single K")
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3"],
                    help="cfg2 (default): the power-law benchmark graph; cfg3: the uniform sparse graph at K = 64 with B "
                         "replicated (a secondary measurement, kernel time only)")
    ap.add_argument("--ceilings", action="store_true",
                    help="one GPU: measure the load-path ceilings (bare gathers) instead of the benchmark")
    ap.add_argument("--row-weight", type=float, default=8.0,
                    help="N > 1: cut the row blocks by entries + ROW_WEIGHT per row (0 = by entries alone).  A block of "
                         "many short rows owns more vertices, hence sends more rows of B; on the benchmark graph the "
                         "step is shortest around 8 to 12")
    ap.add_argument("--narrow-first", action="store_true",
                    help="N > 1: begin the exchanges in the order K = 32, 64, 128 instead of widest first")
    ap.add_argument("--no-compare", action="store_true",
                    help="skip the off-path comparison columns (cuSPARSE and the reference's kernels at N = 1, "
                         "the plain all-gather at N > 1)")
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
            run_reference_arm(args, pkg, max(world, args.gpus))
        return 0

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    if args.ceilings:
        if rank == 0:
            run_ceilings(pkg)
        return 0
    if args.workload == "cfg3":
        return run_cfg3_replicated(args, pkg, rank, local_rank, world)
    if world == 1:
        return run_single(args, pkg)
    return run_sharded(args, pkg, rank, local_rank, world)


if __name__ == "__main__":
    sys.exit(main())
