"""Generates the golden vectors under tests/golden/ from the REFERENCE's own kernels.

Run on a B200 (the reference is CUDA-only), after `make -C oracle ref` has built
oracle/_ref/libref_spmm.so from the reference's sources:

    python tests/golden/make_golden.py [--out DIR] [--time-bench-graph] [--only-cfg2]

For every case it stores the inputs and what the reference's GESpMM (CSR, overwrite) and
LBSpMM (padded COO, 200 accumulating launches, divided by 200 as the reference's checker
does) leave in C.  The power-law benchmark graph (R-MAT scale 20, K = 32) is stored as sampled rows plus
column sums (cfg2_k32_sampled_rows.npz; --only-cfg2 writes that file alone).  --time-bench-graph additionally times both reference entry points on the
benchmark graph (R-MAT scale 20) and writes the milliseconds to reference_timings.json.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def load_ref():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_spmm.so"))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_float)
    lib.ref_gespmm.argtypes = [I, I, I, I, P, P, P, P, P, F]
    lib.ref_lbspmm.argtypes = [I, I, I, I, P, P, P, P, P, F]
    return lib


def run_ref(lib, g, B, oracle_lib):
    M, N, nnz, K = g["M"], g["N"], g["nnz"], B.shape[1]
    ms = ctypes.c_float()
    C_ge = np.empty((M, K), dtype=np.float32)
    rc = lib.ref_gespmm(M, N, K, nnz, g["row_ptr"].ctypes.data, g["col_idx"].ctypes.data,
                        g["vals"].ctypes.data, B.ctypes.data, C_ge.ctypes.data, ctypes.byref(ms))
    assert rc == 0
    ge_ms = ms.value
    r, c, v = oracle_lib.csr_to_coo_padded(g["row_ptr"], g["col_idx"], g["vals"], 32)
    C_lb = np.empty((M, K), dtype=np.float32)
    rc = lib.ref_lbspmm(M, N, K, len(r), r.ctypes.data, c.ctypes.data, v.ctypes.data, B.ctypes.data,
                        C_lb.ctypes.data, ctypes.byref(ms))
    assert rc == 0
    launches = lib.ref_launches_per_call()
    C_lb = (C_lb / np.float32(launches)).astype(np.float32)   # spmm/utils/compare.cpp:12-13
    return C_ge, C_lb, ge_ms, ms.value


def cfg2_sample_rows(row_ptr):
    """The rows of the scale-20 benchmark graph that are stored: the four heaviest, 120 spread over the rows that
    hold entries, and four empty ones."""
    deg = np.diff(row_ptr)
    heavy = np.argsort(deg, kind="stable")[-4:]
    nonempty = np.flatnonzero(deg > 0)
    spread = nonempty[np.linspace(0, len(nonempty) - 1, 120).astype(np.int64)]
    empty = np.flatnonzero(deg == 0)[:4]
    return np.unique(np.concatenate([heavy, spread, empty])).astype(np.int64)


def golden_cfg2(pkg, lib, oracle_lib, out_dir):
    """The power-law benchmark configuration at full size (R-MAT scale 20, K = 32, the benchmark's seeds):
    inputs are regenerated from their seeds by the tests; sampled rows of both reference outputs and the
    column sums of GESpMM's are stored."""
    g = pkg.gen_rmat(20, 16, seed=2)
    K = 32
    B = pkg.host_fill_uniform(g["N"] * K, 2, 100 + K, -1.0, 1.0).reshape(g["N"], K)
    C_ge, C_lb, ge_ms, lb_ms = run_ref(lib, g, B, oracle_lib)
    rows = cfg2_sample_rows(g["row_ptr"])
    np.savez_compressed(os.path.join(out_dir, "cfg2_k32_sampled_rows.npz"), rows=rows, C_gespmm=C_ge[rows],
                        C_lbspmm_div200=C_lb[rows], col_sum_gespmm=C_ge.astype(np.float64).sum(axis=0))
    info = {"M": g["M"], "N": g["N"], "nnz": g["nnz"], "K": K, "rows_stored": int(len(rows)),
            "max_degree": int(np.diff(g["row_ptr"]).max()),
            "gespmm_equals_fp32_oracle": bool(np.array_equal(
                C_ge, oracle_lib.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B))),
            "gespmm_ms": ge_ms, "lbspmm_ms": lb_ms}
    json.dump(info, open(os.path.join(out_dir, "cfg2_k32_summary.json"), "w"), indent=1)
    return info


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--time-bench-graph", action="store_true")
    ap.add_argument("--only-cfg2", action="store_true")
    args = ap.parse_args()
    import __graft_entry__ as entry
    import oracle_lib
    pkg = entry.load_package()
    lib = load_ref()
    os.makedirs(args.out, exist_ok=True)

    if args.only_cfg2:
        print(json.dumps(golden_cfg2(pkg, lib, oracle_lib, args.out)))
        return

    cases = {
        "uniform512_k32": (pkg.gen_uniform_degree(512, 512, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1), 32),
        "rmat9_k64": (pkg.gen_rmat(9, 16, seed=2), 64),
        "rmat8_k128": (pkg.gen_rmat(8, 16, seed=3), 128),
    }
    summary = {}
    for name, (g, K) in cases.items():
        B = pkg.host_fill_uniform(g["N"] * K, 7, K, -1.0, 1.0).reshape(g["N"], K)
        C_ge, C_lb, ge_ms, lb_ms = run_ref(lib, g, B, oracle_lib)
        np.savez_compressed(os.path.join(args.out, name + ".npz"), row_ptr=g["row_ptr"], col_idx=g["col_idx"],
                            vals=g["vals"], B=B, C_gespmm=C_ge, C_lbspmm_div200=C_lb)
        summary[name] = {"M": g["M"], "N": g["N"], "nnz": g["nnz"], "K": K,
                         "max_degree": int(np.diff(g["row_ptr"]).max()),
                         "gespmm_equals_fp32_oracle": bool(np.array_equal(
                             C_ge, oracle_lib.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)))}

    # The small uniform-degree benchmark configuration (4096 x 4096, K = 32) at full size: inputs are regenerated from their seeds by the test;
    # 64 sampled rows of the reference's output are stored.
    g = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1)
    B = pkg.host_fill_uniform(4096 * 32, 1, 10, -1.0, 1.0).reshape(4096, 32)
    C_ge, C_lb, ge_ms, lb_ms = run_ref(lib, g, B, oracle_lib)
    rows = np.arange(0, 4096, 64)
    np.savez_compressed(os.path.join(args.out, "cfg1_sampled_rows.npz"), rows=rows, C_gespmm=C_ge[rows],
                        C_lbspmm_div200=C_lb[rows], col_sum_gespmm=C_ge.astype(np.float64).sum(axis=0))
    summary["cfg1"] = {"M": 4096, "N": 4096, "nnz": g["nnz"], "K": 32,
                       "gespmm_equals_fp32_oracle": bool(np.array_equal(
                           C_ge, oracle_lib.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B))),
                       "gespmm_ms": ge_ms, "lbspmm_ms": lb_ms}

    if args.time_bench_graph:
        g = pkg.gen_rmat(20, 16, seed=2)
        timings = {"graph": "rmat scale 20 ef 16 seed 2", "nnz": g["nnz"], "kernels": "reference sources recompiled for sm_100a"}
        for K in (32, 64, 128):
            B = pkg.host_fill_uniform(g["N"] * K, 2, 100 + K, -1.0, 1.0).reshape(g["N"], K)
            C_ge, C_lb, ge_ms, lb_ms = run_ref(lib, g, B, oracle_lib)
            ref, abs_sum = oracle_lib.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
            timings[str(K)] = {"gespmm_ms": ge_ms, "lbspmm_ms": lb_ms,
                               "gespmm_gflops": 2.0 * g["nnz"] * K / ge_ms / 1e6,
                               "lbspmm_gflops": 2.0 * g["nnz"] * K / lb_ms / 1e6,
                               "lbspmm_backward_err": float(np.max(np.abs(C_lb - ref) / np.maximum(abs_sum, 1e-30)))}
        json.dump(timings, open(os.path.join(args.out, "reference_timings.json"), "w"), indent=1)
        print(json.dumps(timings))
    summary["cfg2_k32"] = golden_cfg2(pkg, lib, oracle_lib, args.out)
    json.dump(summary, open(os.path.join(args.out, "summary.json"), "w"), indent=1)
    print(json.dumps(summary))


if __name__ == "__main__":
    main()
