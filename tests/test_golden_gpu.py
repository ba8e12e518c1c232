"""The CUDA path against golden vectors produced by the reference's own kernels."""
import os

import numpy as np
import pytest

from helpers import gpu_spmm, guarded_output

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["uniform512_k32", "rmat9_k64", "rmat8_k128"])
def test_csr_paths_against_reference_outputs(gpu_ctx, pkg, oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    rp, ci, v, B = z["row_ptr"], z["col_idx"], z["vals"], z["B"]
    # row-split algorithm: the reference's GESpMM arithmetic, bit for bit
    C = gpu_spmm(gpu_ctx, pkg, rp, ci, v, B, opts=pkg.Opts(algo=pkg.ALGO_ROW_SPLIT))
    assert np.array_equal(C, z["C_gespmm"])
    # nnz-balanced kernel: summation order differs, max relative error 1e-4 on well-conditioned elements
    C = gpu_spmm(gpu_ctx, pkg, rp, ci, v, B)
    _, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    ref = z["C_gespmm"].astype(np.float64)
    assert np.max(np.abs(C - ref) / np.maximum(abs_sum, 1e-30)) <= 1e-5
    well = (np.abs(ref) >= 1e-2 * abs_sum) & (abs_sum > 0)
    assert np.max(np.abs(C - ref)[well] / np.abs(ref)[well]) <= 1e-4
    assert np.max(np.abs(C - z["C_lbspmm_div200"]) / np.maximum(abs_sum, 1e-30)) <= 2e-5


@pytest.mark.parametrize("name", ["uniform512_k32", "rmat9_k64", "rmat8_k128"])
def test_coo_path_against_reference_lbspmm(gpu_ctx, pkg, oracle, name):
    ctx = gpu_ctx
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    rp, ci, v, B = z["row_ptr"], z["col_idx"], z["vals"], z["B"]
    M, (N, K) = len(rp) - 1, B.shape
    r, c, vv = oracle.csr_to_coo_padded(rp, ci, v, 32)
    d_r, d_c, d_v, d_B = ctx.upload(r), ctx.upload(c), ctx.upload(vv), ctx.upload(B)
    buf, ptr, read = guarded_output(ctx, (M, K), fill=np.float32(0))
    ctx.spmm_coo(M, N, K, len(r), d_r, d_c, d_v, d_B, ptr)
    ctx.stream_sync()
    C = read()
    _, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    assert np.max(np.abs(C - z["C_lbspmm_div200"]) / np.maximum(abs_sum, 1e-30)) <= 2e-5
    assert oracle.max_abs_err(C, z["C_gespmm"]) < 0.1     # the reference checker's criterion
    for b in (d_r, d_c, d_v, d_B, buf):
        b.free()


def test_cfg1_against_reference_rows(gpu_ctx, pkg):
    z = np.load(os.path.join(GOLDEN, "cfg1_sampled_rows.npz"))
    g = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1)
    B = pkg.host_fill_uniform(4096 * 32, 1, 10, -1.0, 1.0).reshape(4096, 32)
    C = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, opts=pkg.Opts(algo=pkg.ALGO_ROW_SPLIT))
    assert np.array_equal(C[z["rows"]], z["C_gespmm"])
    C = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B)
    assert np.allclose(C[z["rows"]], z["C_gespmm"], rtol=1e-4, atol=1e-5)


def test_cfg2_against_reference_rows(gpu_ctx, pkg, oracle):
    """The benchmark graph at K = 32 against sampled rows of the reference's own outputs: the row-split
    algorithm bit for bit, the balanced kernel (with the plan the benchmark uses) within the tolerance."""
    from helpers import BACKWARD_TOL
    z = np.load(os.path.join(GOLDEN, "cfg2_k32_sampled_rows.npz"))
    g = pkg.gen_rmat(20, 16, seed=2)
    B = pkg.host_fill_uniform(g["N"] * 32, 2, 132, -1.0, 1.0).reshape(g["N"], 32)
    rows = z["rows"]
    C = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, opts=pkg.Opts(algo=pkg.ALGO_ROW_SPLIT))
    assert np.array_equal(C[rows], z["C_gespmm"])
    C = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, use_plan=True)
    sub = np.concatenate([np.arange(g["row_ptr"][r], g["row_ptr"][r + 1]) for r in rows])
    sub_rp = np.concatenate([[0], np.cumsum(np.diff(g["row_ptr"])[rows])]).astype(np.int32)
    _, abs_sum = oracle.spmm_f64(sub_rp, g["col_idx"][sub], g["vals"][sub], B)
    ref = z["C_gespmm"].astype(np.float64)
    assert np.max(np.abs(C[rows] - ref) / np.maximum(abs_sum, 1e-30)) <= BACKWARD_TOL
    assert np.max(np.abs(C[rows] - z["C_lbspmm_div200"]) / np.maximum(abs_sum, 1e-30)) <= 1e-5
    assert np.allclose(C.astype(np.float64).sum(axis=0), z["col_sum_gespmm"], rtol=0, atol=0.05)
