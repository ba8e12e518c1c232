"""The large benchmark configurations at full size, checked through sampled rows.

B is filled on the device by the library's counter-based generator, so the rows of B that a sampled row
of A needs can be regenerated on the host (helpers.uniform_rows) without holding the 8.6 GB operand: every
sampled row of C (the heaviest, the first, the last, rows behind the 2^31-element mark, rows whose columns
lie behind it) is compared with a float64 sum over those regenerated rows.  A wrong 64-bit offset into B or
C shows up as a wrong row.  The uniform sparse case is also compared with the oracle in full.
"""
import numpy as np
import pytest

from helpers import BACKWARD_TOL, check_against_f64, uniform_rows

pytestmark = pytest.mark.gpu


def _rows_vs_f64(ctx, pkg, g, K, sample_rows, seed, stream_id, use_plan=True):
    M, N, nnz = g["M"], g["N"], g["nnz"]
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    d_B = ctx.alloc((N, K), np.float32)
    ctx.fill_uniform(d_B, N * K, seed, stream_id, -1.0, 1.0)
    d_C = ctx.alloc((M, K), np.float32)
    ctx.fill(d_C, M * K, -5.0)                      # stale data must be overwritten everywhere
    plan = ctx.plan_create(M, nnz, d_rp, K, N=N, col_idx=d_ci) if use_plan else None
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan)
    ctx.stream_sync()
    rp = g["row_ptr"].astype(np.int64)
    worst = 0.0
    for r in sample_rows:
        got = np.empty(K, dtype=np.float32)
        ctx.memcpy_d2h(got, d_C.ptr + int(r) * K * 4)
        ctx.stream_sync()
        cols = g["col_idx"][rp[r]:rp[r + 1]]
        if len(cols) == 0:
            assert np.all(got == 0), r
            continue
        vals = g["vals"][rp[r]:rp[r + 1]].astype(np.float64)
        Brows = uniform_rows(seed, stream_id, cols, K, -1.0, 1.0).astype(np.float64)
        want = vals @ Brows
        scale = np.abs(vals) @ np.abs(Brows)
        err = float(np.max(np.abs(got - want) / np.maximum(scale, 1e-30)))
        worst = max(worst, err)
        assert err <= BACKWARD_TOL, (r, len(cols), err, got[:4], want[:4])
    if plan:
        ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_v, d_B, d_C):
        b.free()
    return worst


def _sample(g, extra=()):
    deg = np.diff(g["row_ptr"])
    M = g["M"]
    rows = {0, 1, M - 1, M - 2, M // 2, int(deg.argmax())}
    rows.update(int(r) for r in np.argsort(deg)[-4:])            # heaviest rows
    rows.update(int(r) for r in np.flatnonzero(deg == 0)[:3])    # empty rows
    rows.update(int(r) for r in np.random.default_rng(0).integers(0, M, 40))
    rows.update(extra)
    return sorted(rows)


def test_cfg3_erdos_renyi_full_size(gpu_ctx, pkg, oracle):
    """Uniform sparse case: M = N = 2,450,000, Poisson(50) degrees, K = 64, against the oracle."""
    ctx = gpu_ctx
    g = pkg.gen_erdos_renyi(2_450_000, 2_450_000, 50.0, seed=3)
    assert 121_000_000 < g["nnz"] < 124_000_000
    _rows_vs_f64(ctx, pkg, g, 64, _sample(g), 3, 64)
    K, M, N, nnz = 64, g["M"], g["N"], g["nnz"]
    B = pkg.host_fill_uniform(N * K, 3, 64, -1.0, 1.0).reshape(N, K)
    d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
    d_C = ctx.alloc((M, K), np.float32)
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C)
    C = d_C.to_host()
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    check_against_f64(C, ref, abs_sum, "cfg3")
    for b in (d_rp, d_ci, d_v, d_B, d_C):
        b.free()


def _rows_with_columns_from(g, first_col, count):
    """Rows that hold an entry whose column is at least first_col."""
    pos = np.flatnonzero(g["col_idx"] >= first_col)
    if len(pos) == 0:
        return []
    pick = pos[np.linspace(0, len(pos) - 1, count).astype(np.int64)]
    return [int(r) for r in np.searchsorted(g["row_ptr"], pick, side="right") - 1]


def test_offsets_beyond_2_31_elements(gpu_ctx, pkg):
    """N*K and M*K above 2^31 elements: the dense operands need 64-bit offsets, into C (rows behind the mark)
    and into B (columns behind the mark)."""
    M = N = 17_500_000
    K = 128
    g = pkg.gen_uniform_degree(M, N, 0, 6, seed=9, vals_kind=pkg.VALS_UPM1)
    mark = 2 ** 31 // K                                  # first row / column whose element offset exceeds 2^31
    assert M > mark
    last = [M - 1 - i for i in range(0, 200, 7)]         # rows of C behind the mark
    far = _rows_with_columns_from(g, mark, 40)           # rows of A that read B behind the mark
    assert len(far) == 40 and all(np.any(g["col_idx"][g["row_ptr"][r]:g["row_ptr"][r + 1]] >= mark) for r in far)
    _rows_vs_f64(gpu_ctx, pkg, g, K, _sample(g, last + far), 9, 1, use_plan=False)


def test_cfg4_rmat_scale24_k128(gpu_ctx, pkg):
    """Large skewed case: R-MAT scale 24 (about 263 M entries, max degree > 10^5), K = 128, B = 8.6 GB of U(-1,1)
    (N*K = 2^31 elements exactly: the last rows of B and C sit at byte offsets beyond 2^33)."""
    g = pkg.gen_rmat(24, 16, seed=4)
    deg = np.diff(g["row_ptr"])
    assert g["M"] == 1 << 24 and g["nnz"] > 250_000_000 and deg.max() > 100_000
    far = _rows_with_columns_from(g, g["N"] - 4096, 20)  # rows that read the last rows of B
    _rows_vs_f64(gpu_ctx, pkg, g, 128, _sample(g, far), 4, 128)


def test_cfg5_gnn_layer_full_size(gpu_ctx, pkg, oracle):
    """A GNN layer on the R-MAT scale-20 graph at K = 64: forward C = A H, SDDMM dA = pattern(A) .* (dC H^T),
    backward dH = A^T dC through the transposed CSR built on the device; one plan reused."""
    ctx = gpu_ctx
    K = 64
    g = pkg.gen_rmat(20, 16, seed=2)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    H = pkg.host_fill_uniform(N * K, 5, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(M * K, 5, 2, -1.0, 1.0).reshape(M, K)
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    d_H, d_dC = ctx.upload(H), ctx.upload(dC)
    d_C = ctx.alloc((M, K), np.float32)
    d_dA = ctx.alloc((nnz,), np.float32)
    plan = ctx.plan_create(M, nnz, d_rp, K, N=N, col_idx=d_ci)
    # forward
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_H, d_C, plan=plan)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], H)
    check_against_f64(d_C.to_host(), ref, abs_sum, "cfg5 forward")
    # SDDMM over the pattern
    ctx.sddmm_csr(M, N, K, nnz, d_rp, d_ci, d_dC, d_H, d_dA, plan=plan)
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], dC, H)
    check_against_f64(d_dA.to_host(), ref, abs_sum, "cfg5 sddmm")
    # backward through the device transpose
    d_rpt, d_cit, d_vt = ctx.alloc((N + 1,), np.int32), ctx.alloc((nnz,), np.int32), ctx.alloc((nnz,), np.float32)
    ctx.csr_transpose(M, N, nnz, d_rp, d_ci, d_v, d_rpt, d_cit, d_vt)
    rpt, cit, vt, _ = oracle.csr_transpose(M, N, g["row_ptr"], g["col_idx"], g["vals"])
    assert np.array_equal(d_rpt.to_host(), rpt) and np.array_equal(d_cit.to_host(), cit)
    assert np.array_equal(d_vt.to_host(), vt)
    d_dH = ctx.alloc((N, K), np.float32)
    plan_t = ctx.plan_create(N, nnz, d_rpt, K, N=M, col_idx=d_cit)
    ctx.spmm_csr(N, M, K, nnz, d_rpt, d_cit, d_vt, d_dC, d_dH, plan=plan_t)
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, dC)
    check_against_f64(d_dH.to_host(), ref, abs_sum, "cfg5 backward")
    ctx.plan_destroy(plan)
    ctx.plan_destroy(plan_t)
    for b in (d_rp, d_ci, d_v, d_H, d_dC, d_C, d_dA, d_rpt, d_cit, d_vt, d_dH):
        b.free()


def test_cfg2_graph_at_k256_runs_as_two_slabs(gpu_ctx, pkg, oracle):
    """The R-MAT scale-20 graph at K = 256 (two strided 128-column slabs): the product against the oracle, the COO
    product and the SDDMM on the same operands."""
    ctx = gpu_ctx
    K = 256
    g = pkg.gen_rmat(20, 16, seed=2)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    B = pkg.host_fill_uniform(N * K, 2, 256, -1.0, 1.0).reshape(N, K)
    d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
    d_C = ctx.alloc((M, K), np.float32)
    plan = ctx.plan_create(M, nnz, d_rp, K, N=N, col_idx=d_ci)
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    check_against_f64(d_C.to_host(), ref, abs_sum, "K=256 CSR")
    # COO contract on the same graph: zero C, accumulate once
    padded = (nnz + 31) // 32 * 32
    d_r, d_c, d_w = ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.float32)
    ctx.csr_to_coo_padded(M, nnz, d_rp, d_ci, d_v, 32, d_r, d_c, d_w)
    ctx.fill(d_C, M * K, 0.0)
    ctx.spmm_coo(M, N, K, padded, d_r, d_c, d_w, d_B, d_C)
    check_against_f64(d_C.to_host(), ref, abs_sum, "K=256 COO")
    del ref, abs_sum
    # SDDMM with X = a second dense matrix
    X = pkg.host_fill_uniform(M * K, 2, 257, -1.0, 1.0).reshape(M, K)
    d_X = ctx.upload(X)
    d_o = ctx.alloc((nnz,), np.float32)
    ctx.sddmm_csr(M, N, K, nnz, d_rp, d_ci, d_X, d_B, d_o, plan=plan)
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], X, B)
    check_against_f64(d_o.to_host(), ref, abs_sum, "K=256 SDDMM")
    ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_v, d_B, d_C, d_r, d_c, d_w, d_X, d_o):
        b.free()
