"""COO SpMM (accumulating), SDDMM, CSR transpose, COO expansion and validation on the GPU."""
import numpy as np
import pytest

from helpers import check_against_f64, guarded_output, random_csr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [32, 64, 128, 20, 7, 640, 96, 160, 256, 512])
def test_coo_accumulates_like_lbspmm(gpu_ctx, pkg, oracle, K):
    ctx = gpu_ctx
    g = pkg.gen_rmat(11, 16, seed=5)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    B = pkg.host_fill_uniform(N * K, 5, K, -1.0, 1.0).reshape(N, K)
    r, c, v = oracle.csr_to_coo_padded(g["row_ptr"], g["col_idx"], g["vals"], 32)
    d_r, d_c, d_v, d_B = ctx.upload(r), ctx.upload(c), ctx.upload(v), ctx.upload(B)
    buf, c_ptr, read = guarded_output(ctx, (M, K), fill=np.float32(0))
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    ctx.spmm_coo(M, N, K, len(r), d_r, d_c, d_v, d_B, c_ptr)
    ctx.stream_sync()
    check_against_f64(read(), ref, abs_sum, "coo first call")
    ctx.spmm_coo(M, N, K, len(r), d_r, d_c, d_v, d_B, c_ptr)   # a second call adds again
    ctx.stream_sync()
    check_against_f64(read() / 2.0, ref, abs_sum, "coo second call")
    # the reference's checker convention: max abs error < 0.1 against the fp32 CSR product
    assert oracle.max_abs_err(read() / 2.0, oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)) < 0.1
    for b in (d_r, d_c, d_v, d_B, buf):
        b.free()


def test_coo_reordered_rows_and_nan_in_padding_row(gpu_ctx, pkg, oracle):
    ctx = gpu_ctx
    K = 32
    g = pkg.gen_uniform_degree(500, 400, 0, 12, seed=6)
    M, N = g["M"], g["N"]
    B = pkg.host_fill_uniform(N * K, 6, 1, -1.0, 1.0).reshape(N, K).copy()
    order = np.random.default_rng(2).permutation(M).astype(np.int32)
    r, c, v = oracle.csr_to_coo_reordered(g["row_ptr"], g["col_idx"], g["vals"], order, 32)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    # padding entries point at B[0,:]; poison it in rows that do not use column 0
    uses_col0 = np.zeros(M, dtype=bool)
    uses_col0[np.repeat(np.arange(M), np.diff(g["row_ptr"]))[g["col_idx"] == 0]] = True
    Bp = B.copy()
    Bp[0, :] = np.nan
    d_r, d_c, d_v, d_B = ctx.upload(r), ctx.upload(c), ctx.upload(v), ctx.upload(Bp)
    buf, c_ptr, read = guarded_output(ctx, (M, K), fill=np.float32(0))
    ctx.spmm_coo(M, N, K, len(r), d_r, d_c, d_v, d_B, c_ptr)
    ctx.stream_sync()
    C = read()
    assert np.all(np.isfinite(C[~uses_col0]))          # padding did not leak NaN into row 0
    keep = ~uses_col0
    check_against_f64(C[keep], ref[keep], abs_sum[keep], "coo reordered")
    for b in (d_r, d_c, d_v, d_B, buf):
        b.free()


@pytest.mark.parametrize("K", [32, 64, 128, 48, 224])
@pytest.mark.parametrize("order", ["shuffled", "heavy_rows", "padded_inside"])
def test_coo_triples_in_any_order(gpu_ctx, pkg, oracle, K, order):
    """The COO contract puts no order on the triples: entries of one row scattered over many chunks, runs of
    thousands of equal row ids, and zero-valued padding in the middle of the array all give A·B."""
    ctx = gpu_ctx
    rng = np.random.default_rng(17)
    if order == "heavy_rows":
        rp, ci, v = random_csr(12, 9000, [6000, 0, 1, 33, 2500, 31, 0, 4000, 2, 700, 64, 65], seed=18)
        M, N = 12, 9000
    else:
        g = pkg.gen_rmat(11, 16, seed=19)
        rp, ci, v, M, N = g["row_ptr"], g["col_idx"], g["vals"], g["M"], g["N"]
    v = np.where(v == 0, np.float32(0.5), v).astype(np.float32)     # keep stored entries distinguishable from padding
    r = np.repeat(np.arange(M, dtype=np.int32), np.diff(rp))
    c = ci.copy()
    w = v.copy()
    if order == "shuffled":
        p = rng.permutation(len(r))
        r, c, w = r[p], c[p], w[p]
    elif order == "padded_inside":
        pos = np.sort(rng.choice(len(r) + 1, size=200, replace=True))
        r = np.insert(r, pos, 0).astype(np.int32)
        c = np.insert(c, pos, 0).astype(np.int32)
        w = np.insert(w, pos, np.float32(0)).astype(np.float32)
    B = pkg.host_fill_uniform(N * K, 17, K, -1.0, 1.0).reshape(N, K)
    ref, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    d_r, d_c, d_w, d_B = ctx.upload(r), ctx.upload(c), ctx.upload(w), ctx.upload(B)
    buf, c_ptr, read = guarded_output(ctx, (M, K), fill=np.float32(0))
    ctx.spmm_coo(M, N, K, len(r), d_r, d_c, d_w, d_B, c_ptr)
    ctx.stream_sync()
    check_against_f64(read(), ref, abs_sum, "coo %s K=%d" % (order, K))
    for b in (d_r, d_c, d_w, d_B, buf):
        b.free()


@pytest.mark.parametrize("K", [32, 64, 128, 4, 20, 33, 200, 1, 96, 160, 256, 512])
@pytest.mark.parametrize("use_plan", [False, True])
def test_sddmm(gpu_ctx, pkg, oracle, K, use_plan):
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=7)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    X = pkg.host_fill_uniform(M * K, 7, 1, -1.0, 1.0).reshape(M, K)
    Y = pkg.host_fill_uniform(N * K, 7, 2, -1.0, 1.0).reshape(N, K)
    d_rp, d_ci, d_X, d_Y = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(X), ctx.upload(Y)
    buf, o_ptr, read = guarded_output(ctx, (nnz,))
    plan = ctx.plan_create(M, nnz, d_rp, K, N=N, col_idx=d_ci) if use_plan else None
    ctx.sddmm_csr(M, N, K, nnz, d_rp, d_ci, d_X, d_Y, o_ptr, plan=plan)
    ctx.stream_sync()
    out = read()
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], X, Y)
    check_against_f64(out, ref, abs_sum, "sddmm K=%d" % K)
    if plan:
        ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_X, d_Y, buf):
        b.free()


def test_sddmm_edge_structures(gpu_ctx, pkg, oracle):
    ctx = gpu_ctx
    rng = np.random.default_rng(3)
    for M, N, deg in ((1, 9, [9]), (50, 64, [0] * 20 + [64] + [0] * 28 + [1]), (300, 200, rng.integers(0, 5, 300)),
                      (40, 1000, [1000] * 3 + [0] * 37)):
        row_ptr, col_idx, _ = random_csr(M, N, deg, seed=M)
        for K in (32, 128, 12):
            X = rng.uniform(-1, 1, size=(M, K)).astype(np.float32)
            Y = rng.uniform(-1, 1, size=(N, K)).astype(np.float32)
            nnz = len(col_idx)
            d_rp, d_ci, d_X, d_Y = ctx.upload(row_ptr), ctx.upload(col_idx), ctx.upload(X), ctx.upload(Y)
            buf, o_ptr, read = guarded_output(ctx, (nnz,))
            ctx.sddmm_csr(M, N, K, nnz, d_rp, d_ci, d_X, d_Y, o_ptr)
            ctx.stream_sync()
            ref, abs_sum = oracle.sddmm_f64(row_ptr, col_idx, X, Y)
            check_against_f64(read(), ref, abs_sum, "sddmm edge M=%d K=%d" % (M, K))
            for b in (d_rp, d_ci, d_X, d_Y, buf):
                b.free()


@pytest.mark.parametrize("shape", ["rmat13", "rect", "tiny", "wide", "cols_2_20", "cols_3m", "cols_5m"])
def test_transpose_bit_exact(gpu_ctx, pkg, oracle, shape):
    ctx = gpu_ctx
    if shape == "rmat13":
        g = pkg.gen_rmat(13, 16, seed=8)     # 13 bits of column index: two passes of 8-bit digits
        M, N, row_ptr, col_idx, vals = g["M"], g["N"], g["row_ptr"], g["col_idx"], g["vals"]
    elif shape == "rect":
        M, N = 777, 70001     # 17 bits of column index: two passes of 10-bit digits
        row_ptr, col_idx, vals = random_csr(M, N, np.random.default_rng(1).integers(0, 200, M), seed=1)
    elif shape.startswith("cols_"):
        # 20 bits: two 10-bit passes; 22 bits: two 11-bit passes; 23 bits: three 8-bit passes.  Many tiles
        # of 4096 entries, one heavy row and a hot column block so that digits repeat inside a warp.
        N = {"cols_2_20": 1 << 20, "cols_3m": 3_000_000, "cols_5m": 5_000_000}[shape]
        M = 3000
        rng = np.random.default_rng(N)
        deg = rng.integers(0, 120, M)
        deg[17] = 30000
        row_ptr, col_idx, vals = random_csr(M, N, deg, seed=N % 1000)
        hot = rng.random(len(col_idx)) < 0.2          # a fifth of the entries fall into 64 columns
        col_idx = np.where(hot, col_idx % 64, col_idx).astype(np.int32)
        for r in range(M):                            # keep rows sorted and duplicate-free
            seg = np.unique(col_idx[row_ptr[r]:row_ptr[r + 1]])
            col_idx[row_ptr[r]:row_ptr[r] + len(seg)] = seg
            deg[r] = len(seg)
        keep = np.concatenate([np.arange(row_ptr[r], row_ptr[r] + deg[r]) for r in range(M)])
        col_idx, vals = col_idx[keep].copy(), vals[keep].copy()
        row_ptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    elif shape == "tiny":
        M, N = 3, 2
        row_ptr, col_idx, vals = random_csr(M, N, [2, 0, 1], seed=2)
    else:
        M, N = 5, 300
        row_ptr, col_idx, vals = random_csr(M, N, [300, 0, 300, 1, 299], seed=3)
    nnz = len(col_idx)
    d_rp, d_ci, d_v = ctx.upload(row_ptr), ctx.upload(col_idx), ctx.upload(vals)
    d_rpt = ctx.alloc((N + 1,), np.int32)
    d_cit = ctx.alloc((nnz,), np.int32)
    d_vt = ctx.alloc((nnz,), np.float32)
    d_perm = ctx.alloc((nnz,), np.int32)
    for _ in range(2):   # twice: deterministic
        ctx.csr_transpose(M, N, nnz, d_rp, d_ci, d_v, d_rpt, d_cit, d_vt, d_perm)
        ctx.stream_sync()
        rpt, cit, vt, perm = oracle.csr_transpose(M, N, row_ptr, col_idx, vals)
        assert np.array_equal(d_rpt.to_host(), rpt)
        assert np.array_equal(d_cit.to_host(), cit)
        assert np.array_equal(d_vt.to_host(), vt)
        assert np.array_equal(d_perm.to_host(), perm)
    for b in (d_rp, d_ci, d_v, d_rpt, d_cit, d_vt, d_perm):
        b.free()


def test_transposed_product_matches(gpu_ctx, pkg, oracle):
    """dH = A^T dC through the device transpose equals the oracle's A^T product."""
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=9)
    M, N, nnz, K = g["M"], g["N"], g["nnz"], 64
    dC = pkg.host_fill_uniform(M * K, 9, 3, -1.0, 1.0).reshape(M, K)
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    d_rpt, d_cit, d_vt = ctx.alloc((N + 1,), np.int32), ctx.alloc((nnz,), np.int32), ctx.alloc((nnz,), np.float32)
    ctx.csr_transpose(M, N, nnz, d_rp, d_ci, d_v, d_rpt, d_cit, d_vt)
    d_dC = ctx.upload(dC)
    d_dH = ctx.alloc((N, K), np.float32)
    ctx.spmm_csr(N, M, K, nnz, d_rpt, d_cit, d_vt, d_dC, d_dH)
    ctx.stream_sync()
    rpt, cit, vt, _ = oracle.csr_transpose(M, N, g["row_ptr"], g["col_idx"], g["vals"])
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, dC)
    check_against_f64(d_dH.to_host(), ref, abs_sum, "A^T dC")
    for b in (d_rp, d_ci, d_v, d_rpt, d_cit, d_vt, d_dC, d_dH):
        b.free()


@pytest.mark.parametrize("padding", [32, 1, 0, 100])
def test_csr_to_coo_padded_bit_exact(gpu_ctx, pkg, oracle, padding):
    ctx = gpu_ctx
    g = pkg.gen_rmat(11, 8, seed=10)
    r, c, v = oracle.csr_to_coo_padded(g["row_ptr"], g["col_idx"], g["vals"], padding)
    lib = pkg.load_library()
    assert lib.hpspmm_padded_nnz(g["nnz"], padding) == len(r)
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    o_r, o_c, o_v = ctx.alloc((len(r),), np.int32), ctx.alloc((len(r),), np.int32), ctx.alloc((len(r),), np.float32)
    ctx.csr_to_coo_padded(g["M"], g["nnz"], d_rp, d_ci, d_v, padding, o_r, o_c, o_v)
    ctx.stream_sync()
    assert np.array_equal(o_r.to_host(), r) and np.array_equal(o_c.to_host(), c) and np.array_equal(o_v.to_host(), v)
    for b in (d_rp, d_ci, d_v, o_r, o_c, o_v):
        b.free()


def test_validate_csr(gpu_ctx, pkg):
    ctx = gpu_ctx
    g = pkg.gen_uniform_degree(200, 150, 0, 9, seed=11)
    M, N, nnz = g["M"], g["N"], g["nnz"]

    def run(rp, ci):
        d_rp, d_ci = ctx.upload(rp), ctx.upload(ci)
        out = ctx.validate_csr(M, N, nnz, d_rp, d_ci)
        d_rp.free()
        d_ci.free()
        return out

    assert run(g["row_ptr"], g["col_idx"]) == (pkg.OK, -1)
    rp = g["row_ptr"].copy()
    rp[50], rp[51] = rp[51] + 1, rp[50]            # not monotone
    st, pos = run(rp, g["col_idx"])
    assert st == pkg.ERR_BAD_CSR and 50 <= pos <= 52
    ci = g["col_idx"].copy()
    ci[17] = N                                     # column out of range
    assert run(g["row_ptr"], ci) == (pkg.ERR_BAD_CSR, M + 1 + 17)
    ci[17] = -1
    assert run(g["row_ptr"], ci) == (pkg.ERR_BAD_CSR, M + 1 + 17)
    rp = g["row_ptr"].copy()
    rp[-1] += 1                                    # row_ptr[M] != nnz
    assert run(rp, g["col_idx"])[0] == pkg.ERR_BAD_CSR
    assert run(g["row_ptr"], g["col_idx"]) == (pkg.OK, -1)   # the context is still usable
