"""Row reordering on the device: the reference's reordered COO emission (bit-exact against the oracle), the CSR
permutation, the degree order, and products on reordered operands (needs a B200)."""
import numpy as np
import pytest

from helpers import check_against_f64, random_csr

pytestmark = pytest.mark.gpu


def _graphs(pkg):
    yield "rmat", pkg.gen_rmat(12, 16, seed=41)
    yield "rect", pkg.gen_uniform_degree(3000, 1777, 0, 24, seed=42, vals_kind=pkg.VALS_UPM1)
    rp, ci, v = random_csr(40, 5000, [0, 0, 4000, 1, 0, 33, 32, 31] * 5, seed=43)   # heavy, empty, ragged rows
    yield "ragged", {"M": 40, "N": 5000, "nnz": len(ci), "row_ptr": rp, "col_idx": ci, "vals": v}


@pytest.mark.parametrize("padding", [32, 0, 7])
def test_reordered_coo_emission_is_bit_exact(gpu_ctx, pkg, oracle, padding):
    ctx = gpu_ctx
    for name, g in _graphs(pkg):
        M, nnz = g["M"], g["nnz"]
        order = np.random.default_rng(7).permutation(M).astype(np.int32)
        r, c, v = oracle.csr_to_coo_reordered(g["row_ptr"], g["col_idx"], g["vals"], order, padding)
        padded = len(r)
        d_rp, d_ci, d_v, d_o = (ctx.upload(a) for a in (g["row_ptr"], g["col_idx"], g["vals"], order))
        d_r, d_c, d_w = ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.float32)
        ctx.csr_to_coo_reordered(M, nnz, d_rp, d_ci, d_v, d_o, padding, d_r, d_c, d_w)
        assert np.array_equal(d_r.to_host(), r), name
        assert np.array_equal(d_c.to_host(), c), name
        assert np.array_equal(d_w.to_host(), v), name
        for b in (d_rp, d_ci, d_v, d_o, d_r, d_c, d_w):
            b.free()


def test_reordered_coo_feeds_the_accumulating_product(gpu_ctx, pkg, oracle):
    """The reference's reordered path: emission in permutation order, then the COO product into zeroed C."""
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=44)
    M, N, nnz, K = g["M"], g["N"], g["nnz"], 64
    B = pkg.host_fill_uniform(N * K, 44, 1, -1.0, 1.0).reshape(N, K)
    d_rp, d_ci, d_v, d_B = (ctx.upload(a) for a in (g["row_ptr"], g["col_idx"], g["vals"], B))
    d_o = ctx.alloc((M,), np.int32)
    ctx.order_rows_by_degree(M, d_rp, d_o)
    padded = (nnz + 31) // 32 * 32
    d_r, d_c, d_w = ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.int32), ctx.alloc((padded,), np.float32)
    ctx.csr_to_coo_reordered(M, nnz, d_rp, d_ci, d_v, d_o, 32, d_r, d_c, d_w)
    d_C = ctx.alloc((M, K), np.float32)
    ctx.fill(d_C, M * K, 0.0)
    ctx.spmm_coo(M, N, K, padded, d_r, d_c, d_w, d_B, d_C)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    check_against_f64(d_C.to_host(), ref, abs_sum, "reordered COO product")
    for b in (d_rp, d_ci, d_v, d_B, d_o, d_r, d_c, d_w, d_C):
        b.free()


def test_degree_order_and_inverse(gpu_ctx, pkg):
    ctx = gpu_ctx
    for name, g in _graphs(pkg):
        M = g["M"]
        deg = np.diff(g["row_ptr"].astype(np.int64))
        want = np.argsort(-deg, kind="stable").astype(np.int32)
        d_rp = ctx.upload(g["row_ptr"])
        d_o, d_inv = ctx.alloc((M,), np.int32), ctx.alloc((M,), np.int32)
        ctx.order_rows_by_degree(M, d_rp, d_o)
        ctx.invert_permutation(M, d_o, d_inv)
        got = d_o.to_host()
        assert np.array_equal(got, want), name
        inv = d_inv.to_host()
        assert np.array_equal(inv[got], np.arange(M, dtype=np.int32)), name
        for b in (d_rp, d_o, d_inv):
            b.free()


@pytest.mark.parametrize("symmetric", [False, True])
def test_csr_permute_and_product_in_the_new_numbering(gpu_ctx, pkg, oracle, symmetric):
    """A' = P A (Q): integer arrays equal the numpy restatement; the product on A' with B carried into the new
    column numbering, carried back by the inverse row gather, equals the product on A."""
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=45)
    M, N, nnz, K = g["M"], g["N"], g["nnz"], 32
    rp, ci, v = g["row_ptr"], g["col_idx"], g["vals"]
    order = np.random.default_rng(9).permutation(M).astype(np.int32)
    inv = np.empty(M, dtype=np.int32)
    inv[order] = np.arange(M, dtype=np.int32)
    # numpy restatement of the permutation
    lens = (rp[1:] - rp[:-1])[order]
    rp2 = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    src = np.concatenate([np.arange(rp[r], rp[r + 1]) for r in order]) if nnz else np.zeros(0, dtype=np.int64)
    ci2 = (inv[ci[src]] if symmetric else ci[src]).astype(np.int32)
    v2 = v[src]

    d_rp, d_ci, d_v, d_o, d_inv = (ctx.upload(a) for a in (rp, ci, v, order, inv))
    d_rp2, d_ci2, d_v2 = ctx.alloc((M + 1,), np.int32), ctx.alloc((nnz,), np.int32), ctx.alloc((nnz,), np.float32)
    ctx.csr_permute(M, N, nnz, d_rp, d_ci, d_v, d_o, d_inv if symmetric else None, d_rp2, d_ci2, d_v2)
    assert np.array_equal(d_rp2.to_host(), rp2)
    assert np.array_equal(d_ci2.to_host(), ci2)
    assert np.array_equal(d_v2.to_host(), v2)

    B = pkg.host_fill_uniform(N * K, 45, 1, -1.0, 1.0).reshape(N, K)
    d_B = ctx.upload(B)
    d_B2 = ctx.alloc((N, K), np.float32)
    if symmetric:
        ctx.gather_rows(N, K, d_B, d_o, d_B2)          # B'[i] = B[order[i]]: row inv[c] of B' is row c of B
        assert np.array_equal(d_B2.to_host(), B[order])
    d_C2, d_C = ctx.alloc((M, K), np.float32), ctx.alloc((M, K), np.float32)
    ctx.spmm_csr(M, N, K, nnz, d_rp2, d_ci2, d_v2, d_B2 if symmetric else d_B, d_C2)
    ctx.gather_rows(M, K, d_C2, d_inv, d_C)            # C[r] = C'[inv[r]]
    ref, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    check_against_f64(d_C.to_host(), ref, abs_sum, "product in the new numbering")
    for b in (d_rp, d_ci, d_v, d_o, d_inv, d_rp2, d_ci2, d_v2, d_B, d_B2, d_C2, d_C):
        b.free()


def test_gather_rows_unaligned_width(gpu_ctx, pkg):
    ctx = gpu_ctx
    src = np.arange(50 * 7, dtype=np.float32).reshape(50, 7)
    order = np.random.default_rng(3).permutation(50).astype(np.int32)
    d_s, d_o, d_d = ctx.upload(src), ctx.upload(order), ctx.alloc((50, 7), np.float32)
    ctx.gather_rows(50, 7, d_s, d_o, d_d)
    assert np.array_equal(d_d.to_host(), src[order])
    for b in (d_s, d_o, d_d):
        b.free()


def test_bad_row_orders_are_refused(gpu_ctx, pkg):
    ctx = gpu_ctx
    g = pkg.gen_uniform_degree(64, 64, 1, 4, seed=3)
    nnz = g["nnz"]
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    d_r, d_c, d_w = ctx.alloc((nnz,), np.int32), ctx.alloc((nnz,), np.int32), ctx.alloc((nnz,), np.float32)
    d_rp2 = ctx.alloc((65,), np.int32)
    for bad in (np.zeros(64, dtype=np.int32), np.arange(1, 65, dtype=np.int32), np.full(64, -1, dtype=np.int32)):
        d_o = ctx.upload(bad)
        with pytest.raises(pkg.HpspmmError) as ei:
            ctx.csr_to_coo_reordered(64, nnz, d_rp, d_ci, d_v, d_o, 0, d_r, d_c, d_w)
        assert ei.value.status == pkg.ERR_INVALID
        with pytest.raises(pkg.HpspmmError):
            ctx.csr_permute(64, 64, nnz, d_rp, d_ci, d_v, d_o, None, d_rp2, d_c, d_w)
        d_o.free()
    for b in (d_rp, d_ci, d_v, d_r, d_c, d_w, d_rp2):
        b.free()
