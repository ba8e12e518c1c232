"""The CPU oracle against scipy.sparse and hand-computed cases (no GPU)."""
import numpy as np
import pytest
import scipy.sparse as sp

from helpers import random_csr


@pytest.fixture(scope="module")
def case():
    rng = np.random.default_rng(7)
    M, N, K = 300, 257, 32
    deg = rng.integers(0, 40, size=M)
    deg[5] = 0
    deg[6] = 0
    deg[100] = 200
    row_ptr, col_idx, vals = random_csr(M, N, deg, seed=3)
    B = rng.uniform(-1, 1, size=(N, K)).astype(np.float32)
    return M, N, K, row_ptr, col_idx, vals, B


def test_spmm_matches_scipy(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    A = sp.csr_matrix((vals.astype(np.float64), col_idx, row_ptr), shape=(M, N))
    want = A @ B.astype(np.float64)
    got64, abs_sum = oracle.spmm_f64(row_ptr, col_idx, vals, B)
    assert np.allclose(got64, want, rtol=1e-12, atol=1e-12)
    got32 = oracle.spmm_f32(row_ptr, col_idx, vals, B)
    assert np.max(np.abs(got32 - want) / np.maximum(abs_sum, 1e-30)) < 1e-5
    assert np.all(got32[5] == 0) and np.all(got32[6] == 0)
    absA = sp.csr_matrix((np.abs(vals).astype(np.float64), col_idx, row_ptr), shape=(M, N))
    assert np.allclose(abs_sum, absA @ np.abs(B.astype(np.float64)), rtol=1e-12, atol=1e-12)


def test_spmm_f32_is_sequential_fma(oracle):
    # hand-rolled single row: acc = fma(v, b, acc) in storage order, in float32
    row_ptr = np.array([0, 4], dtype=np.int32)
    col_idx = np.array([2, 0, 1, 3], dtype=np.int32)  # storage order, not sorted
    vals = np.array([1e8, 1.0, -1e8, 0.5], dtype=np.float32)
    B = np.ones((4, 1), dtype=np.float32)
    got = oracle.spmm_f32(row_ptr, col_idx, vals, B)
    acc = np.float32(0)
    for v in vals:
        acc = np.float32(np.float64(v) * 1.0 + np.float64(acc))  # exact product, one rounding
    assert got[0, 0] == acc == np.float32(0.5)  # 1e8 + 1 rounds back to 1e8 in fp32


def test_coo_padded_and_product(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    r, c, v = oracle.csr_to_coo_padded(row_ptr, col_idx, vals, 32)
    nnz = len(col_idx)
    assert len(r) % 32 == 0 and len(r) - nnz < 32
    A = sp.csr_matrix((vals, col_idx, row_ptr), shape=(M, N)).tocoo()
    assert np.array_equal(r[:nnz], A.row) and np.array_equal(c[:nnz], col_idx)
    assert np.all(r[nnz:] == 0) and np.all(c[nnz:] == 0) and np.all(v[nnz:] == 0)
    C = oracle.spmm_coo_f32(M, r, c, v, B)
    assert np.array_equal(C, oracle.spmm_f32(row_ptr, col_idx, vals, B))  # same order -> same bits


def test_coo_reordered(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    order = np.random.default_rng(1).permutation(M).astype(np.int32)
    r, c, v = oracle.csr_to_coo_reordered(row_ptr, col_idx, vals, order, 32)
    t = 0
    for i in order:
        n = row_ptr[i + 1] - row_ptr[i]
        assert np.all(r[t:t + n] == i)
        assert np.array_equal(c[t:t + n], col_idx[row_ptr[i]:row_ptr[i + 1]])
        t += n
    assert t == len(col_idx) and np.all(v[t:] == 0)
    C = oracle.spmm_coo_f32(M, r, c, v, B)
    assert np.array_equal(C, oracle.spmm_f32(row_ptr, col_idx, vals, B))


def test_sddmm_matches_scipy(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    rng = np.random.default_rng(11)
    X = rng.uniform(-1, 1, size=(M, K)).astype(np.float32)
    want = np.einsum("jk,jk->j", X.astype(np.float64)[np.repeat(np.arange(M), np.diff(row_ptr))],
                     B.astype(np.float64)[col_idx])
    got64, abs_sum = oracle.sddmm_f64(row_ptr, col_idx, X, B)
    assert np.allclose(got64, want, rtol=1e-12, atol=1e-12)
    got32 = oracle.sddmm_f32(row_ptr, col_idx, X, B)
    assert np.max(np.abs(got32 - want) / np.maximum(abs_sum, 1e-30)) < 1e-5


def test_transpose_matches_scipy(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    rpt, cit, vt, perm = oracle.csr_transpose(M, N, row_ptr, col_idx, vals)
    At = sp.csr_matrix((vals, col_idx, row_ptr), shape=(M, N)).T.tocsr()
    At.sort_indices()
    assert np.array_equal(rpt, At.indptr) and np.array_equal(cit, At.indices)
    assert np.array_equal(vt, At.data)
    assert np.array_equal(vals[perm], vt) and np.array_equal(col_idx[perm], np.repeat(np.arange(N), np.diff(rpt)))
    for c in range(N):  # ascending source rows inside every transposed row
        assert np.all(np.diff(cit[rpt[c]:rpt[c + 1]]) > 0)


def test_shard_bounds(oracle, case):
    M, N, K, row_ptr, col_idx, vals, B = case
    nnz = row_ptr[-1]
    for G in (1, 2, 3, 4, 8):
        b = oracle.shard_bounds(row_ptr, G)
        assert b[0] == 0 and b[-1] == M and np.all(np.diff(b) >= 0)
        for g in range(1, G):
            target = nnz * g // G
            assert row_ptr[b[g]] >= target and (b[g] == 0 or row_ptr[b[g] - 1] < target)


def test_metric_formulas(oracle):
    assert oracle.gflops(16_777_216, 64, 1.0) == pytest.approx(2 * 16_777_216 * 64 / 1e6)
    row_ptr = np.array([0, 1, 3, 6, 10], dtype=np.int32)
    lens = np.array([1, 2, 3, 4], dtype=np.float64)
    assert oracle.row_length_cv(row_ptr) == pytest.approx(lens.std() / lens.mean())
    a = np.array([200.0, 400.0], dtype=np.float32)
    b = np.array([1.0, 2.05], dtype=np.float32)
    assert oracle.max_abs_err(a, b, True) == pytest.approx(0.05, abs=1e-6)
    assert oracle.max_abs_err(a, b, False) == pytest.approx(398.0, rel=1e-3)
