"""ctypes face of oracle/liboracle.so, the CPU restatement used as the checker.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes
import os
import subprocess
from ctypes import c_double, c_int, c_int32, c_int64, c_void_p

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "liboracle.so")

_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    src = os.path.join(ORACLE_DIR, "oracle.c")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    L = ctypes.CDLL(LIB_PATH)
    P, I64 = c_void_p, c_int64
    L.oracle_num_threads.restype = c_int
    L.oracle_set_num_threads.argtypes = [c_int]
    L.oracle_spmm_csr_f32.argtypes = [I64, I64, P, P, P, P, P]
    L.oracle_spmm_csr_f64.argtypes = [I64, I64, P, P, P, P, P, P]
    L.oracle_spmm_coo_f32.argtypes = [I64, I64, P, P, P, P, P]
    L.oracle_sddmm_csr_f32.argtypes = [I64, I64, P, P, P, P, P]
    L.oracle_sddmm_csr_f64.argtypes = [I64, I64, P, P, P, P, P, P]
    L.oracle_csr_transpose.argtypes = [I64, I64, P, P, P, P, P, P, P]
    L.oracle_csr_to_coo_padded.argtypes = [I64, P, P, P, I64, P, P, P]
    L.oracle_csr_to_coo_padded.restype = I64
    L.oracle_csr_to_coo_reordered.argtypes = [I64, P, P, P, P, I64, P, P, P]
    L.oracle_csr_to_coo_reordered.restype = I64
    L.oracle_row_length_cv.argtypes = [I64, P]
    L.oracle_row_length_cv.restype = c_double
    L.oracle_gflops.argtypes = [I64, I64, c_double]
    L.oracle_gflops.restype = c_double
    L.oracle_shard_bounds.argtypes = [I64, P, c_int32, P]
    L.oracle_max_abs_err.argtypes = [I64, P, P, c_int]
    L.oracle_max_abs_err.restype = c_double
    _lib = L
    return L


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads():
    return lib().oracle_num_threads()


def spmm_f32(row_ptr, col_idx, vals, B, out=None):
    row_ptr, col_idx, vals, B = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(vals, np.float32), _c(B, np.float32)
    M, K = len(row_ptr) - 1, B.shape[1]
    C = out if out is not None else np.empty((M, K), dtype=np.float32)
    lib().oracle_spmm_csr_f32(M, K, row_ptr.ctypes.data, col_idx.ctypes.data, vals.ctypes.data,
                              B.ctypes.data, C.ctypes.data)
    return C


def spmm_f64(row_ptr, col_idx, vals, B):
    """Returns (C in fp64, sum of |terms| per element)."""
    row_ptr, col_idx, vals, B = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(vals, np.float32), _c(B, np.float32)
    M, K = len(row_ptr) - 1, B.shape[1]
    C = np.empty((M, K), dtype=np.float64)
    A = np.empty((M, K), dtype=np.float64)
    lib().oracle_spmm_csr_f64(M, K, row_ptr.ctypes.data, col_idx.ctypes.data, vals.ctypes.data,
                              B.ctypes.data, C.ctypes.data, A.ctypes.data)
    return C, A


def spmm_coo_f32(M, row_idx, col_idx, vals, B):
    row_idx, col_idx, vals, B = _c(row_idx, np.int32), _c(col_idx, np.int32), _c(vals, np.float32), _c(B, np.float32)
    K = B.shape[1]
    C = np.zeros((M, K), dtype=np.float32)
    lib().oracle_spmm_coo_f32(K, len(vals), row_idx.ctypes.data, col_idx.ctypes.data,
                              vals.ctypes.data, B.ctypes.data, C.ctypes.data)
    return C


def sddmm_f32(row_ptr, col_idx, X, Y):
    row_ptr, col_idx, X, Y = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(X, np.float32), _c(Y, np.float32)
    M, K = len(row_ptr) - 1, X.shape[1]
    out = np.empty(len(col_idx), dtype=np.float32)
    lib().oracle_sddmm_csr_f32(M, K, row_ptr.ctypes.data, col_idx.ctypes.data, X.ctypes.data,
                               Y.ctypes.data, out.ctypes.data)
    return out


def sddmm_f64(row_ptr, col_idx, X, Y):
    row_ptr, col_idx, X, Y = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(X, np.float32), _c(Y, np.float32)
    M, K = len(row_ptr) - 1, X.shape[1]
    out = np.empty(len(col_idx), dtype=np.float64)
    a = np.empty(len(col_idx), dtype=np.float64)
    lib().oracle_sddmm_csr_f64(M, K, row_ptr.ctypes.data, col_idx.ctypes.data, X.ctypes.data,
                               Y.ctypes.data, out.ctypes.data, a.ctypes.data)
    return out, a


def csr_transpose(M, N, row_ptr, col_idx, vals):
    row_ptr, col_idx, vals = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(vals, np.float32)
    nnz = len(col_idx)
    rpt = np.empty(N + 1, dtype=np.int32)
    cit = np.empty(nnz, dtype=np.int32)
    vt = np.empty(nnz, dtype=np.float32)
    perm = np.empty(nnz, dtype=np.int32)
    lib().oracle_csr_transpose(M, N, row_ptr.ctypes.data, col_idx.ctypes.data, vals.ctypes.data,
                               rpt.ctypes.data, cit.ctypes.data, vt.ctypes.data, perm.ctypes.data)
    return rpt, cit, vt, perm


def csr_to_coo_padded(row_ptr, col_idx, vals, padding):
    row_ptr, col_idx, vals = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(vals, np.float32)
    M, nnz = len(row_ptr) - 1, len(col_idx)
    padded = nnz if padding <= 0 or nnz % padding == 0 else nnz + padding - nnz % padding
    r = np.empty(padded, dtype=np.int32)
    c = np.empty(padded, dtype=np.int32)
    v = np.empty(padded, dtype=np.float32)
    got = lib().oracle_csr_to_coo_padded(M, row_ptr.ctypes.data, col_idx.ctypes.data,
                                         vals.ctypes.data, padding, r.ctypes.data, c.ctypes.data,
                                         v.ctypes.data)
    assert got == padded
    return r, c, v


def csr_to_coo_reordered(row_ptr, col_idx, vals, row_order, padding):
    row_ptr, col_idx, vals = _c(row_ptr, np.int32), _c(col_idx, np.int32), _c(vals, np.float32)
    row_order = _c(row_order, np.int32)
    M, nnz = len(row_ptr) - 1, len(col_idx)
    padded = nnz if padding <= 0 or nnz % padding == 0 else nnz + padding - nnz % padding
    r = np.empty(padded, dtype=np.int32)
    c = np.empty(padded, dtype=np.int32)
    v = np.empty(padded, dtype=np.float32)
    lib().oracle_csr_to_coo_reordered(M, row_ptr.ctypes.data, col_idx.ctypes.data, vals.ctypes.data,
                                      row_order.ctypes.data, padding, r.ctypes.data, c.ctypes.data,
                                      v.ctypes.data)
    return r, c, v


def shard_bounds(row_ptr, G):
    row_ptr = _c(row_ptr, np.int32)
    out = np.empty(G + 1, dtype=np.int64)
    lib().oracle_shard_bounds(len(row_ptr) - 1, row_ptr.ctypes.data, G, out.ctypes.data)
    return out


def row_length_cv(row_ptr):
    row_ptr = _c(row_ptr, np.int32)
    return lib().oracle_row_length_cv(len(row_ptr) - 1, row_ptr.ctypes.data)


def gflops(nnz, K, ms):
    return lib().oracle_gflops(nnz, K, ms)


def max_abs_err(got, want, div_by_launches=False):
    got, want = _c(got, np.float32), _c(want, np.float32)
    return lib().oracle_max_abs_err(got.size, got.ctypes.data, want.ctypes.data, int(div_by_launches))
