"""The allocation-free SpMM entry point against the ordinary one (needs a B200).

hpspmm_spmm_csr_f32_static_scratch serves callers that may not allocate device memory at
call time (a plugin's enqueue hook, a process whose allocator already owns the device): it
keeps the kernel's chunk table and carry slots in a fixed array inside the library.  The
file name sorts last so that a run stopping at the first failure has already run the rest.
"""
import ctypes

import numpy as np
import pytest

from helpers import check_against_f64, guarded_output

pytestmark = pytest.mark.gpu


def _static_call(pkg, M, N, K, nnz, d_rp, d_ci, d_v, d_B, c_ptr):
    lib = pkg.load_library()
    err = ctypes.create_string_buffer(512)
    st = lib.hpspmm_spmm_csr_f32_static_scratch(0, M, N, K, nnz, d_rp.ptr, d_ci.ptr, d_v.ptr, d_B.ptr,
                                                c_ptr, None, err, len(err))
    return st, err.value.decode()


@pytest.mark.parametrize("K", [32, 128, 20, 96])
def test_static_scratch_matches_ordinary_entry_twice(gpu_ctx, pkg, oracle, K):
    ctx = gpu_ctx
    g = pkg.gen_rmat(13, 16, seed=12)          # heavy rows: the carry slots are exercised
    M, N, nnz = g["M"], g["N"], g["nnz"]
    assert np.diff(g["row_ptr"]).max() > 1000
    B = pkg.host_fill_uniform(N * K, 12, K, -1.0, 1.0).reshape(N, K)
    d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
    buf_a, ptr_a, read_a = guarded_output(ctx, (M, K))
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, ptr_a)
    ctx.stream_sync()
    want = read_a()
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    for call in range(2):                       # two calls in a row share the static array
        buf_b, ptr_b, read_b = guarded_output(ctx, (M, K))
        st, msg = _static_call(pkg, M, N, K, nnz, d_rp, d_ci, d_v, d_B, ptr_b)
        assert st == pkg.OK, msg
        ctx.stream_sync()
        got = read_b()
        check_against_f64(got, ref, abs_sum, "static scratch call %d K=%d" % (call, K))
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
        assert np.array_equal(got, want)        # same chunking, same order of additions
        buf_b.free()
    # a smaller product afterwards must not see leftovers of the larger one
    h = pkg.gen_uniform_degree(300, N, 0, 40, seed=13)
    d_rp2, d_ci2, d_v2 = ctx.upload(h["row_ptr"]), ctx.upload(h["col_idx"]), ctx.upload(h["vals"])
    buf_c, ptr_c, read_c = guarded_output(ctx, (h["M"], K))
    st, msg = _static_call(pkg, h["M"], N, K, h["nnz"], d_rp2, d_ci2, d_v2, d_B, ptr_c)
    assert st == pkg.OK, msg
    ctx.stream_sync()
    ref2, abs2 = oracle.spmm_f64(h["row_ptr"], h["col_idx"], h["vals"], B)
    check_against_f64(read_c(), ref2, abs2, "static scratch after a larger call")
    for b in (d_rp, d_ci, d_v, d_B, buf_a, d_rp2, d_ci2, d_v2, buf_c):
        b.free()


def test_static_scratch_rejects_oversized_matrices(gpu_ctx, pkg):
    ctx = gpu_ctx
    d = ctx.alloc((64,), np.float32)
    lib = pkg.load_library()
    err = ctypes.create_string_buffer(512)
    # 2^27 nnz at K = 128 would need ~0.5 GB of scratch: refused before anything is launched
    st = lib.hpspmm_spmm_csr_f32_static_scratch(0, 1 << 20, 1 << 20, 128, 1 << 27, d.ptr, d.ptr, d.ptr,
                                                d.ptr, d.ptr, None, err, len(err))
    assert st == pkg.ERR_UNSUPPORTED
    assert b"too large for the static scratch" in err.value
    st = lib.hpspmm_spmm_csr_f32_static_scratch(0, 4, 4, 0, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None,
                                                err, len(err))
    assert st == pkg.ERR_INVALID and err.value
    # a device the process does not have is refused by name, even for an empty matrix, and launches nothing
    for M in (4, 0):
        st = lib.hpspmm_spmm_csr_f32_static_scratch(63, M, 4, 32, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None,
                                                    err, len(err))
        assert st == pkg.ERR_INVALID and b"does not exist" in err.value
    st = lib.hpspmm_spmm_csr_f32_static_scratch(64, 4, 4, 32, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None,
                                                err, len(err))
    assert st == pkg.ERR_INVALID and b"out of range" in err.value
    d.free()
