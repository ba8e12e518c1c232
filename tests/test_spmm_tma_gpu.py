"""HPSPMM_ALGO_TMA (needs a B200): the K = 128 product with the rows of B fetched by TMA gather4 into shared
memory.  It keeps the chunking and the order of additions of the default kernel, so its output must equal the
default's bit for bit, on top of meeting the FP64 oracle; its bounded waits must never have run out."""
import numpy as np
import pytest

from helpers import check_against_f64, random_csr
from test_spmm_gpu import _structured_degree_lists

pytestmark = pytest.mark.gpu


def _both(ctx, pkg, oracle, rp, ci, v, B, chunk, what, calls=1):
    M, N, K, nnz = len(rp) - 1, B.shape[0], B.shape[1], len(ci)
    d_rp, d_ci, d_v, d_B = ctx.upload(rp), ctx.upload(ci), ctx.upload(v), ctx.upload(B)
    d_C = ctx.alloc((M, K), np.float32)
    plan = ctx.plan_create(M, nnz, d_rp, K, pkg.Opts(algo=pkg.ALGO_BALANCED, chunk_nnz=chunk), N=N, col_idx=d_ci)
    out = {}
    for algo in (pkg.ALGO_BALANCED, pkg.ALGO_TMA):
        opts = pkg.Opts(algo=algo, chunk_nnz=chunk)
        for call in range(calls):
            ctx.fill(d_C, M * K, -3.0 - call)
            ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan, opts=opts)
            ctx.stream_sync()
            got = d_C.to_host()
            if call:
                assert np.array_equal(got, out[algo]), what + ": call %d differs" % call
            out[algo] = got
    ref, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    check_against_f64(out[pkg.ALGO_TMA], ref, abs_sum, what)
    assert np.array_equal(out[pkg.ALGO_TMA], out[pkg.ALGO_BALANCED]), what + ": TMA and default kernels differ"
    ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_v, d_B, d_C):
        b.free()


@pytest.mark.parametrize("chunk", [32, 128, 256])
def test_tma_kernel_equals_default_on_rows_around_the_chunk_size(gpu_ctx, pkg, oracle, chunk):
    N, K = 20000, 128
    for case, degrees in enumerate(_structured_degree_lists(chunk)):
        rp, ci, v = random_csr(len(degrees), N, degrees, seed=160 + case)
        B = pkg.host_fill_uniform(N * K, 160 + case, 1, -1.0, 1.0).reshape(N, K)
        _both(gpu_ctx, pkg, oracle, rp, ci, v, B, chunk, "S=%d case %d" % (chunk, case), calls=2)
    assert gpu_ctx.tma_fallbacks() == 0


def test_tma_kernel_on_a_power_law_graph(gpu_ctx, pkg, oracle):
    g = pkg.gen_rmat(14, 16, seed=21)
    assert np.diff(g["row_ptr"]).max() > 1000
    B = pkg.host_fill_uniform(g["N"] * 128, 21, 1, -1.0, 1.0).reshape(g["N"], 128)
    _both(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, 0, "rmat14", calls=3)
    assert gpu_ctx.tma_fallbacks() == 0


def test_tma_kernel_never_uses_the_rows_it_fetches_as_padding(gpu_ctx, pkg, oracle):
    """A chunk whose length is not a multiple of four is padded with fetches of row 0 of B; those must not
    reach the sums, whatever row 0 holds."""
    N, K = 5000, 128
    degrees = [7, 0, 1, 2, 301, 3, 0, 5, 66, 1]
    rp, ci, v = random_csr(len(degrees), N, degrees, seed=170)
    ci = np.where(ci == 0, 1, ci).astype(np.int32)             # nothing refers to column 0
    B = pkg.host_fill_uniform(N * K, 170, 1, -1.0, 1.0).reshape(N, K).copy()
    B[0, :64] = np.inf
    B[0, 64:] = np.nan
    M, nnz = len(degrees), len(ci)
    ctx = gpu_ctx
    d_rp, d_ci, d_v, d_B = ctx.upload(rp), ctx.upload(ci), ctx.upload(v), ctx.upload(B)
    d_C = ctx.alloc((M, K), np.float32)
    for chunk in (32, 256):
        plan = ctx.plan_create(M, nnz, d_rp, K, pkg.Opts(chunk_nnz=chunk), N=N, col_idx=d_ci)
        ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan, opts=pkg.Opts(algo=pkg.ALGO_TMA, chunk_nnz=chunk))
        ctx.stream_sync()
        got = d_C.to_host()
        assert np.isfinite(got).all()
        Bz = B.copy()
        Bz[0] = 0.0
        ref, abs_sum = oracle.spmm_f64(rp, ci, v, Bz)
        check_against_f64(got, ref, abs_sum, "padding S=%d" % chunk)
        ctx.plan_destroy(plan)
    assert ctx.tma_fallbacks() == 0
    for b in (d_rp, d_ci, d_v, d_B, d_C):
        b.free()


@pytest.mark.parametrize("K,chunk", [(64, 128), (128, 512), (32, 128)])
def test_calls_the_tma_path_cannot_take_run_as_the_default(gpu_ctx, pkg, oracle, K, chunk):
    """Other widths, and plans whose chunks exceed what the kernel stages, run the default kernel under
    HPSPMM_ALGO_TMA: same bits."""
    N = 9000
    degrees = [900, 0, 3, 1200, 17, 64, 2500, 1]
    rp, ci, v = random_csr(len(degrees), N, degrees, seed=180)
    B = pkg.host_fill_uniform(N * K, 180, 1, -1.0, 1.0).reshape(N, K)
    _both(gpu_ctx, pkg, oracle, rp, ci, v, B, chunk, "declined K=%d S=%d" % (K, chunk))
