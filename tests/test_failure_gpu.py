"""Allocation failures, injected on the host: every entry point that allocates returns HPSPMM_ERR_OOM,
gives back what it had taken and leaves the context usable.  Nothing here faults, traps or hangs a GPU:
hpspmm_debug_fail_device_alloc makes the chosen allocation report out-of-memory before the device is
touched.  (The reference ignores the result of cudaMalloc, spmm/starml/basic/allocator_cuda.cpp:5-13.)"""
import numpy as np
import pytest

from helpers import check_against_f64

pytestmark = pytest.mark.gpu


@pytest.fixture
def seam(pkg):
    lib = pkg.load_library()

    def arm(nth, count=1):
        return lib.hpspmm_debug_fail_device_alloc(nth, count)

    yield arm
    lib.hpspmm_debug_fail_device_alloc(0, 0)


def _free_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info(0)[0]


def _graph(pkg):
    g = pkg.gen_rmat(12, 16, seed=51)
    B = pkg.host_fill_uniform(g["N"] * 64, 51, 1, -1.0, 1.0).reshape(g["N"], 64)
    return g, B


def test_plan_create_reports_oom_and_recovers(pkg, oracle, seam):
    g, B = _graph(pkg)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    with pkg.Context(0) as ctx:
        d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
        d_C = ctx.alloc((M, 64), np.float32)
        before = _free_bytes()
        seam(1)
        with pytest.raises(pkg.HpspmmError) as e:
            ctx.plan_create(M, nnz, d_rp, 64, N=N, col_idx=d_ci)
        assert e.value.status == pkg.ERR_OOM
        assert _free_bytes() == before                      # nothing kept
        plan = ctx.plan_create(M, nnz, d_rp, 64, N=N, col_idx=d_ci)   # the seam fired once; the context still works
        ctx.spmm_csr(M, N, 64, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan)
        ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
        check_against_f64(d_C.to_host(), ref, abs_sum, "after an injected allocation failure")
        ctx.plan_destroy(plan)


def test_planless_and_host_products_report_oom_and_recover(pkg, oracle, seam):
    g, B = _graph(pkg)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    with pkg.Context(0) as ctx:                              # a fresh context owns no scratch yet
        d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
        d_C = ctx.alloc((M, 64), np.float32)
        seam(1)                                              # the scratch is asked for a second, smaller time ...
        ctx.spmm_csr(M, N, 64, nnz, d_rp, d_ci, d_v, d_B, d_C)
        check_against_f64(d_C.to_host(), ref, abs_sum, "plan-less product, second allocation attempt")
    with pkg.Context(0) as ctx:
        d_rp, d_ci, d_v, d_B = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"]), ctx.upload(B)
        d_C = ctx.alloc((M, 64), np.float32)
        seam(1, 2)                                           # ... and when that fails too, the call reports it
        with pytest.raises(pkg.HpspmmError) as e:
            ctx.spmm_csr(M, N, 64, nnz, d_rp, d_ci, d_v, d_B, d_C)
        assert e.value.status == pkg.ERR_OOM
        ctx.spmm_csr(M, N, 64, nnz, d_rp, d_ci, d_v, d_B, d_C)
        check_against_f64(d_C.to_host(), ref, abs_sum, "plan-less product after an injected failure")
    with pkg.Context(0) as ctx:                              # host entry: the staging buffer is the first allocation
        C = np.zeros((M, 64), np.float32)
        seam(1)
        with pytest.raises(pkg.HpspmmError) as e:
            ctx.spmm_csr_host(M, N, 64, nnz, g["row_ptr"], g["col_idx"], g["vals"], B, C)
        assert e.value.status == pkg.ERR_OOM
        seam(2, 2)                                           # ... and the kernel scratch the second (two attempts)
        with pytest.raises(pkg.HpspmmError) as e:
            ctx.spmm_csr_host(M, N, 64, nnz, g["row_ptr"], g["col_idx"], g["vals"], B, C)
        assert e.value.status == pkg.ERR_OOM
        ctx.spmm_csr_host(M, N, 64, nnz, g["row_ptr"], g["col_idx"], g["vals"], B, C)
        check_against_f64(C, ref, abs_sum, "host product after injected failures")


@pytest.mark.parametrize("nth", [1, 2, 3, 4, 5])
def test_layer_create_gives_everything_back(pkg, seam, nth):
    g, _ = _graph(pkg)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    with pkg.Context(0) as ctx:
        d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
        layer = pkg.Layer(ctx, M, N, nnz, d_rp, d_ci, d_v, 64)     # sizes the context's scratch once
        layer.close()
        before = _free_bytes()
        seam(nth)
        with pytest.raises(pkg.HpspmmError) as e:
            pkg.Layer(ctx, M, N, nnz, d_rp, d_ci, d_v, 64)
        assert e.value.status == pkg.ERR_OOM
        assert _free_bytes() == before
        layer = pkg.Layer(ctx, M, N, nnz, d_rp, d_ci, d_v, 64)
        layer.close()


def test_shard_plan_create_reports_oom(pkg, seam):
    g, _ = _graph(pkg)
    bounds = pkg.shard_bounds(g["row_ptr"], 1)
    with pkg.Context(0) as ctx:
        before = _free_bytes()
        seam(1)
        with pytest.raises(pkg.HpspmmError) as e:
            pkg.ShardedSpmm(ctx, 1, 0, None, g["M"], g["N"], g["row_ptr"], g["col_idx"], bounds, 64)
        assert e.value.status == pkg.ERR_OOM
        assert _free_bytes() == before
        sp = pkg.ShardedSpmm(ctx, 1, 0, None, g["M"], g["N"], g["row_ptr"], g["col_idx"], bounds, 64)
        sp.close()


def test_seam_argument_and_disarm(pkg, seam):
    assert seam(-1) == pkg.ERR_INVALID and seam(1, -1) == pkg.ERR_INVALID
    assert seam(3) == pkg.OK and seam(0, 0) == pkg.OK
    with pkg.Context(0) as ctx:                              # disarmed: allocations go through
        d = ctx.alloc((1024,), np.float32)
        ctx.fill(d, 1024, 2.0)
        assert np.all(d.to_host() == 2.0)
