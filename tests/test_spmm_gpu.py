"""Parity of the CUDA CSR SpMM with the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

from helpers import check_against_f64, csr_from_rows, gpu_spmm, random_csr

pytestmark = pytest.mark.gpu


def _check(ctx, pkg, oracle, row_ptr, col_idx, vals, B, what, **kw):
    C = gpu_spmm(ctx, pkg, row_ptr, col_idx, vals, B, **kw)
    ref, abs_sum = oracle.spmm_f64(row_ptr, col_idx, vals, B)
    errs = check_against_f64(C, ref, abs_sum, what)
    return C, errs


def test_cfg1_small_csr(gpu_ctx, pkg, oracle):
    """Small uniform-degree configuration: M=N=4096, degree U{1..32}, K=32, values and B in U(-1,1)."""
    g = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1)
    B = pkg.host_fill_uniform(4096 * 32, 1, 10, -1.0, 1.0).reshape(4096, 32)
    C, _ = _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "cfg1")
    ref32 = oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)
    # the reference checker's own criterion (max abs error < 0.1) holds with a wide margin
    assert oracle.max_abs_err(C, ref32) < 1e-5
    # the row-split algorithm sums every row in CSR order with FMAs: the fp32 oracle bit for bit
    C2 = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B,
                  opts=pkg.Opts(algo=pkg.ALGO_ROW_SPLIT))
    assert np.array_equal(C2, ref32)


@pytest.mark.parametrize("K", [32, 64, 128])
@pytest.mark.parametrize("use_plan", [False, True])
def test_power_law_heavy_rows(gpu_ctx, pkg, oracle, K, use_plan):
    g = pkg.gen_rmat(14, 16, seed=2)
    N = g["N"]
    B = pkg.host_fill_uniform(N * K, 2, 10 + K, -1.0, 1.0).reshape(N, K)
    deg = np.diff(g["row_ptr"])
    assert deg.max() > 1000 and (deg == 0).sum() > 100   # heavy rows and empty rows both present
    C, _ = _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "rmat14 K=%d" % K,
                  use_plan=use_plan)
    if K == 128:
        # one lane group per warp: rows that fit in one chunk are summed in CSR order with
        # FMAs, so they are bit-exact against the fp32 oracle
        ref32 = oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)
        short = deg <= 128
        assert np.array_equal(C[short], ref32[short])


@pytest.mark.parametrize("K", [1, 3, 4, 7, 20, 33, 100, 160, 256, 516, 1000])
def test_generic_widths(gpu_ctx, pkg, oracle, K):
    rng = np.random.default_rng(K)
    deg = rng.integers(0, 50, size=700)
    deg[13] = 900
    row_ptr, col_idx, vals = random_csr(700, 1000, deg, seed=K)
    B = rng.uniform(-1, 1, size=(1000, K)).astype(np.float32)
    _check(gpu_ctx, pkg, oracle, row_ptr, col_idx, vals, B, "generic K=%d" % K)


@pytest.mark.parametrize("K", [32, 64, 128, 48])
def test_edge_structures(gpu_ctx, pkg, oracle, K):
    rng = np.random.default_rng(5)
    N = 513
    B = rng.uniform(-1, 1, size=(N, K)).astype(np.float32)
    cases = {
        "all rows empty": [[] for _ in range(300)],
        "single entry": [[7]],
        "single row with every entry": [list(range(N))],
        "empty rows first and last": [[]] * 70 + [[1, 2, 3], [], [5]] + [[]] * 90,
        "one heavy row between empties": [[]] * 40 + [list(range(0, N))] + [[]] * 40 + [[3]],
        "two heavy rows back to back": [list(range(N)), list(range(1, N)), [0]],
        "rows of length 127,128,129": [list(range(127)), list(range(128)), list(range(129)),
                                        list(range(255)), list(range(256)), list(range(257))],
        "dense-ish": [list(range(0, N, 2)) for _ in range(37)],
    }
    for name, rows in cases.items():
        row_ptr, col_idx, vals = csr_from_rows(rows, N, rng)
        _check(gpu_ctx, pkg, oracle, row_ptr, col_idx, vals, B, name + " K=%d" % K)
        _check(gpu_ctx, pkg, oracle, row_ptr, col_idx, vals, B, name + " plan K=%d" % K, use_plan=True)


def test_nnz_not_multiple_of_32_and_ragged_m(gpu_ctx, pkg, oracle):
    for M, seed in ((1, 1), (3, 2), (257, 3), (1023, 4)):
        rng = np.random.default_rng(seed)
        deg = rng.integers(0, 9, size=M)
        row_ptr, col_idx, vals = random_csr(M, 300, deg, seed)
        B = rng.uniform(-1, 1, size=(300, 64)).astype(np.float32)
        _check(gpu_ctx, pkg, oracle, row_ptr, col_idx, vals, B, "ragged M=%d" % M)


@pytest.mark.parametrize("chunk", [32, 64, 512, 4096])
def test_chunk_size_option(gpu_ctx, pkg, oracle, chunk):
    g = pkg.gen_rmat(12, 16, seed=9)
    B = pkg.host_fill_uniform(g["N"] * 64, 9, 1, -1.0, 1.0).reshape(g["N"], 64)
    opts = pkg.Opts(algo=pkg.ALGO_BALANCED, chunk_nnz=chunk)
    _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "chunk %d" % chunk, opts=opts)
    _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "chunk %d plan" % chunk,
           opts=opts, use_plan=True)


@pytest.mark.parametrize("K", [32, 64, 128, 24])
def test_row_split_algorithm_is_bit_exact(gpu_ctx, pkg, oracle, K):
    """The GESpMM-shaped kernel sums every row in CSR order: identical bits to the fp32 oracle."""
    g = pkg.gen_rmat(12, 16, seed=3)
    B = pkg.host_fill_uniform(g["N"] * K, 3, K, -1.0, 1.0).reshape(g["N"], K)
    opts = pkg.Opts(algo=pkg.ALGO_ROW_SPLIT)
    C = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, opts=opts)
    assert np.array_equal(C, oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B))


def test_run_to_run_determinism(gpu_ctx, pkg):
    g = pkg.gen_rmat(14, 16, seed=6)
    B = pkg.host_fill_uniform(g["N"] * 128, 6, 1, -1.0, 1.0).reshape(g["N"], 128)
    first = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B)
    for _ in range(3):
        assert np.array_equal(first, gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B))
    # the order in which chunks are scheduled (by cost; with col_idx also by column band) never changes a bit
    assert np.array_equal(first, gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, use_plan=True))
    assert np.array_equal(first, gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B, use_plan=True,
                                          plan_cols=False))


def test_overwrites_stale_output_and_linearity(gpu_ctx, pkg, oracle):
    g = pkg.gen_uniform_degree(2000, 2000, 0, 20, seed=8)
    rng = np.random.default_rng(8)
    B1 = rng.uniform(-1, 1, size=(2000, 64)).astype(np.float32)
    ones = np.ones((2000, 64), dtype=np.float32)
    C1 = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], ones)
    rowsum = np.add.reduceat(np.concatenate([g["vals"].astype(np.float64), [0.0]]),
                             np.minimum(g["row_ptr"][:-1], g["nnz"]))
    rowsum[np.diff(g["row_ptr"]) == 0] = 0
    assert np.allclose(C1, rowsum[:, None], rtol=1e-5, atol=1e-5)       # A * ones = row sums
    C2 = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B1)
    C3 = gpu_spmm(gpu_ctx, pkg, g["row_ptr"], g["col_idx"], g["vals"], B1 + ones)
    assert np.allclose(C3, C1 + C2, rtol=1e-4, atol=1e-4)              # linear in B


@pytest.mark.parametrize("K", [32, 64, 128])
def test_full_size_cfg2(gpu_ctx, pkg, oracle, K):
    """The power-law benchmark graph (R-MAT scale 20) at full size with a plan -- the kernel instantiations and
    chunk sizes the benchmark times -- against the oracle, every element."""
    g = pkg.gen_rmat(20, 16, seed=2)
    B = pkg.host_fill_uniform(g["N"] * K, 2, 100 + K, -1.0, 1.0).reshape(g["N"], K)
    C, errs = _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "cfg2 K=%d" % K,
                     use_plan=True)
    deg = np.diff(g["row_ptr"])
    assert np.all(C[deg == 0] == 0)


def test_host_entry_with_several_products(gpu_ctx, pkg, oracle):
    """hpspmm_spmm_csr_f32_host_multi: A uploaded once, the slabs of all products through one pipeline."""
    g = pkg.gen_rmat(12, 16, seed=6)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    Ks = [32, 64, 128, 40, 96]
    Bs = [pkg.host_fill_uniform(N * K, 6, K, -1.0, 1.0).reshape(N, K) for K in Ks]
    Cs = [np.full((M, K), np.nan, dtype=np.float32) for K in Ks]
    gpu_ctx.spmm_csr_host_multi(M, N, nnz, g["row_ptr"], g["col_idx"], g["vals"], Ks, Bs, Cs)
    for K, B, C in zip(Ks, Bs, Cs):
        ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
        check_against_f64(C, ref, abs_sum, "host multi K=%d" % K)
    # no products, and an empty matrix, are fine; a bad width is refused
    gpu_ctx.spmm_csr_host_multi(M, N, nnz, g["row_ptr"], g["col_idx"], g["vals"], [], [], [])
    with pytest.raises(pkg.HpspmmError) as e:
        gpu_ctx.spmm_csr_host_multi(M, N, nnz, g["row_ptr"], g["col_idx"], g["vals"], [0], [Bs[0]], [Cs[0]])
    assert e.value.status == pkg.ERR_INVALID


@pytest.mark.parametrize("K", [32, 64, 128, 192, 96, 40])
def test_host_buffer_entry_point(gpu_ctx, pkg, oracle, K):
    """K = 64 / 96 / 128 / 192 take the slab pipeline (32- or 64-column slabs), the others the plain path."""
    g = pkg.gen_rmat(12, 16, seed=4)
    B = pkg.host_fill_uniform(g["N"] * K, 4, 1, -1.0, 1.0).reshape(g["N"], K)
    C = np.full((g["M"], K), np.nan, dtype=np.float32)
    gpu_ctx.spmm_csr_host(g["M"], g["N"], K, g["nnz"], g["row_ptr"], g["col_idx"], g["vals"], B, C)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    check_against_f64(C, ref, abs_sum, "host entry")


def test_argument_errors_return_codes(gpu_ctx, pkg):
    lib = pkg.load_library()
    d = gpu_ctx.alloc((64,), np.float32)
    h = gpu_ctx.handle
    f = lib.hpspmm_spmm_csr_f32
    assert f(h, None, 4, 4, 0, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, None) == pkg.ERR_INVALID   # K = 0
    assert f(h, None, -1, 4, 32, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, None) == pkg.ERR_INVALID
    assert f(h, None, 4, 4, 32, 0, None, d.ptr, d.ptr, d.ptr, d.ptr, None, None) == pkg.ERR_INVALID  # null row_ptr
    assert f(h, None, 4, 4, 32, 8, d.ptr, d.ptr, d.ptr, d.ptr + 4, d.ptr, None, None) == pkg.ERR_INVALID  # misaligned B
    assert f(h, None, 1 << 40, 4, 32, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, None) == pkg.ERR_UNSUPPORTED
    assert f(None, None, 4, 4, 32, 0, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, None) == pkg.ERR_INVALID
    assert b"invalid" in lib.hpspmm_last_error(h) or b"sizes" in lib.hpspmm_last_error(h)
    bad_algo = pkg.Opts(algo=99)
    rp = gpu_ctx.upload(np.zeros(5, dtype=np.int32))
    import ctypes
    assert f(h, None, 4, 4, 32, 0, rp.ptr, d.ptr, d.ptr, d.ptr, d.ptr, ctypes.byref(bad_algo), None) == pkg.ERR_INVALID
    d.free()
    rp.free()


def test_fill_factories_match_host(gpu_ctx, pkg):
    n = 100_003
    d = gpu_ctx.alloc((n,), np.float32)
    gpu_ctx.fill_uniform(d, n, 42, 7, -1.0, 1.0)
    assert np.array_equal(d.to_host(), pkg.host_fill_uniform(n, 42, 7, -1.0, 1.0))   # bit exact
    gpu_ctx.fill_uniform(d, n, 42, 8, 0.0, 1.0)
    assert np.array_equal(d.to_host(), pkg.host_fill_uniform(n, 42, 8, 0.0, 1.0))
    gpu_ctx.fill(d, n, 2.5)
    assert np.all(d.to_host() == 2.5)
    d.free()


@pytest.mark.parametrize("with_cols", [False, True])
def test_plan_tables_tile_the_matrix_and_schedule_every_chunk_once(gpu_ctx, pkg, with_cols):
    ctx = gpu_ctx
    g = pkg.gen_rmat(13, 16, seed=12)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    d_rp, d_ci = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"])
    plan = ctx.plan_create(M, nnz, d_rp, 32, N=N, col_idx=d_ci if with_cols else None)
    n = ctx.plan_info(plan)["n_chunks"]
    p_start, p_row, p_order = ctx.plan_tables(plan)

    def read(ptr, count):
        out = np.empty(count, dtype=np.int32)
        ctx.memcpy_d2h(out, ptr)
        ctx.stream_sync()
        return out

    start, row, order = read(p_start, n + 1), read(p_row, n), read(p_order, n)
    assert start[0] == 0 and start[-1] == nnz and np.all(np.diff(start) >= 0)
    assert np.all(np.diff(start) <= 2 * 128)                       # nominal size 128; snapping moves a cut by < 128
    rp = g["row_ptr"]
    nonempty = np.diff(start) > 0
    assert np.all(rp[row[nonempty]] <= start[:-1][nonempty]) and np.all(start[:-1][nonempty] < rp[row[nonempty] + 1])
    assert np.array_equal(np.sort(order), np.arange(n, dtype=np.int32))
    # the list of rows that hold entries: exactly those rows, in order, with their ends and a sentinel
    p_id, p_end, p_ri = ctx.plan_row_list(plan)
    want_id = np.flatnonzero(np.diff(rp) > 0).astype(np.int32)
    n_nz = len(want_id)
    got_id, got_end, ri = read(p_id, n_nz + 1), read(p_end, n_nz + 1), read(p_ri, n)
    assert np.array_equal(got_id[:n_nz], want_id) and got_id[n_nz] == M
    assert np.array_equal(got_end[:n_nz], rp[want_id + 1]) and got_end[n_nz] == np.iinfo(np.int32).max
    assert np.array_equal(got_id[ri], row)
    ctx.plan_destroy(plan)
    d_rp.free()
    d_ci.free()


@pytest.mark.parametrize("K", [64, 128])
@pytest.mark.parametrize("chunk", [32, 256])
def test_split_rows_settled_inside_the_kernel_on_repeated_calls(gpu_ctx, pkg, oracle, K, chunk):
    """With a plan, K = 64/128 add the carries of split rows inside the product kernel, through per-row
    counters that must be back at zero after every launch: three calls on one plan, rows of 1 to 20,000
    entries (up to 625 pieces), each call checked."""
    ctx = gpu_ctx
    N = 30000
    degrees = [20000, 0, 1, 33, 5000, 31, 0, 12000, 2, 700, 64, 65, 0, 300] * 3
    rp, ci, v = random_csr(len(degrees), N, degrees, seed=51)
    M, nnz = len(degrees), len(ci)
    B = pkg.host_fill_uniform(N * K, 51, 1, -1.0, 1.0).reshape(N, K)
    ref, abs_sum = oracle.spmm_f64(rp, ci, v, B)
    d_rp, d_ci, d_v, d_B = ctx.upload(rp), ctx.upload(ci), ctx.upload(v), ctx.upload(B)
    d_C = ctx.alloc((M, K), np.float32)
    opts = pkg.Opts(algo=pkg.ALGO_BALANCED, chunk_nnz=chunk)
    plan = ctx.plan_create(M, nnz, d_rp, K, opts, N=N, col_idx=d_ci)
    first = None
    for call in range(3):
        ctx.fill(d_C, M * K, float(call))            # stale contents differ from call to call
        ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan, opts=opts)
        ctx.stream_sync()
        got = d_C.to_host()
        check_against_f64(got, ref, abs_sum, "settled in kernel, call %d" % call)
        if first is None:
            first = got
        assert np.array_equal(got, first)            # bit-reproducible from call to call
    # the same plan at a narrower width takes the separate fix-up kernel and leaves the counters alone
    B32 = np.ascontiguousarray(B[:, :32])
    d_B32, d_C32 = ctx.upload(B32), ctx.alloc((M, 32), np.float32)
    ctx.spmm_csr(M, N, 32, nnz, d_rp, d_ci, d_v, d_B32, d_C32, plan=plan, opts=opts)
    r32, a32 = oracle.spmm_f64(rp, ci, v, B32)
    check_against_f64(d_C32.to_host(), r32, a32, "same plan, K = 32")
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C, plan=plan, opts=opts)
    assert np.array_equal(d_C.to_host(), first)
    ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_v, d_B, d_C, d_B32, d_C32):
        b.free()


def _structured_degree_lists(S):
    """Row-length patterns around the nominal chunk size S: rows that end or start exactly on a cut, rows one
    longer or shorter than a chunk, heavy rows first, last, adjacent, and separated by empty rows."""
    yield [S, S + 1, 2 * S, 2 * S - 1, 0, S - 1, 1, 3 * S + 5, 0, 0, S]
    yield [S + 1]
    yield [5 * S]
    yield [1, 5 * S]
    yield [S - 1, S + 1, S - 1, S + 1]
    yield [3 * S, 3 * S, 3 * S]
    yield [0, 0, 4 * S + 1, 0, 0, 7, 0]
    yield [S // 2] * 9 + [2 * S + S // 2] + [S // 2] * 3
    yield [1] * (2 * S) + [10 * S + 3] + [2] * S
    yield [S - 1, 1, S, S, 1, S - 1, 2 * S, 1]
    yield [40 * S + 17, 3, 33 * S, 0, 35 * S - 1]      # runs longer than 32 carries


@pytest.mark.parametrize("K", [32, 64, 128, 24])
@pytest.mark.parametrize("chunk", [32, 128])
def test_rows_around_the_chunk_size(gpu_ctx, pkg, oracle, K, chunk):
    N = 20000
    for case, degrees in enumerate(_structured_degree_lists(chunk)):
        rp, ci, v = random_csr(len(degrees), N, degrees, seed=60 + case)
        B = pkg.host_fill_uniform(N * K, 60 + case, 1, -1.0, 1.0).reshape(N, K)
        opts = pkg.Opts(algo=pkg.ALGO_BALANCED, chunk_nnz=chunk)
        for use_plan in (False, True):
            _check(gpu_ctx, pkg, oracle, rp, ci, v, B, "S=%d case %d plan=%s K=%d" % (chunk, case, use_plan, K),
                   opts=opts, use_plan=use_plan)


def test_products_with_a_plan_can_be_captured_in_a_cuda_graph(pkg, oracle):
    """With a plan a product only enqueues kernels (no allocation, no synchronisation), so a training step's
    products can be recorded once into a CUDA graph and replayed; the carry counters return to zero by themselves."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    ctx = pkg.Context(0)
    g = pkg.gen_rmat(13, 16, seed=71)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    rp, ci, v = (torch.from_numpy(g[k]).to(dev) for k in ("row_ptr", "col_idx", "vals"))
    Ks = (32, 64, 128)
    Bh = {K: pkg.host_fill_uniform(N * K, 71, K, -1.0, 1.0).reshape(N, K) for K in Ks}
    B = {K: torch.from_numpy(Bh[K]).to(dev) for K in Ks}
    C = {K: torch.full((M, K), 7.0, dtype=torch.float32, device=dev) for K in Ks}
    plans = {K: ctx.plan_create(M, nnz, rp.data_ptr(), K, N=N, col_idx=ci.data_ptr()) for K in Ks}
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for K in Ks:   # warm-up outside the capture
            ctx.spmm_csr(M, N, K, nnz, rp.data_ptr(), ci.data_ptr(), v.data_ptr(), B[K].data_ptr(), C[K].data_ptr(),
                         plan=plans[K], stream=side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            s = torch.cuda.current_stream(dev).cuda_stream
            for K in Ks:
                ctx.spmm_csr(M, N, K, nnz, rp.data_ptr(), ci.data_ptr(), v.data_ptr(), B[K].data_ptr(),
                             C[K].data_ptr(), plan=plans[K], stream=s)
    first = None
    for replay in range(3):
        for K in Ks:
            C[K].fill_(float(replay))
        graph.replay()
        torch.cuda.synchronize(dev)
        got = {K: C[K].cpu().numpy() for K in Ks}
        for K in Ks:
            ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], Bh[K])
            check_against_f64(got[K], ref, abs_sum, "graph replay %d K=%d" % (replay, K))
        if first is None:
            first = got
        assert all(np.array_equal(got[K], first[K]) for K in Ks)
    del graph
    for K in Ks:
        ctx.plan_destroy(plans[K])
    ctx.close()


@pytest.mark.parametrize("K", [96, 160, 192, 224, 256, 320, 512])
@pytest.mark.parametrize("use_plan", [False, True])
def test_other_multiples_of_32_run_as_column_slabs(gpu_ctx, pkg, oracle, K, use_plan):
    """K = 32·m beyond 32/64/128 runs the specialised kernel over column slabs of 128, 64 and 32 (strided B, C and
    carry slots); heavy rows make every slab hand on and settle carries; canaries guard the neighbouring columns."""
    g = pkg.gen_rmat(12, 16, seed=81)
    N = g["N"]
    B = pkg.host_fill_uniform(N * K, 81, K, -1.0, 1.0).reshape(N, K)
    for chunk in (0, 32):
        opts = pkg.Opts(algo=pkg.ALGO_BALANCED, chunk_nnz=chunk)
        C, _ = _check(gpu_ctx, pkg, oracle, g["row_ptr"], g["col_idx"], g["vals"], B, "slabs K=%d S=%d" % (K, chunk),
                      opts=opts, use_plan=use_plan)
        # a slab is the product with that slab of B: columns 0..31 equal the K = 32 product bit for bit when the
        # first slab is 32 wide... not in general (slab widths differ), but every slab must agree with the oracle
        assert np.all(np.isfinite(C))
